/*
 * es_b200.h -- C ABI of the B200-native kernel layer for einsummable's
 * memgraph apply nodes (einsummable_t / touch_t kernels, fills, move_t copies).
 *
 * Plain pointers and sizes only; no C++ or torch types.  Every function returns
 * an es_status_t (0 = ok); es_b200_last_error() gives the text of the last
 * failure on the calling thread.  Nothing here traps or asserts on the device.
 *
 * All launches are asynchronous on the given stream; the caller observes
 * completion through the stream, exactly as the reference's exec nodes do
 * (src/engine/gpu/exec_graph.cc:318-332).  All device memory is owned by the
 * caller (src/engine/gpu/exec_graph.cc:295-312).
 *
 * Each declaration cites the reference interface it stands in for
 * (paths relative to the reference project).
 */
#ifndef ES_B200_H
#define ES_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ES_MAX_RANK 12
#define ES_MAX_INNS 8

typedef enum {
    ES_OK = 0,
    ES_NOT_SUPPORTED = 1,       /* kernel_manager_t::build returning nullopt */
    ES_BAD_DESCRIPTOR = 2,      /* malformed einsummable / touch / fill */
    ES_WORKSPACE_TOO_SMALL = 3, /* src/engine/gpu/gpu_kernel_manager.cc:1585-1587 */
    ES_CUDA_ERROR = 4,          /* src/engine/gpu/utility.cc:114-143 */
    ES_NOT_BUILT = 5,           /* src/engine/gpu/gpu_kernel_manager.cc:1257-1261 */
    ES_BAD_ARGUMENT = 6,
    ES_COMPILE_ERROR = 7
} es_status_t;

/* dtype_t order of src/einsummable/scalarop.h:10 */
typedef enum { ES_F16 = 0, ES_F32 = 1, ES_F64 = 2, ES_C64 = 3 } es_dtype_t;

/* castable_t order of src/einsummable/scalarop.h:4; -1 = no castable */
typedef enum {
    ES_CASTABLE_NONE = -1,
    ES_CASTABLE_ADD = 0,
    ES_CASTABLE_MUL = 1,
    ES_CASTABLE_MIN = 2,
    ES_CASTABLE_MAX = 3
} es_castable_t;

/* Policy for f32 contractions on the tensor cores. */
typedef enum {
    ES_F32_3XTF32 = 0, /* default: hi/lo split, 3 MMAs, ~fp32 accuracy */
    ES_F32_TF32 = 1    /* single TF32 MMA, ~1e-3 relative accuracy */
} es_f32_policy_t;

/*
 * einsummable_t (src/einsummable/einsummable.h:8-31) as a POD.
 * All tensors are dense row-major; input k has shape join_shape[inn_modes[k][*]];
 * the output is join modes 0..out_rank-1.  `join` is the scalarop in the
 * reference's text form (operator<<, src/einsummable/scalarop.cc:2878-3011),
 * e.g. "*[hole|f32@0,hole|f32@1]".
 */
typedef struct {
    int32_t     join_rank;
    uint64_t    join_shape[ES_MAX_RANK];
    int32_t     n_inn;
    int32_t     inn_rank[ES_MAX_INNS];
    int32_t     inn_modes[ES_MAX_INNS][ES_MAX_RANK];
    int32_t     out_rank;
    int32_t     castable; /* es_castable_t */
    const char* join;
} es_einsummable_desc_t;

/* touchdim_t (src/einsummable/touch.h:8-14) */
typedef struct {
    uint64_t d_inn, d_out, offset_inn, offset_out, size;
} es_touchdim_t;

/* One touch of a batched launch (see es_b200_launch_touch_batch). */
typedef struct {
    es_touchdim_t dims[4];
    int32_t       rank;
    int32_t       castable; /* es_castable_t */
    void*         out;
    const void*   inn;
} es_touch_item_t;

typedef struct es_b200 es_b200_t;

/* kernel_manager_t::kernel_manager_t(int device) / ~kernel_manager_t
 * (src/engine/gpu/gpu_kernel_manager.h:274-277, gpu_kernel_manager.cc:29-57). */
int es_b200_create(int device, es_b200_t** out);
int es_b200_destroy(es_b200_t* h);

/* Options on the handle; the reference has only compile-time switches here. */
int es_b200_set_f32_policy(es_b200_t* h, int policy /* es_f32_policy_t */);

/* kernel_manager_t::build(einsummable_t const&) -> optional<workspace_info_t>
 * (src/engine/gpu/gpu_kernel_manager.h:300, gpu_kernel_manager.cc:590-958).
 * Idempotent, keyed on the merged (merge_adjacent_dims) einsummable.
 * ES_NOT_SUPPORTED plays the role of nullopt. */
int es_b200_build_einsummable(es_b200_t*                   h,
                              const es_einsummable_desc_t* desc,
                              uint64_t*                    workspace_bytes,
                              uint64_t*                    kernel_id);

/* kernel_manager_t::workspace_size (src/engine/gpu/gpu_kernel_manager.h:302). */
int es_b200_workspace_size(es_b200_t* h, uint64_t kernel_id, uint64_t* workspace_bytes);

/* kernel_manager_t::operator()(einsummable_t const&, cudaStream_t, void* out,
 * vector<void const*> inns, optional<tuple<void*,uint64_t>> workspace)
 * (src/engine/gpu/gpu_kernel_manager.h:304-309, gpu_kernel_manager.cc:1000-1252).
 * stream is a cudaStream_t. */
int es_b200_launch_einsummable(es_b200_t*         h,
                               uint64_t           kernel_id,
                               void*              stream,
                               void*              out,
                               const void* const* inns,
                               int                n_inn,
                               void*              workspace,
                               uint64_t           workspace_bytes);

/* kernel_manager_t::operator()(touch_t const&, cudaStream_t, void* out, void const* inn)
 * (src/engine/gpu/gpu_kernel_manager.h:311, gpu_kernel_manager.cc:980-998;
 *  kernels: src/engine/gpu/cuda_kernels.cu:99-515).  Any rank >= 1 is accepted
 * (the touch is simplified first, src/einsummable/touch.cc:3-28; at most 4
 * dims may remain). */
int es_b200_launch_touch(es_b200_t*           h,
                         const es_touchdim_t* dims,
                         int                  rank,
                         int                  castable,
                         int                  dtype,
                         void*                stream,
                         void*                out,
                         const void*          inn);

/* Many touches of one dtype in a single launch.  Stands in for a run of
 * gpu_touch_t::launch calls (src/engine/gpu/exec_graph.cc:354-404) whose
 * destinations do not overlap; items are staged through a caller-provided
 * device buffer `items_dev` of n * sizeof(es_touch_item_t) bytes. */
int es_b200_launch_touch_batch(es_b200_t*             h,
                               const es_touch_item_t* items,
                               int                    n,
                               int                    dtype,
                               void*                  stream,
                               void*                  items_dev);

/* The same in two steps, for exec graphs whose touches are fixed: prepare once
 * (validates, lowers and copies the descriptors to items_dev on `stream`), then
 * launch any number of times with no per-touch host work. */
typedef struct {
    int32_t  n, dtype, width, pad;
    uint64_t max_slots;
    void*    items_dev;
} es_touch_batch_t;
int es_b200_prepare_touch_batch(es_b200_t*             h,
                                const es_touch_item_t* items,
                                int                    n,
                                int                    dtype,
                                void*                  stream,
                                void*                  items_dev,
                                es_touch_batch_t*      prepared);
int es_b200_launch_prepared_touch_batch(es_b200_t* h, const es_touch_batch_t* prepared, void* stream);

/* kernel_manager_t::constant_fill (src/engine/gpu/gpu_kernel_manager.h:319,
 * gpu_kernel_manager.cc:1064-1089).  value8 = the scalar's 8 raw bytes. */
int es_b200_fill_constant(es_b200_t*  h,
                          int         dtype,
                          const void* value8,
                          uint64_t    nelem,
                          void*       stream,
                          void*       out);

/* kernel_manager_t::lowerTri_fill (src/engine/gpu/gpu_kernel_manager.h:315,
 * gpu_kernel_manager.cc:1037-1062): out[i,j] = (i - start >= j) ? lower : upper,
 * start signed (src/einsummable/fill.h:17-26). */
int es_b200_fill_lowertri(es_b200_t*  h,
                          int         dtype,
                          const void* lower8,
                          const void* upper8,
                          uint64_t    nrow,
                          uint64_t    ncol,
                          int64_t     start,
                          void*       stream,
                          void*       out);

/* gpu_copy_t::launch (src/engine/gpu/exec_graph.cc:406-467): copy `bytes` from
 * src on src_device to dst on dst_device.  The handle must belong to
 * dst_device; the stream is a stream of dst_device. */
int es_b200_move(es_b200_t*  h,
                 int         src_device,
                 const void* src,
                 int         dst_device,
                 void*       dst,
                 uint64_t    bytes,
                 void*       stream);

/* Host storage for evicted tensors: gpu_storage_t (src/engine/gpu/storage.h:20-86, storage.cc:4-29:
 * one pinned, portable host allocation of the whole storage size; write-combined there, optional
 * here because saved tensors that end up in storage are read back by the host).  Every storage id
 * owns one block.  write / read / remove / reference are the host-side members of the same names. */
typedef struct es_b200_storage es_b200_storage_t;
int es_b200_storage_create(uint64_t bytes, int write_combined, es_b200_storage_t** out);
int es_b200_storage_destroy(es_b200_storage_t* s);
int es_b200_storage_write(es_b200_storage_t* s, int id, const void* host_src, uint64_t bytes);
int es_b200_storage_read(es_b200_storage_t* s, int id, void* host_dst, uint64_t bytes);
int es_b200_storage_remove(es_b200_storage_t* s, int id);
int es_b200_storage_reference(es_b200_storage_t* s, int id, void** host_ptr, uint64_t* bytes);
/* gpu_evict_t::launch (src/engine/gpu/exec_graph.cc:469-515): reserve `id` and copy `bytes` from
 * device memory into it, asynchronously on `stream`.
 * gpu_load_t::launch (:517-577): copy the id's bytes back to device memory on `stream`; the id
 * leaves the storage at once and its block is reused once that copy has finished. */
int es_b200_evict(es_b200_t* h, es_b200_storage_t* s, int id, const void* dev_src, uint64_t bytes, void* stream);
int es_b200_load(es_b200_t* h, es_b200_storage_t* s, int id, void* dev_dst, uint64_t bytes, void* stream);

/* move_t between two processes that each drive one GPU (the reference drives all
 * GPUs of a box from one process and needs no hand-shake: src/engine/gpu/exec_graph.cc:406-467;
 * these three calls have no counterpart there).  `flag` is a zero-initialised 32-bit word
 * in memory both GPUs can address (e.g. symmetric / IPC-mapped memory):
 *   es_b200_flag_signal : stream-ordered; waits until *flag == 0, then stores 1.  Used on the
 *                         peer's flag ("my data is ready" / "I have finished reading").
 *   es_b200_flag_wait   : stream-ordered; waits until *flag == 1, then stores 0.
 *   es_b200_pull        : SM copy of `bytes` from a peer-mapped `src` into local `dst`
 *                         (128-bit loads over NVLink), any size.
 * Waits are bounded by limit_ms (0 = 2000 ms): on expiry the kernel records an error word
 * (bits 8..15 of es_b200_device_status: 1 = signal, 2 = wait) and returns; nothing traps. */
int es_b200_flag_signal(es_b200_t* h, void* flag, uint32_t limit_ms, void* stream);
int es_b200_flag_wait(es_b200_t* h, void* flag, uint32_t limit_ms, void* stream);
int es_b200_pull(es_b200_t* h, const void* src, void* dst, uint64_t bytes, void* stream);

/* The attention chain of a transformer layer as one launch.  It stands for FIVE consecutive apply
 * nodes of the reference -- the scores contraction, the max and sum reductions and the elementwise
 * node of the softmax (src/einsummable/gwriter.cc:830-855), and the contraction with the values
 * (attention_t::forward, llama/modules.cc:285-383) -- each of which the reference launches through
 * kernel_manager_t::operator() (src/engine/gpu/gpu_kernel_manager.cc:852-978):
 *   S[b,h,i,j] = sum_d Q[b,h,i,d] K[b,h,j,d]    f16 inputs, f32 accumulate, rounded to f16
 *   X          = S + mask[i,j]                  f16 add (mask may be NULL), taken to f32
 *   P          = exp(X - max_j X) / sum_j exp(X - max_j X), rounded to f16
 *   O[b,h,i,d] = sum_j P[b,h,i,j] V[b,h,j,d]    f32 accumulate, rounded to f16
 * Q, K, V, O are f16 views with arbitrary element strides for (batch, head, row) -- multiples of 8
 * -- and the head dim (a multiple of 8, at most 128) contiguous; all 16-byte aligned.  The
 * [b,h,i,j] tensors never exist in memory. */
typedef struct {
    uint32_t batch, heads, rows, keys, head_dim;
    int32_t  skip_known;    /* nonzero: the mask is exactly a lower-triangular fill, mask[i][j] = 0 for
                               j <= i - skip_from and -inf above: it is then computed, not read, and
                               blocks of keys no row of a tile may see are not visited */
    int32_t  skip_from;
    int32_t  reserved;
    int64_t  q_stride[3];   /* elements: batch, head, row */
    int64_t  k_stride[3];   /* batch, head, key */
    int64_t  v_stride[3];   /* batch, head, key */
    int64_t  out_stride[3]; /* batch, head, row */
    int64_t  mask_stride;   /* row stride of the f16 mask [rows, keys]; keys contiguous */
} es_attention_t;
int es_b200_launch_attention(es_b200_t* h, const es_attention_t* a, void* stream, void* out,
                             const void* q, const void* k, const void* v, const void* mask);

/* Introspection: "kind|merged str|vector width|..." of a built kernel. */
int es_b200_kernel_info(es_b200_t* h, uint64_t kernel_id, char* buf, int buf_len);

/* Host-only helpers (no GPU needed): what build() would generate.  `what`:
 * 0 = merged form "str|join_shape|out_rank|inns", 1 = kernel kind,
 * 2 = generated CUDA source (empty for precompiled kinds),
 * 3 = compile the generated source for sm_100a and return the log,
 * 4 = the tensor-core contraction's plan (tile shape, stages, schedule; empty for other kinds),
 * 5 = compile the generated source the way build() does -- through the kernel cache on disk
 *     ($ES_B200_CACHE_DIR, default ~/.cache/es_b200, "0" = off: one file per kernel source and compiler
 *     version, so that a later process pays a file read instead of an NVRTC run) -- and return its size. */
int es_b200_describe(const es_einsummable_desc_t* desc, int what, char* buf, int buf_len);

/* Simplify a touch (src/einsummable/touch.cc:3-28); returns the new rank in
 * *out_rank, dims_out must hold `rank` entries. */
int es_b200_touch_simplify(const es_touchdim_t* dims,
                           int                  rank,
                           es_touchdim_t*       dims_out,
                           int*                 out_rank);

/* Row sum of a dense f32 matrix, out[a] = sum_b in[a,b] (the "ab->a" castable-add
 * einsummable), for callers that cannot allocate device memory: engines that
 * have already given all of the GPU's memory to one memgraph buffer (a later
 * cudaMalloc has nothing to return), and event loops that must not take
 * cudaMalloc's device-wide synchronisation.  It has no counterpart in the
 * reference, whose workspace manager allocates on demand.
 * The partial sums of the two-pass reduction live in a fixed array inside the
 * library (65536 floats = 256 KiB per GPU, held from load to exit), so:
 *   - rows must be <= 65536, otherwise ES_NOT_SUPPORTED (use
 *     es_b200_launch_einsummable with a workspace instead);
 *   - the first call on a device looks up the array's address; issue it before
 *     any stream capture begins;
 *   - all calls on one device share the array: calls whose kernels can overlap
 *     on that GPU race.  Nothing needs clearing between calls.
 * Never calls cudaMalloc/cudaFree or any allocating routine. */
int es_b200_rowsum_f32_noalloc(es_b200_t*   h,
                               const float* in,
                               float*       out,
                               uint64_t     rows,
                               uint64_t     cols,
                               void*        stream);

/* Synchronises the device and returns (and clears) the error word of the
 * tensor-core kernels: 0 = fine; nonzero = a bounded wait inside a kernel gave
 * up (1 producer, 2/3 MMA issuer, 4 epilogue) and that launch's output is not
 * valid; 0x11..0x16 = the same inside the attention kernel (Q copy, K copy, scores, P tile,
 * V copy, P V).  The reference has no counterpart: its library kernels cannot report. */
int es_b200_device_status(es_b200_t* h, unsigned int* error_word);

/* Clock trace of the tensor-core contraction kernel (trace builds only: the library compiled
 * with -DES_B200_TRACE records clock64() at the role boundaries of CTA 0, 8 slots of 1000
 * entries, see csrc/contraction.cu; entries 8000..8511: 16 slots of 32 entries of the attention
 * kernel, see csrc/attention.cu).  Copies up to `n` samples of the last launch; a normal
 * build returns ES_NOT_SUPPORTED.  The reference has no counterpart (its timetracker hooks in
 * src/engine/cpu/kernel_executor.cc:459-591 are host-side and commented out). */
int es_b200_debug_trace(es_b200_t* h, unsigned long long* out, int n, int* n_out);

/* Launch counters since creation: launches[class], class order =
 * einsummable, touch, fill, move.  The reference has no counterpart (its counters are the
 * commented-out timetracker hooks of src/engine/cpu/kernel_executor.cc:459-591). */
int es_b200_query_counters(es_b200_t* h, uint64_t launches[4]);

/* Algorithmic work launched since creation, per class in the same order: bytes every launch
 * must move (inputs once + output once; touch copy 2x, accumulate 3x the region; fills and
 * moves their size) and the multiply-add flops of the contractions (2 * prod(join_shape), the
 * reference counts prod(join_shape): src/einsummable/taskgraph.cc:2262-2271). */
int es_b200_query_work(es_b200_t* h, uint64_t bytes[4], uint64_t* contraction_flops);

/* ---------------------------------------------------------------------------------------------
 * Program: the nodes of one memgraph that run on this GPU, as a static schedule.
 *
 * Stands in for make_gpu_exec_graph + exec_state_t::event_loop
 * (src/engine/gpu/exec_graph.cc:37-256, src/engine/exec_state.cc:110-219): there every node is
 * launched from the host when the stream callbacks of its dependencies have fired
 * (cudaStreamAddCallback, src/engine/gpu/exec_graph.cc:318-332; at most 5 streams per device,
 * src/server/gpu/server.h:81).  Here every op names the earlier ops it depends on, finalize
 * assigns the ops to lanes (CUDA streams) joined by events, and a launch issues the whole
 * schedule without returning to the host; instantiate captures it into one CUDA graph.
 *
 * Ops are added in an order in which every dependency comes first (the memgraph's node order
 * is one, src/einsummable/memgraph.h:167-173); `deps` holds indices of earlier ops, *op_index
 * receives the new op's index.  Pointers are device pointers owned by the caller and must stay
 * valid while the program exists.  A program is used from one host thread, one launch at a time.
 *
 * Exchange between processes that each drive one GPU (no counterpart in the reference, whose
 * one process copies between its GPUs directly, src/engine/gpu/exec_graph.cc:406-467): flags
 * are zero-initialised 32-bit words both GPUs can address.  Every run of a program increments
 * the program's own run counter; `signal` stores it into flags in the peers' memory, `wait`
 * waits for local flags (a move's ready flag, or the done flags of moves this rank sent) to
 * reach it, `pull` copies over NVLink and then stores it into the done flag in the source
 * rank's memory (a remote touch does the same after reading its input).
 * All ranks must therefore run their programs the same number of times.  Ops that wait for a
 * peer (pull, wait) are issued on a few lanes of their own, each in program order: add them in
 * one global order on every rank, along which every dependency points forward.  Waits are bounded (es_b200_program_set_wait_limit, default 2000 ms): on
 * expiry the kernel records a code in bits 8..15 of es_b200_device_status (3 = pull, 4 = wait)
 * and the schedule carries on; nothing traps. */
typedef struct es_b200_program es_b200_program_t;

typedef struct {
    const void* src;        /* peer-mapped source, 16-byte aligned */
    void*       dst;        /* local destination, 16-byte aligned */
    uint64_t    bytes;
    void*       ready_flag; /* local flag raised by the source rank's signal; NULL when a wait op
                               the pull depends on has already waited for it (then the pull itself
                               does not wait for a peer and runs on any lane) */
    void*       done_flag;  /* flag in the source rank's memory: raised after the copy */
} es_pull_item_t;

/* h may be NULL: the program can then be filled, finalized and described (host only, for
 * inspecting the schedule) but not launched. */
int es_b200_program_create(es_b200_t* h, es_b200_program_t** out);
int es_b200_program_destroy(es_b200_program_t* p);

/* gpu_einsummable_t::launch (src/engine/gpu/exec_graph.cc:277-335); kernel_id from
 * es_b200_build_einsummable; the workspace comes from es_b200_program_set_workspace. */
int es_b200_program_add_einsummable(es_b200_program_t* p, uint64_t kernel_id, void* out,
                                    const void* const* inns, int n_inn,
                                    const int* deps, int n_deps, int* op_index);
/* gpu_touch_t::launch (src/engine/gpu/exec_graph.cc:354-404).  The caller resolves the
 * first-touch-of-a-group-is-a-copy rule (:167-172, 368-378) by passing the castable to use
 * and by making the touches of one group depend on one another. */
int es_b200_program_add_touch(es_b200_program_t* p, const es_touchdim_t* dims, int rank, int castable,
                              int dtype, void* out, const void* inn,
                              const int* deps, int n_deps, int* op_index);
/* A touch whose input lies in a peer GPU's memory (move_t followed by the touch that consumes it,
 * src/engine/gpu/exec_graph.cc:354-467, as one kernel: the bytes cross NVLink once, straight into
 * the region they belong to).  A wait op among `deps` must have seen the move's ready flag; the
 * last CTA raises `done_flag` (in the source rank's memory) when the input has been read. */
int es_b200_program_add_remote_touch(es_b200_program_t* p, const es_touchdim_t* dims, int rank, int castable,
                                     int dtype, void* out, const void* inn_peer, void* done_flag,
                                     const int* deps, int n_deps, int* op_index);
/* Many touches of one dtype whose destinations do not overlap, as one launch. */
int es_b200_program_add_touch_batch(es_b200_program_t* p, const es_touch_item_t* items, int n, int dtype,
                                    const int* deps, int n_deps, int* op_index);
/* gpu_constant_t / gpu_lowerTri_t::launch (src/engine/gpu/exec_graph.cc:623,675). */
int es_b200_program_add_fill_constant(es_b200_program_t* p, int dtype, const void* value8, uint64_t nelem,
                                      void* out, const int* deps, int n_deps, int* op_index);
int es_b200_program_add_fill_lowertri(es_b200_program_t* p, int dtype, const void* lower8, const void* upper8,
                                      uint64_t nrow, uint64_t ncol, int64_t start, void* out,
                                      const int* deps, int n_deps, int* op_index);
/* gpu_copy_t::launch for a move or copy inside this GPU (src/engine/gpu/exec_graph.cc:406-467). */
int es_b200_program_add_copy(es_b200_program_t* p, const void* src, void* dst, uint64_t bytes,
                             const int* deps, int n_deps, int* op_index);
/* evict_t / load_t of a static schedule: the host block of every storage id is fixed by the caller
 * (pinned memory, e.g. es_b200_storage_reference), the op is the one cudaMemcpyAsync. */
int es_b200_program_add_evict(es_b200_program_t* p, const void* dev_src, void* host_dst, uint64_t bytes,
                              const int* deps, int n_deps, int* op_index);
int es_b200_program_add_load(es_b200_program_t* p, const void* host_src, void* dev_dst, uint64_t bytes,
                             const int* deps, int n_deps, int* op_index);
/* The fused attention chain (es_b200_launch_attention) as one op of the program. */
int es_b200_program_add_attention(es_b200_program_t* p, const es_attention_t* a, void* out,
                                  const void* q, const void* k, const void* v, const void* mask,
                                  const int* deps, int n_deps, int* op_index);
int es_b200_program_add_signal(es_b200_program_t* p, void* const* flags, int n,
                               const int* deps, int n_deps, int* op_index);
int es_b200_program_add_pull(es_b200_program_t* p, const es_pull_item_t* items, int n,
                             const int* deps, int n_deps, int* op_index);
int es_b200_program_add_wait(es_b200_program_t* p, void* const* flags, int n,
                             const int* deps, int n_deps, int* op_index);

/* Computes the schedule (max_lanes compute lanes, 0 = 8; plus the exchange lane when the
 * program has pull / wait ops), creates streams and events and uploads the descriptor arrays.
 * *workspace_bytes = what es_b200_program_set_workspace must be given (each lane has its own
 * slice, as gpu_workspace_manager_t lends one workspace per node in flight,
 * src/engine/gpu/workspace.cc:49-91). */
int es_b200_program_finalize(es_b200_program_t* p, int max_lanes, uint64_t* workspace_bytes);
int es_b200_program_set_workspace(es_b200_program_t* p, void* workspace, uint64_t bytes);
int es_b200_program_set_wait_limit(es_b200_program_t* p, uint32_t limit_ms);
/* Before finalize: how many lanes the pull / wait ops share (1..4, default 1; round robin in
 * program order).  More lanes let exchanges that arrive out of the expected order overtake, but
 * put more kernels that spin on a peer's flag in flight at once: with 4, launched eagerly on more
 * streams than the GPU has hardware queues, bounded waits have run out on an 8-GPU box. */
int es_b200_program_set_exchange_lanes(es_b200_program_t* p, int lanes);

/* One run, asynchronous: everything is ordered after the work already on `stream`, and
 * `stream` continues only when every op has finished. */
int es_b200_program_launch(es_b200_program_t* p, void* stream);
/* The same with a CUDA event pair around every op; synchronises `stream` and returns the
 * milliseconds each op held its lane (for pull / wait ops this includes the time spent
 * waiting for the peer). */
int es_b200_program_launch_timed(es_b200_program_t* p, void* stream, float* ms_per_op, int n);
/* Captures one run into a CUDA graph (run the program once before, so that everything is
 * loaded); replay launches that graph on `stream`. */
int es_b200_program_instantiate(es_b200_program_t* p);
int es_b200_program_replay(es_b200_program_t* p, void* stream);
/* One replay of the run captured with a time stamp (the GPU's nanosecond timer) before and
 * after every op: ns[2*i], ns[2*i+1] = when op i could start on its lane and when it had
 * finished; ns[2*n_ops], ns[2*n_ops+1] = begin and end of the run.  Synchronises `stream`.
 * The first call captures that second graph (run the program once before). */
int es_b200_program_replay_timed(es_b200_program_t* p, void* stream, unsigned long long* ns, int n);
/* Synchronises the device and sets the run counter back to zero (flags are the caller's to
 * clear); all ranks do this together, between runs. */
int es_b200_program_reset_epoch(es_b200_program_t* p);
/* The schedule as JSON: lanes, per op its kind, lane, dependencies and the events it waits for.
 * With buf == NULL only *needed (bytes incl. the terminator) is returned. */
int es_b200_program_describe(es_b200_program_t* p, char* buf, int buf_len, int* needed);

/* ---------------------------------------------------------------------------------------------
 * Interchange formats (host only, no GPU needed).
 *
 * The protobuf messages of src/proto/einsummable.proto:5-320 that carry graphs between processes
 * (memgraph_t::to_wire / from_wire, src/einsummable/memgraph.cc:258-380, src/server/mg_base.cc:118;
 * likewise taskgraph_t, einsummable_t, touch_t, fill_t, partition_t, placement_t): `message` is the
 * message name ("MemGraph", "TaskGraph", "Einsummable", ...); the JSON side uses the .proto's field
 * names, repeated fields as arrays, absent optional fields left out.  With buf == NULL only
 * *needed is returned.  to_json output is NUL-terminated; from_json output is the raw bytes. */
int es_b200_wire_to_json(const char* message, const void* bytes, uint64_t n, char* buf, uint64_t buf_len,
                         uint64_t* needed);
int es_b200_wire_from_json(const char* message, const char* json, void* buf, uint64_t buf_len, uint64_t* needed);

/* The weight file of llama/from_pth2.py:27-35, read by llama/reader.cc:42-110: records of a 50-byte
 * space-padded tensor name, an int64 element count and that many f16 values.
 * list: '\n'-separated names into `names`, element counts into nelems[0..max_records), *count records.
 * read: the named tensor's f16 values into dst (dst == NULL: only *nelem).  append: one more record. */
int es_b200_weight_file_list(const char* path, char* names, uint64_t names_len, uint64_t* nelems, int max_records,
                             int* count);
int es_b200_weight_file_read(const char* path, const char* tensor_name, void* dst, uint64_t dst_bytes, uint64_t* nelem);
int es_b200_weight_file_append(const char* path, const char* tensor_name, const void* f16_data, uint64_t nelem);

const char* es_b200_last_error(void);
const char* es_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif
