// Precompiled (sm_100a) kernels: touch, fills, move.
#pragma once
#include <cuda_runtime.h>

#include "common.h"

namespace es {

// Exact division of numerators below 2^31 by a fixed divisor d:
// q = umulhi(n, m) >> s with l = ceil(log2 d), m = ceil(2^(31+l) / d), s = l - 1.
struct fastdiv_t {
    uint32_t m;
    uint32_t s;
    uint32_t d;
    uint32_t pad;
};

// A simplified touch prepared for the device: byte pointers already advanced to
// the first element of the region, byte strides of the (up to three) outer
// dims, and the innermost row expressed in vectors of `W` bytes.
struct touch_args_t {
    char const* inn;
    char*       out;
    uint64_t    sin[3];
    uint64_t    sout[3];
    fastdiv_t   div_n1, div_n2, div_segs; // divisors: n1, n2, segments per row
    uint32_t    n_rows;                   // n0*n1*n2
    uint32_t    row_vecs;                 // vectors per innermost row
    uint32_t    seg_shift;                // log2(vectors per segment)
    uint32_t    segs_per_row;
    uint64_t    total_slots;              // n_rows * segs_per_row << seg_shift  (< 2^31)
    int32_t     castable;
    int32_t     pad;
    // A touch that reads a peer GPU's memory (`inn` peer-mapped) acknowledges the read: the last
    // CTA to finish stores *epoch into *done (a flag in the source GPU's memory).  Null otherwise.
    uint32_t*       done;
    uint32_t*       counter; // CTAs finished so far; returns to zero
    uint32_t const* epoch;
};

// Host: simplify (src/einsummable/touch.cc:3-28) + bounds checks + lowering.
// Returns the widest vector width (16/8/4/2 bytes, or 8 for f64/c64 minimum)
// that the region's alignment allows; fills `a` for that width.
int prepare_touch(es_touchdim_t const* dims,
                  int                  rank,
                  int                  castable,
                  int                  dtype,
                  void*                out,
                  void const*          inn,
                  touch_args_t&        a);

// Re-expresses `a` (prepared at width w_from) at the narrower width w_to.
void narrow_touch(touch_args_t& a, int w_from, int w_to);

int simplify_touch(es_touchdim_t const* dims, int rank, es_touchdim_t* out);

void launch_touch(touch_args_t const& a, int width, int dtype, cudaStream_t stream);
void launch_touch_batch(touch_args_t const* items_dev,
                        int                 n,
                        uint64_t            max_slots,
                        int                 width,
                        int                 dtype,
                        cudaStream_t        stream);

void launch_fill_constant(int dtype, void const* value8, uint64_t nelem, cudaStream_t s, void* out);
void launch_fill_lowertri(int          dtype,
                          void const*  lower8,
                          void const*  upper8,
                          uint64_t     nrow,
                          uint64_t     ncol,
                          int64_t      start,
                          cudaStream_t s,
                          void*        out);

// Cross-GPU flags for move hand-shakes between processes that each drive one GPU.
// A flag is a 32-bit word in memory both GPUs can address (peer-mapped).
//   signal: wait (bounded) until *flag == 0, then store 1 (system-scope release)
//   wait  : wait (bounded) until *flag == 1, then store 0 (the flag is local)
// A wait that exceeds `limit_ms` records an error word and returns; nothing traps.
void launch_flag_signal(uint32_t* flag, uint32_t limit_ms, cudaStream_t s);
void launch_flag_wait(uint32_t* flag, uint32_t limit_ms, cudaStream_t s);
unsigned int read_and_clear_flag_error();

// SM pull-copy: 128-bit loads from `src` (possibly peer-mapped) into local `dst`.
void launch_pull_copy(void const* src, void* dst, uint64_t bytes, cudaStream_t s);

} // namespace es
