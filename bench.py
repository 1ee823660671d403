#!/usr/bin/env python3
"""Benchmark of the memgraph apply-node kernels on B200.

Workload (N=1): BASELINE config 2 -- f16 tensors x, y of shape [8192, 11008]
~ N(0,1); one step = one pass of the four einsummables over them, launched
through the C ABI on one stream:
    (i)   a,a->a    silu(x) * y
    (ii)  ab->a     castable max            (row max of x)
    (iii) ab,a->ab  exp(x - rowmax)
    (iv)  ab->a     castable add            (row sum of (iii))
Metric: algorithmic GB/s (inputs + outputs of every op, broadcast inputs at
their own size) over the whole step.  Under torchrun every rank runs the same
workload on its own GPU (the path shards by blocks with no data-path
collective), value = bytes of all ranks / max-over-ranks device time.

Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of
the reference's CPU kernels (oracle/es_oracle.c) on the host cores instead.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS = 8192, 11008
N = ROWS * COLS
# algorithmic bytes of one step (f16 = 2 bytes)
BYTES_SILU_MUL = 3 * N * 2
BYTES_ROWMAX = N * 2 + ROWS * 2
BYTES_EXP_SUB = 2 * N * 2 + ROWS * 2
BYTES_ROWSUM = N * 2 + ROWS * 2
BYTES_STEP = BYTES_SILU_MUL + BYTES_ROWMAX + BYTES_EXP_SUB + BYTES_ROWSUM
WORKLOAD = "C2 f16 [8192,11008]: silu(x)*y; rowmax; exp(x-rowmax); rowsum"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the silu*y kernel: ncu capture of
# the [4096,11008] case (180.37 MB read + 47.75 MB written, profiles/c2_kernels_f16_4096x11008.md)
# scaled x2 to the full launch.  Below the algorithmic 541 MB because part of the output is still
# dirty in the 126 MB L2 when the kernel ends.
SILU_MUL_DRAM_TRAFFIC = 2 * (180374528 + 47752960)


def set_rows(rows):
    global ROWS, N, BYTES_SILU_MUL, BYTES_ROWMAX, BYTES_EXP_SUB, BYTES_ROWSUM, BYTES_STEP, WORKLOAD
    if rows == ROWS:
        return
    ROWS, N = rows, rows * COLS
    BYTES_SILU_MUL = 3 * N * 2
    BYTES_ROWMAX = N * 2 + ROWS * 2
    BYTES_EXP_SUB = 2 * N * 2 + ROWS * 2
    BYTES_ROWSUM = N * 2 + ROWS * 2
    BYTES_STEP = BYTES_SILU_MUL + BYTES_ROWMAX + BYTES_EXP_SUB + BYTES_ROWSUM
    WORKLOAD = "REDUCED (profiling only) f16 [%d,11008]: silu(x)*y; rowmax; exp(x-rowmax); rowsum" % rows


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------
# CPU baseline: the C restatement of the reference CPU engine's kernels
# --------------------------------------------------------------------------
def load_cpu_oracle():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "libes_oracle.so"))
    lib.oracle_num_threads.restype = ctypes.c_int
    return lib


def cpu_pass(lib, rows, x, y, out, m, ex, s):
    p = lambda a: ctypes.c_void_p(a.ctypes.data)
    n = rows * COLS
    lib.oracle_silu_mul_f16(ctypes.c_uint64(n), p(out), p(x), p(y))
    lib.oracle_reduce_ab_a_f16(3, ctypes.c_uint64(rows), ctypes.c_uint64(COLS), p(m), p(x))
    lib.oracle_exp_sub_ab_a_f16(ctypes.c_uint64(rows), ctypes.c_uint64(COLS), p(ex), p(x), p(m))
    lib.oracle_reduce_ab_a_f16(0, ctypes.c_uint64(rows), ctypes.c_uint64(COLS), p(s), p(ex))


def cpu_bytes(rows):
    n = rows * COLS
    return 3 * n * 2 + (n * 2 + rows * 2) + (2 * n * 2 + rows * 2) + (n * 2 + rows * 2)


def cpu_buffers(rows, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(rows * COLS).astype(np.float16)
    y = rng.standard_normal(rows * COLS).astype(np.float16)
    return (x, y, np.empty_like(x), np.empty(rows, np.float16), np.empty_like(x), np.empty(rows, np.float16))


def cpu_baseline(budget_s=10.0, rows=1024):
    lib = load_cpu_oracle()
    bufs = cpu_buffers(rows)
    cpu_pass(lib, rows, *bufs)  # warm
    t0 = time.perf_counter()
    passes = 0
    while True:
        cpu_pass(lib, rows, *bufs)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or passes >= 200:
            break
    res = {
        "value": cpu_bytes(rows) * passes / dt / 1e9, "unit": "GB/s", "cores": lib.oracle_num_threads(),
        "kind": "port",
        "sample": "%d passes over the first %d of %d rows (same 4 ops, OpenMP over row blocks), %.1f s"
                  % (passes, rows, ROWS, dt),
    }
    try:
        res["other_classes"] = cpu_other_classes(lib)
    except Exception as exc:  # reported, never hidden
        res["other_classes"] = {"error": repr(exc)[:200]}
    return res


def cpu_other_classes(lib):
    """The other kernel classes on the host cores, bounded samples: the C1 block contraction
    (f32 2048^3) through the C port's blocked loops and through torch's CPU sgemm (the
    closest stand-in here for the cblas_sgemm the reference's executor calls,
    src/engine/cpu/kernel_executor.cc:1293-1548), and a C3 copy / accumulate touch through
    the port of execute_touch (src/engine/touch.cc:155-237)."""
    import torch
    out = {}
    p = lambda a: ctypes.c_void_p(a.ctypes.data)
    rng = np.random.default_rng(1)
    n = 2048
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    c = np.empty((n, n), np.float32)
    rows = 256  # the port's triple loop: a 256-row slab of the block
    t0 = time.perf_counter()
    lib.oracle_matmul_f32(ctypes.c_uint64(rows), ctypes.c_uint64(n), ctypes.c_uint64(n), p(c), p(a), p(b))
    dt = time.perf_counter() - t0
    out["C1 block ij,jk->ik f32 (port, %d of 2048 rows)" % rows] = {"TFLOP/s": 2.0 * rows * n * n / dt / 1e12}
    ta, tb = torch.from_numpy(a), torch.from_numpy(b)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    torch.matmul(ta, tb)
    t0 = time.perf_counter()
    for _ in range(3):
        torch.matmul(ta, tb)
    dt = (time.perf_counter() - t0) / 3
    out["C1 block ij,jk->ik f32 2048^3 (torch CPU sgemm, stand-in for cblas_sgemm)"] = {
        "TFLOP/s": 2.0 * n ** 3 / dt / 1e12, "threads": torch.get_num_threads()}
    # C3 p=2 block: [16,256,16,64] of f16 into a [32,512,32,128] tensor
    sel = [(16, 32, 0, 16, 16), (256, 512, 0, 256, 256), (16, 32, 0, 16, 16), (64, 128, 0, 64, 64)]
    dims = (ctypes.c_uint64 * 20)(*[v for d in sel for v in d])
    src = rng.uniform(-1, 1, 16 * 256 * 16 * 64).astype(np.float16)
    dst = np.zeros(32 * 512 * 32 * 128, np.float16)
    for name, castable, factor in (("copy", -1, 2), ("add", 0, 3)):
        lib.oracle_touch(4, dims, castable, 0, p(dst), p(src))
        t0 = time.perf_counter()
        for _ in range(5):
            lib.oracle_touch(4, dims, castable, 0, p(dst), p(src))
        dt = (time.perf_counter() - t0) / 5
        out["touch C3 p=2 f16 %s (port of execute_touch)" % name] = {"GB/s": factor * src.nbytes / dt / 1e9}
    return out


def run_reference_arm(args):
    """The reference's CPU implementation of the path on the host cores.  The
    reference's MKL executor cannot be built here (no MKL; merge-conflict markers
    in src/engine/cpu/kernel_executor.cc:1323-1445), so this is the C port of its
    loops; each step is one pass over a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1024
    lib = load_cpu_oracle()
    bufs = cpu_buffers(rows)
    for _ in range(args.warmup):
        cpu_pass(lib, rows, *bufs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(lib, rows, *bufs)
    dt = time.perf_counter() - t0
    value = cpu_bytes(rows) * args.steps / dt / 1e9
    cores = lib.oracle_num_threads()
    sample = "each step = one pass over the first %d of %d rows (same 4 ops)" % (rows, ROWS)
    print(json.dumps({
        "impl": "reference", "metric": "elementwise+reduction algorithmic GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------
# clocks during the timed region
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [l for (t, l) in self.samples if t_begin <= t <= t_end] or [l for (_, l) in self.samples]
        sm, mx, reasons = [], [], set()
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import einsummable_b200 as es
    from einsummable_b200 import einsummable_t, scalarop_t as S, touch_t

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    km = es.kernel_manager_t(local)  # raises if the CUDA library or device is missing

    f16 = "f16"
    e_silu = einsummable_t([ROWS, COLS], [[0, 1], [0, 1]], 2,
                           S.combine(S.make_mul(f16), [S.make_silu(f16), S.make_identity(f16)]))
    e_max = einsummable_t([ROWS, COLS], [[0, 1]], 1, S.make_identity(f16), "max")
    e_exp = einsummable_t([ROWS, COLS], [[0, 1], [0]], 2, S.combine(S.make_exp(f16), [S.make_sub(f16)]))
    e_sum = einsummable_t([ROWS, COLS], [[0, 1]], 1, S.make_identity(f16), "add")
    ops = [e_silu, e_max, e_exp, e_sum]
    ws_bytes = max(km.build(e) for e in ops)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    wsarg = (ws, ws_bytes) if ws_bytes else None

    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    x = torch.randn(N, dtype=torch.float16, device=dev, generator=g)
    y = torch.randn(N, dtype=torch.float16, device=dev, generator=g)
    o_silu = torch.empty(N, dtype=torch.float16, device=dev)
    o_max = torch.empty(ROWS, dtype=torch.float16, device=dev)
    o_exp = torch.empty(N, dtype=torch.float16, device=dev)
    o_sum = torch.empty(ROWS, dtype=torch.float16, device=dev)
    stream = torch.cuda.current_stream(dev)

    def step(events=None):
        if events is not None:
            events[0].record(stream)
        km(e_silu, stream, o_silu, [x, y], wsarg)
        if events is not None:
            events[1].record(stream)
        km(e_max, stream, o_max, [x], wsarg)
        if events is not None:
            events[2].record(stream)
        km(e_exp, stream, o_exp, [x, o_max], wsarg)
        if events is not None:
            events[3].record(stream)
        km(e_sum, stream, o_sum, [o_exp], wsarg)
        if events is not None:
            events[4].record(stream)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    c0 = km.counters()
    barrier()
    t_begin = time.perf_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for k in range(args.steps):
        step(ev[k])
    end.record(stream)
    barrier()
    t_end = time.perf_counter()
    c1 = km.counters()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ms = start.elapsed_time(end)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    per_kernel_ms = [float(np.mean([ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(args.steps)]))
                     for i in range(4)]
    launches = sum(c1[k] - c0[k] for k in c0)

    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"metric": "elementwise+reduction algorithmic GB/s (kernels only)",
                              "value": BYTES_STEP * world * args.steps / (ms * 1e-3) / 1e9, "unit": "GB/s",
                              "config": {"workload": WORKLOAD}, "ms_per_step": ms / args.steps,
                              "per_kernel_ms": per_kernel_ms, "gpu_launches": int(launches)}))
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return

    # ---- end to end: host buffers in, results back on the host, every step ----
    # Every step copies its own inputs from pinned host memory and its results back.  The copies
    # of neighbouring steps overlap the kernels on separate streams (double-buffered device
    # inputs and outputs): H2D of step i+1 and D2H of step i-1 run while step i computes.
    hx = torch.randn(N, dtype=torch.float16).pin_memory()
    hy = torch.randn(N, dtype=torch.float16).pin_memory()
    h_silu = torch.empty(N, dtype=torch.float16).pin_memory()
    h_max = torch.empty(ROWS, dtype=torch.float16).pin_memory()
    h_sum = torch.empty(ROWS, dtype=torch.float16).pin_memory()
    xs, ys = [x, torch.empty_like(x)], [y, torch.empty_like(y)]
    o_silus = [o_silu, torch.empty_like(o_silu)]
    o_maxs, o_sums = [o_max, torch.empty_like(o_max)], [o_sum, torch.empty_like(o_sum)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]      # inputs of buffer b have landed
    ev_done = [torch.cuda.Event() for _ in range(2)]    # kernels reading buffer b have finished
    ev_out = [torch.cuda.Event() for _ in range(2)]     # results of buffer b are on the host

    def e2e_step(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[b])                 # the step that last used these buffers is done
            xs[b].copy_(hx, non_blocking=True)
            ys[b].copy_(hy, non_blocking=True)
            ev_in[b].record(s_in)
        stream.wait_event(ev_in[b])
        stream.wait_event(ev_out[b])                    # previous results of this buffer were read out
        km(e_silu, stream, o_silus[b], [xs[b], ys[b]], wsarg)
        km(e_max, stream, o_maxs[b], [xs[b]], wsarg)
        km(e_exp, stream, o_exp, [xs[b], o_maxs[b]], wsarg)
        km(e_sum, stream, o_sums[b], [o_exp], wsarg)
        ev_done[b].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            h_silu.copy_(o_silus[b], non_blocking=True)
            h_max.copy_(o_maxs[b], non_blocking=True)
            h_sum.copy_(o_sums[b], non_blocking=True)
            ev_out[b].record(s_out)

    e2e_steps = max(4, min(args.steps, 10))
    for b in range(2):
        ev_done[b].record(stream)
        ev_out[b].record(stream)
    e2e_step(0)
    e2e_step(1)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record(stream)
    s_in.wait_event(s2)
    for i in range(e2e_steps):
        e2e_step(i)
    stream.wait_stream(s_out)
    stream.wait_stream(s_in)
    e2.record(stream)
    barrier()
    e2e_ms = s2.elapsed_time(e2)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    # the end-to-end result must be the same bits as the device-resident one for the same inputs
    x.copy_(hx)
    y.copy_(hy)
    step()
    torch.cuda.synchronize(dev)
    e2e_ok = bool(torch.equal(o_silu.cpu(), h_silu) and torch.equal(o_sum.cpu(), h_sum))

    # ---- other kernel classes of the metric (outside the timed region above; rank 0 only).  They
    # are kernels timed alone, so they run here, before the long graph legs heat the GPU into its
    # power cap: their fractions are quoted against the burst peak ----
    classes = {}
    if rank == 0:
        try:
            classes = other_classes(km, dev, stream)
        except Exception as exc:  # reported, never hidden
            classes = {"error": repr(exc)}
        torch.cuda.empty_cache()

    # ---- configs 4 and 5: LLaMA-7B-shape graphs, the reference's own memgraphs for `world` GPUs ----
    llama, llama_train = None, None
    try:
        llama = llama_layer_leg(rank, world, dev)
    except Exception as exc:  # reported, never hidden
        llama = {"error": repr(exc)[:300]}
    try:
        llama_train = llama_layer_leg(rank, world, dev, fixture="llama7b_train_l4", runs=5)
    except Exception as exc:  # reported, never hidden
        llama_train = {"error": repr(exc)[:300]}
    # config 5 at the batch it names (8 x 1024 tokens): 117 GB of device memory on one GPU
    llama_train_full = None
    try:
        if os.environ.get("ES_B200_BENCH_C5_FULL", "1") != "0":
            llama_train_full = llama_layer_leg(rank, world, dev, fixture="llama7b_train_b8s1024_l4", runs=3)
        else:
            llama_train_full = {"skipped": "ES_B200_BENCH_C5_FULL=0"}
    except Exception as exc:  # reported, never hidden
        llama_train_full = {"error": repr(exc)[:300]}

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    achieved = BYTES_SILU_MUL / (per_kernel_ms[0] * 1e-3) / 1e9
    line = {
        "metric": "elementwise+reduction algorithmic GB/s", "value": BYTES_STEP * world * args.steps / (ms * 1e-3) / 1e9,
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "inputs larger than L2 (3 x 180 MB per op); no flush",
                   "algorithmic_bytes_per_step": BYTES_STEP,
                   "kernels": dict(zip(["silu_mul", "rowmax", "exp_sub", "rowsum"],
                                       [km.kernel_info(e).split("|")[0] for e in ops]))},
        "clocks": clocks,
        "e2e": {"value": BYTES_STEP * world * e2e_steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": 2 * N * 2, "d2h_bytes_per_step": N * 2 + 2 * ROWS * 2,
                "ms_per_step": e2e_ms / e2e_steps, "results_match_device_run": e2e_ok,
                "overlap": "copies of neighbouring steps overlap the kernels (3 streams, double buffering)"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "silu(x)*y a,a->a f16 (generated ew_vec)", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": SILU_MUL_DRAM_TRAFFIC if ROWS == 8192 else None, "algorithmic_bytes_per_launch": BYTES_SILU_MUL},
        "per_kernel": {name: {"ms": t, "GB/s": b / (t * 1e-3) / 1e9, "frac_of_" + peak_kind: b / (t * 1e-3) / 1e9 / peak}
                       for name, t, b in zip(["silu_mul", "rowmax", "exp_sub", "rowsum"], per_kernel_ms,
                                             [BYTES_SILU_MUL, BYTES_ROWMAX, BYTES_EXP_SUB, BYTES_ROWSUM])},
        "per_kernel_note": "CUDA-event intervals between the kernels of one step: a reduction's interval also carries "
                           "the write-back of the 180 MB the kernel before it wrote (L2 holds 126 MB), so its own "
                           "rate reads low and the elementwise kernel's high; the step total is what is exact",
        "classes": classes,
        "llama7b_layer": llama,
        "llama7b_train_4layers": llama_train,
        "llama7b_train_4layers_b8_s1024": llama_train_full,
        "cpu_baseline": cpu_baseline() if world == 1 else None,
    }
    print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def llama_layer_leg(rank, world, dev, fixture="llama7b_layer", runs=10):
    """tokens/s of a LLaMA-7B-shape graph (dim 4096, 32 heads, FFN 11008, B=4, S=512, f16) executed
    from the memgraph the reference's compilers produce for `world` locations, one process per GPU,
    moves over peer memory (or NCCL send/recv).  `llama7b_layer`: one transformer layer forward plus
    final norm and last-token vocabulary projection.  `llama7b_train_l4`: four layers forward, the
    log-softmax loss, backward and the vanilla weight update.  Synthetic N(0, 0.02) weights."""
    import torch
    from einsummable_b200.memgraph import load_memgraph, memgraph_runner_t
    path = os.path.join(ROOT, "tests", "golden", "graphs", "%s_locs%d.json.gz" % (fixture, world))
    if not os.path.exists(path):
        return {"skipped": "no memgraph fixture for %d locations" % world}
    mg = load_memgraph(path)
    need = int(max(mg["mem_sizes"])) + (8 << 30)
    free = torch.cuda.mem_get_info(dev)[0]
    if free < need:
        return {"skipped": "needs %.0f GB of device memory, %.0f GB free" % (need / 1e9, free / 1e9)}
    tokens = 2048
    for t in mg["inputs"]:
        if t["name"] == "embeddings":
            tokens = int(t["shape"][0]) * int(t["shape"][1])
    transport = os.environ.get("ES_B200_MOVE_TRANSPORT", "p2p")
    if world > 1:
        try:
            r = memgraph_runner_t(mg, rank=rank, world=world, transport=transport)
        except Exception as exc:
            # symmetric memory could not be set up on this box: every rank fails the same way
            sys.stderr.write("p2p transport unavailable (%r); using NCCL send/recv\n" % (exc,))
            transport = "nccl"
            r = memgraph_runner_t(mg, rank=rank, world=world, transport="nccl")
    else:
        transport = "local"
        r = memgraph_runner_t(mg, devices=[dev.index])
    def fill_inputs(runner):
        rng = np.random.default_rng(7)
        for t in mg["inputs"]:
            shape, name = t["shape"], t["name"]
            if name == "freqs_cis":
                seq, half = shape
                ang = np.outer(np.arange(seq), 1.0 / (10000.0 ** (np.arange(half) / half)))
                v = (np.cos(ang) + 1j * np.sin(ang)).astype(np.complex64)
            elif name.endswith("norm.weight"):
                v = np.ones(shape, dtype=np.float16)
            elif name == "labels":
                v = np.zeros(shape, dtype=np.float16)
                v[np.arange(shape[0]), rng.integers(0, shape[1], shape[0])] = 1.0
            else:
                v = (rng.standard_normal(shape).astype(np.float32) * 0.02).astype(np.float16)
            runner.set_input(name, v)

    fill_inputs(r)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn):
        fn()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        for _ in range(runs):
            fn()
        e.record(stream)
        barrier()
        ms = s.elapsed_time(e) / runs
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    out = {"tokens": tokens, "gpus": world, "move_transport": transport, "nodes_this_rank": dict(r.stats),
           "taskgraph": mg["taskgraph"], "contraction_gflop": mg["taskgraph"]["contraction_flops"] / 1e9}
    ms_eager = timed(lambda: r.run(stream))
    out["eager"] = {"ms": ms_eager, "tokens/s": tokens / (ms_eager * 1e-3)}
    try:
        if transport == "nccl":
            # a process group holding captured NCCL send/recv nodes did not shut down cleanly here
            raise RuntimeError("not captured with the NCCL transport")
        r.capture()
        ms_graph = timed(r.replay)
        out["cuda_graph"] = {"ms": ms_graph, "tokens/s": tokens / (ms_graph * 1e-3),
                             "TFLOP/s": mg["taskgraph"]["contraction_flops"] / (ms_graph * 1e-3) / 1e12}
    except Exception as exc:
        out["cuda_graph"] = {"error": repr(exc)[:200]}
    out["device_status"] = r.device_status()
    r.graph = None
    r.close()
    del r
    torch.cuda.empty_cache()
    fused_multi = os.environ.get("ES_B200_BENCH_FUSED_MULTI", "1" if world <= 2 else "0") == "1"
    if transport != "nccl" and (world == 1 or fused_multi):
        # the same memgraph with elementwise producers folded into their readers (fusion across
        # node boundaries: a rewrite of the graph, not something the reference's engine does);
        # on more than two GPUs only when ES_B200_BENCH_FUSED_MULTI=1
        try:
            if world == 1:
                rf = memgraph_runner_t(mg, devices=[dev.index], fuse=True)
            else:
                rf = memgraph_runner_t(mg, rank=rank, world=world, transport=transport, fuse=True)
            fill_inputs(rf)
            rf.capture()
            ms_fused = timed(rf.replay)
            out["fused_cuda_graph"] = {"ms": ms_fused, "tokens/s": tokens / (ms_fused * 1e-3),
                                       "nodes_folded": rf.folded, "einsummables": rf.stats["einsummable"],
                                       "device_status": rf.device_status()}
            rf.graph = None
            rf.close()
            del rf
            torch.cuda.empty_cache()
        except Exception as exc:  # reported, never hidden
            out["fused_cuda_graph"] = {"error": repr(exc)[:200]}
    return out


def time_launches(fn, stream, iters=20, warm=3):
    import torch
    for _ in range(warm):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record(stream)
    for _ in range(iters):
        fn()
    e.record(stream)
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def other_classes(km, dev, stream):
    """Short measurements of the other kernel classes named by the metric:
    contraction TFLOP/s and touch / permutation GB/s (CUDA events, 20 launches)."""
    import torch
    from einsummable_b200 import einsummable_t, scalarop_t as S, touch_t
    out = {}
    # LLaMA FFN w1: ij,kj->ik f16 2048 x 11008 x 4096
    mul16 = S.make_mul("f16")
    specs = {
        "ffn_w1 ij,kj->ik f16 2048x4096x11008": einsummable_t.from_matmul_st(2048, 4096, 11008, "f16"),
        "qkv ij,kj->ik f16 2048x4096x4096": einsummable_t.from_matmul_st(2048, 4096, 4096, "f16"),
        "C1 block ij,jk->ik f32 2048^3 (3xTF32)": einsummable_t.from_matmul(2048, 2048, 2048, "f32"),
        "ij,jk->ik f16 2048x4096x4096 (B MN-major)": einsummable_t.from_str(
            "ij,jk->ik", dict(i=2048, j=4096, k=4096), mul16, "add"),
        "ji,jk->ik f16 4096x2048x4096 (both MN-major, weight-gradient shape)": einsummable_t.from_str(
            "ji,jk->ik", dict(i=4096, j=2048, k=4096), mul16, "add"),
        "attn scores acbe,adbe->abcd f16 [4,32,512,512,128]": einsummable_t.from_str(
            "acbe,adbe->abcd", dict(a=4, b=32, c=512, d=512, e=128), mul16, "add"),
        "attn PV abce,aebd->abcd f16 [4,32,512,128,512]": einsummable_t.from_str(
            "abce,aebd->abcd", dict(a=4, b=32, c=512, d=128, e=512), mul16, "add"),
    }
    for name, e in specs.items():
        i, k, j = 0, 0, 0
        ws = km.build(e)
        if "contraction_tc" not in km.kernel_info(e):
            out[name] = {"kind": km.kernel_info(e).split("|")[0], "note": "SIMT fallback; not timed"}
            continue
        tdt = torch.float16 if e.out_dtype() == "f16" else torch.float32
        a = torch.randn(int(np.prod(e.inn_shape(0))), dtype=tdt, device=dev)
        b = torch.randn(int(np.prod(e.inn_shape(1))), dtype=tdt, device=dev)
        c = torch.empty(e.out_nelem(), dtype=tdt, device=dev)
        w = torch.empty(max(ws, 16), dtype=torch.uint8, device=dev)
        ms = time_launches(lambda: km(e, stream, c, [a, b], (w, ws) if ws else None), stream)
        nbytes = (a.numel() + b.numel() + c.numel()) * a.element_size()
        out[name] = {"ms": ms, "TFLOP/s": 2.0 * float(np.prod(e.join_shape)) / (ms * 1e-3) / 1e12,
                     "GB/s": nbytes / (ms * 1e-3) / 1e9, "kind": km.kernel_info(e).split("|")[0]}
    # C3: one source block of [32,512,32,128] split 2 per dim, copy and accumulate, f16
    full = (32, 512, 32, 128)
    sel = [(16, 32, 0, 16, 16), (256, 512, 0, 256, 256), (16, 32, 0, 16, 16), (64, 128, 0, 64, 64)]
    src = torch.randn(16 * 256 * 16 * 64, dtype=torch.float16, device=dev)
    dst = torch.zeros(int(np.prod(full)), dtype=torch.float16, device=dev)
    nbytes = src.numel() * 2
    for castable, mult in ((None, 2), ("add", 3)):
        t = touch_t(sel, castable, "f16")
        ms = time_launches(lambda: km(t, stream, dst, src), stream)
        out["touch C3 p=2 f16 %s" % (castable or "copy")] = {"ms": ms, "GB/s": mult * nbytes / (ms * 1e-3) / 1e9}
    # C1: one partial-sum block, rank-1 after simplify, 4194304 f32 (copy then accumulate)
    n1 = 2048 * 2048
    p0 = torch.randn(n1, dtype=torch.float32, device=dev)
    acc = torch.zeros(n1, dtype=torch.float32, device=dev)
    for castable, mult in ((None, 2), ("add", 3)):
        t = touch_t([(n1, n1, 0, 0, n1)], castable, "f32")
        ms = time_launches(lambda: km(t, stream, acc, p0), stream)
        out["touch C1 block f32 4194304 %s" % (castable or "copy")] = {"ms": ms, "GB/s": mult * n1 * 4 / (ms * 1e-3) / 1e9}
    # the whole C3 sweep at p blocks per dim as ONE batched launch: every source block of the
    # [32,512,32,128] tensor is copied (or accumulated) into its place in the destination
    for pdim in (2, 4, 8):
        bs = [f // pdim for f in full]
        blk = int(np.prod(bs))
        nblk = pdim ** 4
        srcs = torch.randn(nblk * blk, dtype=torch.float16, device=dev)
        items = torch.empty(nblk * 256, dtype=torch.uint8, device=dev)
        for castable, mult in ((None, 2), ("add", 3)):
            touches, outs, inns = [], [], []
            for b in range(nblk):
                idx = np.unravel_index(b, (pdim,) * 4)
                sel_b = [(bs[d], full[d], 0, int(idx[d]) * bs[d], bs[d]) for d in range(4)]
                touches.append(touch_t(sel_b, castable, "f16"))
                outs.append(dst)
                inns.append(srcs[b * blk:(b + 1) * blk])
            prepared = km.prepare_touch_batch(touches, stream, outs, inns, items)
            ms = time_launches(lambda: km.launch_prepared_touch_batch(prepared, stream), stream, iters=10, warm=2)
            out["touch C3 sweep p=%d f16 %s (1 prepared batched launch, %d touches)" % (pdim, castable or "copy", nblk)] = {
                "ms": ms, "GB/s": mult * nblk * blk * 2 / (ms * 1e-3) / 1e9}
        del srcs
    e = einsummable_t([32, 32, 512, 128], [[0, 2, 1, 3]], 4, S.make_identity("f16"))
    km.build(e)
    big = torch.randn(int(np.prod(full)), dtype=torch.float16, device=dev)
    ms = time_launches(lambda: km(e, stream, dst, [big]), stream)
    out["permute bshd->bhsd f16 [32,512,32,128]"] = {"ms": ms, "GB/s": 2 * big.numel() * 2 / (ms * 1e-3) / 1e9}
    del big, dst
    # the f32 variant of the headline workload, [4096,4096], and the fused form of its last two ops
    # (ab,a->a: sum_b exp(x[a,b] - m[a]), the reference's softmax_v3 reduction) on the f16 tensors
    def timed_ew(name, e, ins, out_elems, dt, algorithmic_bytes):
        ws = km.build(e)
        o = torch.empty(out_elems, dtype=dt, device=dev)
        w = torch.empty(max(ws or 0, 16), dtype=torch.uint8, device=dev)
        ms = time_launches(lambda: km(e, stream, o, ins, (w, ws) if ws else None), stream)
        out[name] = {"ms": ms, "GB/s": algorithmic_bytes / (ms * 1e-3) / 1e9, "kind": km.kernel_info(e).split("|")[0]}
    r32, c32 = 4096, 4096
    x32 = torch.randn(r32 * c32, dtype=torch.float32, device=dev)
    y32 = torch.randn(r32 * c32, dtype=torch.float32, device=dev)
    m32 = torch.randn(r32, dtype=torch.float32, device=dev)
    f32 = "f32"
    timed_ew("C2 f32 [4096,4096] silu(x)*y (64 MB tensors: partly L2-resident)", einsummable_t([r32, c32], [[0, 1], [0, 1]], 2,
             S.combine(S.make_mul(f32), [S.make_silu(f32), S.make_identity(f32)])), [x32, y32], r32 * c32,
             torch.float32, 3 * r32 * c32 * 4)
    timed_ew("C2 f32 [4096,4096] row max (L2-resident)", einsummable_t([r32, c32], [[0, 1]], 1, S.make_identity(f32), "max"),
             [x32], r32, torch.float32, r32 * c32 * 4 + r32 * 4)
    timed_ew("C2 f32 [4096,4096] exp(x-rowmax) (partly L2-resident)", einsummable_t([r32, c32], [[0, 1], [0]], 2,
             S.combine(S.make_exp(f32), [S.make_sub(f32)])), [x32, m32], r32 * c32, torch.float32,
             2 * r32 * c32 * 4 + r32 * 4)
    timed_ew("C2 f32 [4096,4096] row sum (L2-resident)", einsummable_t([r32, c32], [[0, 1]], 1, S.make_identity(f32), "add"),
             [x32], r32, torch.float32, r32 * c32 * 4 + r32 * 4)
    timed_ew("C2 f32 [4096,4096] fused sum_b exp(x-m) ab,a->a (L2-resident)", einsummable_t([r32, c32], [[0, 1], [0]], 1,
             S.combine(S.make_exp(f32), [S.make_sub(f32)]), "add"), [x32, m32], r32, torch.float32,
             r32 * c32 * 4 + 2 * r32 * 4)
    del x32, y32
    x16 = torch.randn(ROWS * COLS, dtype=torch.float16, device=dev)
    m16 = torch.randn(ROWS, dtype=torch.float16, device=dev)
    timed_ew("C2 f16 [8192,11008] fused sum_b exp(x-m) ab,a->a", einsummable_t([ROWS, COLS], [[0, 1], [0]], 1,
             S.combine(S.make_exp("f16"), [S.make_sub("f16")]), "add"), [x16, m16], ROWS, torch.float16,
             ROWS * COLS * 2 + 2 * ROWS * 2)
    return out


def run_only(args):
    """One kernel class alone, `steps` launches after `warmup`, CUDA events."""
    import torch
    import einsummable_b200 as es
    from einsummable_b200 import einsummable_t, scalarop_t as S, touch_t
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    km = es.kernel_manager_t(0)
    stream = torch.cuda.current_stream(dev)
    mul16 = S.make_mul("f16")
    if args.only in ("llama_layer", "llama_layer_fused", "llama_train", "llama_train_fused"):
        # the LLaMA-7B-shape layer memgraph (1 location), `steps` eager runs after `warmup`
        # (profiler launch lists: every node is one or two launches of the library's kernels)
        from einsummable_b200.memgraph import load_memgraph, memgraph_runner_t
        fixture = "llama7b_layer_locs1" if args.only.startswith("llama_layer") else "llama7b_train_l4_locs1"
        mg = load_memgraph(os.path.join(ROOT, "tests", "golden", "graphs", fixture + ".json.gz"))
        r = memgraph_runner_t(mg, devices=[0], fuse=args.only.endswith("fused"))
        rng = np.random.default_rng(7)
        for t in mg["inputs"]:
            shape, name = t["shape"], t["name"]
            if name == "freqs_cis":
                ang = np.outer(np.arange(shape[0]), 1.0 / (10000.0 ** (np.arange(shape[1]) / shape[1])))
                v = (np.cos(ang) + 1j * np.sin(ang)).astype(np.complex64)
            elif name.endswith("norm.weight"):
                v = np.ones(shape, dtype=np.float16)
            elif name == "labels":
                v = np.zeros(shape, dtype=np.float16)
                v[np.arange(shape[0]), rng.integers(0, shape[1], shape[0])] = 1.0
            else:
                v = (rng.standard_normal(shape).astype(np.float32) * 0.02).astype(np.float16)
            r.set_input(name, v)
        for _ in range(args.warmup):
            r.run(stream)
        torch.cuda.synchronize()
        ms = time_launches(lambda: r.run(stream), stream, iters=args.steps, warm=0)
        print(json.dumps({"only": args.only, "ms": ms, "launches_per_run": len(r.program), "nodes_folded": r.folded,
                          "nodes": dict(r.stats), "device_status": r.device_status()}))
        return
    if args.only == "move":
        # move_t between two GPUs driven by one process (the reference's server model):
        # source buffer on cuda:1, destination on cuda:0, through es_b200_move
        if torch.cuda.device_count() < 2:
            print(json.dumps({"only": "move", "skipped": "needs 2 visible GPUs"}))
            return
        res = {}
        for nbytes in (64 << 10, 1 << 20, 4 << 20, 16 << 20, 90 << 20, 512 << 20):
            src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda:1")
            dst = torch.zeros(nbytes, dtype=torch.uint8, device="cuda:0")
            torch.cuda.synchronize(1)
            ms = time_launches(lambda: km.move(1, src, dst, nbytes, stream), stream, iters=args.steps, warm=args.warmup)
            ok = bool((dst == src.to("cuda:0")).all().item())
            res["%d KiB" % (nbytes >> 10)] = {"ms": ms, "GB/s": nbytes / (ms * 1e-3) / 1e9, "bit_exact": ok}
        print(json.dumps({"only": "move", "path": "<=4 MiB: SM pull kernel over NVLink; larger: copy engine",
                          "reference_peer_copy_GB/s": 770, "sizes": res}))
        return
    if args.only.startswith("gemm") or args.only.startswith("attn"):
        if args.only == "gemm_qkv":
            e = einsummable_t.from_matmul_st(2048, 4096, 4096, "f16")
        elif args.only == "gemm_ffn":
            e = einsummable_t.from_matmul_st(2048, 4096, 11008, "f16")
        elif args.only == "gemm_f32":
            e = einsummable_t.from_matmul(2048, 2048, 2048, "f32")
        elif args.only == "gemm_nn":    # ij,jk->ik: the second operand's innermost mode is an output mode
            e = einsummable_t.from_str("ij,jk->ik", dict(i=2048, j=4096, k=4096), mul16, "add")
        elif args.only == "gemm_tn":    # ji,jk->ik: both are (the weight-gradient shape of a backward pass)
            e = einsummable_t.from_str("ji,jk->ik", dict(i=4096, j=2048, k=4096), mul16, "add")
        elif args.only == "attn_scores":
            e = einsummable_t.from_str("acbe,adbe->abcd", dict(a=4, b=32, c=512, d=512, e=128), mul16, "add")
        else:
            e = einsummable_t.from_str("abce,aebd->abcd", dict(a=4, b=32, c=512, d=128, e=512), mul16, "add")
        dt = torch.float16 if e.out_dtype() == "f16" else torch.float32
        ws = km.build(e)
        ins = [torch.randn(int(np.prod(e.inn_shape(k))), dtype=dt, device=dev) for k in range(2)]
        out = torch.empty(e.out_nelem(), dtype=dt, device=dev)
        w = torch.empty(max(ws, 16), dtype=torch.uint8, device=dev)
        fn = lambda: km(e, stream, out, ins, (w, ws) if ws else None)
        work, unit = 2.0 * float(np.prod(e.join_shape)), "TFLOP/s"
        nbytes = sum(t.numel() * t.element_size() for t in ins + [out])
        info = km.kernel_info(e)
    elif args.only == "touch":
        sel = [(16, 32, 0, 16, 16), (256, 512, 0, 256, 256), (16, 32, 0, 16, 16), (64, 128, 0, 64, 64)]
        src = torch.randn(16 * 256 * 16 * 64, dtype=torch.float16, device=dev)
        dst = torch.zeros(32 * 512 * 32 * 128, dtype=torch.float16, device=dev)
        t = touch_t(sel, "add", "f16")
        fn = lambda: km(t, stream, dst, src)
        work, unit, nbytes, info = 3.0 * src.numel() * 2, "GB/s", 3 * src.numel() * 2, "touch add f16 C3 p=2"
    else:
        e = einsummable_t([32, 32, 512, 128], [[0, 2, 1, 3]], 4, S.make_identity("f16"))
        km.build(e)
        src = torch.randn(32 * 512 * 32 * 128, dtype=torch.float16, device=dev)
        dst = torch.empty_like(src)
        fn = lambda: km(e, stream, dst, [src])
        work, unit, nbytes, info = 2.0 * src.numel() * 2, "GB/s", 2 * src.numel() * 2, km.kernel_info(e)
    ms = time_launches(fn, stream, iters=args.steps, warm=args.warmup)
    scale = 1e12 if unit == "TFLOP/s" else 1e9
    print(json.dumps({"only": args.only, "ms": ms, "value": work / (ms * 1e-3) / scale, "unit": unit,
                      "bytes": nbytes, "device_status": km.device_status(), "info": info}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows of the [rows, 11008] tensors (default: the full C2 workload); "
                         "smaller values are for profiler captures only")
    ap.add_argument("--only", default=None,
                    choices=["llama_layer", "llama_layer_fused", "llama_train", "llama_train_fused", "gemm_qkv", "gemm_ffn", "gemm_f32", "gemm_nn", "gemm_tn", "attn_scores", "attn_pv", "touch", "permute", "move"],
                    help="time one other kernel class alone (profiler captures); prints its own small JSON line")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end, other-class and CPU-baseline legs (profiler captures)")
    args = ap.parse_args()
    set_rows(args.rows)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.only:
        run_only(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
