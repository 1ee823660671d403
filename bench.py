#!/usr/bin/env python3
"""Benchmark of the B200 execution path for einsummable's memgraph apply nodes.

Headline (every N): the LLaMA-7B-shape transformer layer of BASELINE config 4 -- batch 4 x seq 512 =
2048 tokens, f16, seeded synthetic weights ~ N(0, 0.02) -- executed from the memgraph the reference's
own compilers produce for N locations (autoplace01), one process per GPU, moves over peer memory.
One step = one run of that graph (one CUDA-graph replay of the dependency-ordered schedule).
Metric: tokens/s = 2048 * steps / max-over-ranks device time; "scaling": "strong" (the same layer at
every N).  The saved `scores` of the timed configuration are checked against the CPU oracle's.

Also in the line: `e2e` (the step's input copied from pinned host memory and the result copied back
inside the timed region), `roofline` of the step's largest kernel plus one fraction per kernel class,
the BASELINE config 2 step (elementwise + reductions, GB/s), config 5 training graphs, and at N=1 the
CPU baseline.  `--impl reference` runs the same layer on the host cores through oracle/cpu_engine.py,
a restatement of the reference's CPU engine (its MKL executor cannot be built here).

Prints ONE JSON line on rank 0.
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

def profiled_traffic(key):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the committed table of ncu
    captures (profiles/traffic.json); None when that kernel was not captured."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get(key)


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


def measured_peaks_all():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


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


def cpu_layer_engine():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from cpu_engine import cpu_engine_t
    mg = load_layer_graph(1)
    eng = cpu_engine_t(mg, accumulate="f32", threads=os.cpu_count() or 1)
    for k, v in layer_inputs(mg).items():
        eng.set_input(k, v)
    return eng


CPU_SAMPLE = ("each step = the whole 1-location layer memgraph (2048 tokens) on the host cores: torch CPU einsum as the "
              "stand-in for cblas_sgemm, elementwise / reductions / touches with the reference CPU executor's conventions, "
              "nodes in memgraph order, every kernel on all cores")


def cpu_baseline(budget_s=15.0):
    """The same layer on this box's host cores (oracle/cpu_engine.py), a bounded number of passes."""
    eng = cpu_layer_engine()
    eng.run()
    t0 = time.perf_counter()
    passes = 0
    while True:
        eng.run()
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or passes >= 20:
            break
    res = {"value": LAYER_TOKENS * passes / dt, "unit": "tokens/s", "cores": eng.threads, "kind": "port",
           "sample": "%d passes, %.1f s; %s" % (passes, dt, CPU_SAMPLE),
           "contraction_TFLOP/s": eng.flops / (dt / passes) / 1e12}
    try:
        lib = load_cpu_oracle()
        other = cpu_other_classes(lib)
        sys.stderr.write("CPU port, other classes:\n%s\n" % json.dumps(other, indent=1))
        res["c2_step_GB/s"] = cpu_c2(lib)
    except Exception as exc:  # reported, never hidden
        res["other_error"] = repr(exc)[:200]
    return res


def cpu_c2(lib, budget_s=4.0):
    """BASELINE config 2 (all 8192 rows) through the C port's loops on the host cores."""
    bufs = cpu_buffers(ROWS)
    cpu_pass(lib, ROWS, *bufs)
    t0 = time.perf_counter()
    passes = 0
    while True:
        cpu_pass(lib, ROWS, *bufs)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s:
            break
    return round(cpu_bytes(ROWS) * passes / dt / 1e9, 2)


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
    """The reference's CPU implementation of the path on the host cores, same workload as the GPU
    arm: the whole layer memgraph per step.  The reference's MKL executor cannot be built here (no
    MKL; merge-conflict markers in src/engine/cpu/kernel_executor.cc:1323-1445), so this is the
    restatement in oracle/cpu_engine.py.  Under torchrun rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    eng = cpu_layer_engine()          # sets the thread count explicitly (torchrun exports OMP_NUM_THREADS=1)
    for _ in range(max(1, min(args.warmup, 2))):
        eng.run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        eng.run()
    dt = time.perf_counter() - t0
    value = LAYER_TOKENS * args.steps / dt
    want = golden_scores()
    got = eng.get_output("scores").astype(np.float64)
    parity = None if want is None else float(np.abs(got - want).max() / np.abs(want).max())
    print(json.dumps({
        "impl": "reference", "metric": "LLaMA-7B layer tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 math on f16 tensors",
        "data": "synthetic",
        "config": {"workload": LAYER_WORKLOAD, "tokens_per_step": LAYER_TOKENS, "sample": CPU_SAMPLE},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": eng.threads, "kind": "port", "sample": CPU_SAMPLE},
        "parity": {"max_abs_err_over_max_abs_vs_f64_oracle": parity},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
LAYER_FIXTURE = "llama7b_layer"
LAYER_WORKLOAD = ("C4 LLaMA-7B-shape transformer layer forward (dim 4096, 32 heads x 128, FFN 11008 SwiGLU, RMSNorm, "
                  "RoPE, causal attention, last-token vocabulary projection), batch 4 x seq 512 = 2048 tokens, f16, "
                  "the memgraph the reference's compilers emit for N locations (placement: see config.placement)")
LAYER_TOKENS = 2048


def layer_inputs(mg):
    """Seeded synthetic inputs of the layer graph (the same on every rank and in the golden fixture)."""
    from einsummable_b200.memgraph import synthetic_llama_inputs
    return synthetic_llama_inputs(mg, seed=7)


def load_layer_graph(world, fixture=LAYER_FIXTURE):
    from einsummable_b200.memgraph import load_memgraph
    path = os.path.join(ROOT, "tests", "golden", "graphs", "%s_locs%d.json.gz" % (fixture, world))
    if not os.path.exists(path):
        raise RuntimeError("no memgraph fixture of %s for %d locations" % (fixture, world))
    return load_memgraph(path)


def golden_scores():
    """`scores` of the layer for layer_inputs(), computed once by the CPU oracle with f64 accumulation
    (tests/golden/make_c4_full.py) and committed; None when the fixture is missing."""
    path = os.path.join(ROOT, "tests", "golden", "c4_full.npz")
    if not os.path.exists(path):
        return None
    return np.load(path)["scores"].astype(np.float64)


class Ranks:
    """torch.distributed plumbing of the bench: barrier, max over ranks, sum of a result."""
    def __init__(self):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        # the exchange uses plain peer loads and flags: no NVLink multicast objects, neither NCCL's nor
        # symmetric memory's (a rank that dies while bound to one disturbs the others)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max(self, v):
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_array(self, a):
        if self.world == 1:
            return a
        t = self.torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.dev)
        self.dist.all_reduce(t)
        return t.cpu().numpy()

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_steps(rk, stream, fn, steps):
    """ms per step of `steps` calls of fn: CUDA events on the launching stream, a barrier and a
    synchronise on both sides, max over ranks."""
    torch = rk.torch
    rk.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(stream)
    for _ in range(steps):
        fn()
    e.record(stream)
    rk.barrier()
    return rk.max(s.elapsed_time(e)) / steps


def make_runner(rk, mg, fuse, **kw):
    from einsummable_b200.memgraph import memgraph_runner_t
    if rk.world > 1:
        transport = os.environ.get("ES_B200_MOVE_TRANSPORT", "p2p")
        try:
            return memgraph_runner_t(mg, rank=rk.rank, world=rk.world, transport=transport, fuse=fuse,
                                     wait_limit_ms=int(os.environ.get("ES_B200_WAIT_LIMIT_MS", "2000")), **kw)
        except Exception as exc:
            if transport == "nccl":
                raise
            # peer-mapped (symmetric) memory could not be set up on this box -- every rank fails the same
            # way, at the same collective call -- : moves over NCCL send / recv, one stream in node order
            sys.stderr.write("peer-memory transport unavailable (%r); using NCCL send/recv\n" % (exc,))
            kw.pop("schedule", None)
            return memgraph_runner_t(mg, rank=rk.rank, world=rk.world, transport="nccl", fuse=fuse, **kw)
    return memgraph_runner_t(mg, devices=[rk.local], fuse=fuse, **kw)


def parity_of(rk, runner, want):
    """The saved `scores` of all ranks summed (every block has one owner) against the oracle's."""
    got = rk.sum_array(runner.get_output("scores").astype(np.float32)).astype(np.float64)
    if want is None:
        return {"ok": None, "note": "tests/golden/c4_full.npz missing"}
    scale = float(np.abs(want).max())
    err = float(np.abs(got - want).max())
    return {"max_abs_err_over_max_abs": err / scale, "tolerance": 1e-2, "ok": bool(err <= 1e-2 * scale),
            "against": "CPU oracle, f64-accumulated contractions, same seeded inputs (tests/golden/c4_full.npz)"}


def run_gpu(args):
    import torch
    import einsummable_b200 as es
    rk = Ranks()
    rank, world, dev = rk.rank, rk.world, rk.dev
    stream = torch.cuda.current_stream(dev)
    warmup = max(args.warmup, 3)
    peaks = measured_peaks_all()
    want = golden_scores()

    # ---------------- headline: the layer graph for `world` locations, one process per GPU ----------------
    # The headline is the graph the reference's autoplace01 gives for `world` locations (the configuration the
    # baseline names).  At N > 1 the same layer under the hand-written tensor-parallel placement
    # (tests/golden/make_tp_graphs.py; both graphs come out of the reference's own taskgraph and memgraph
    # compilers and give the same scores) is measured beside it in `config.variants`;
    # ES_B200_BENCH_PLACEMENT=tensor_parallel swaps the two.
    placement = "autoplace01"
    if world > 1 and os.environ.get("ES_B200_BENCH_PLACEMENT", "autoplace01") == "tensor_parallel":
        placement = "tensor_parallel"
    mg_auto = load_layer_graph(world)
    mg = mg_auto if placement == "autoplace01" else load_layer_graph(world, LAYER_FIXTURE + "_tp")
    inputs = layer_inputs(mg)
    r = make_runner(rk, mg, fuse=True)
    for k, v in inputs.items():
        r.set_input(k, v)
    c0 = r.km(rank if world > 1 else 0).counters()
    r.run(stream)
    torch.cuda.synchronize(dev)
    c1 = r.km(rank if world > 1 else 0).counters()
    launches_per_step = int(sum(c1[k] - c0[k] for k in c0))
    ms_eager = timed_steps(rk, stream, lambda: r.run(stream), 5)
    r.capture()
    for _ in range(warmup):
        r.replay(stream)
    sampler = ClockSampler(rk.local)
    if rank == 0:
        sampler.start()
    t_begin = time.perf_counter()
    ms = timed_steps(rk, stream, lambda: r.replay(stream), args.steps)
    t_end = time.perf_counter()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    status = int(rk.max(r.device_status()))
    parity = parity_of(rk, r, want)

    # the dominant kernel inside the step: the GPU's own timer read before and after every op of one replay
    try:
        tl, run_us = r.timeline(stream)
        units = r.units
    except Exception as exc:        # the NCCL fallback has no per-op timer
        sys.stderr.write("no per-op timeline: %r\n" % (exc,))
        tl, units = [], []
    dom = None
    for (cls, label, a, b), u in zip(tl, units):
        if cls == "contraction":
            node = r.mg["nodes"][u["node"]]
            flops = 2.0 * float(np.prod(node["einsummable"]["join_shape"]))
            if dom is None or flops > dom["flops"]:
                dom = {"flops": flops, "us": b - a, "label": label}
    by_class = {}
    for cls, _, a, b in tl:
        by_class[cls] = by_class.get(cls, 0.0) + (b - a)
    # the fused attention chains of this rank inside the step: Q, K, V read and O written once
    att = None
    att_ops = [(b - a, r.mg["nodes"][u["node"]]["attention"]) for (cls, _, a, b), u in zip(tl, units) if cls == "attention"]
    if att_ops:
        from einsummable_b200.attention import attention_t
        us = sum(t for t, _ in att_ops)
        nbytes = sum(attention_t.from_json(a).algorithmic_bytes() for _, a in att_ops)
        flops = sum(attention_t.from_json(a).flops() for _, a in att_ops)
        att = {"launches": len(att_ops), "us": round(us, 1), "algorithmic_MB": round(nbytes / 1e6, 1),
               "GB/s": round(nbytes / (us * 1e-6) / 1e9, 1), "frac_of_hbm": round(nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 3),
               "TFLOP/s_counting_every_key_block": round(flops / (us * 1e-6) / 1e12, 1),
               "replaces": "scores contraction, max, sum of exponentials, normalisation, contraction with V"}

    # ---------------- end to end: the step's input from pinned host memory, its result back to the host ----------------
    e2e = e2e_layer(rk, r, mg, inputs, stream, min(max(args.steps, 4), 50))

    # ---------------- the graph as the reference compiled it (nothing folded), and the old list schedule ----------------
    variants = {}
    r.close()
    del r
    torch.cuda.empty_cache()
    # (the other placement first: at N > 1 the autoplacer's graph when the headline is the tensor-parallel one,
    # and the other way round)
    other = "autoplace01" if placement == "tensor_parallel" else "tensor_parallel_placement"
    for name, kw in ((other, dict(fuse=True)),
                     ("autoplace01_folded_without_the_attention_kernel", dict(fuse="elementwise")),
                     ("autoplace01_as_compiled", dict(fuse=False)),
                     ("autoplace01_as_compiled_list_schedule", dict(fuse=False, schedule="list"))):
        try:
            if name.endswith("list_schedule") and os.environ.get("ES_B200_BENCH_LIST", "1") == "0":
                continue
            mgv = mg_auto
            if name == "tensor_parallel_placement":
                if world == 1:
                    continue
                mgv = load_layer_graph(world, LAYER_FIXTURE + "_tp")
            elif name == "autoplace01" and world == 1:
                continue
            rv = make_runner(rk, mgv, **kw)
            for k, v in layer_inputs(mgv).items() if mgv is not mg else inputs.items():
                rv.set_input(k, v)
            rv.capture()
            for _ in range(3):
                rv.replay() if kw.get("schedule") == "list" else rv.replay(stream)
            msv = timed_steps(rk, stream, (lambda: rv.replay()) if kw.get("schedule") == "list" else (lambda: rv.replay(stream)),
                              min(args.steps, 50))
            variants[name] = {"ms": round(msv, 4), "tokens/s": round(LAYER_TOKENS / (msv * 1e-3)),
                              "parity_ok": parity_of(rk, rv, want)["ok"], "device_status": int(rk.max(rv.device_status()))}
            rv.graph = None
            rv.close()
            del rv
            torch.cuda.empty_cache()
        except Exception as exc:  # reported, never hidden
            variants[name] = {"error": repr(exc)[:200]}

    # ---------------- other legs: rank 0's kernel classes (N=1), the C2 step, config 5 ----------------
    classes, c2 = {}, None
    km = es.kernel_manager_t(rk.local)
    if world == 1:
        try:
            c2 = c2_step_leg(km, dev, stream, peaks)
            classes = class_fractions(other_classes(km, dev, stream), c2, peaks)
        except Exception as exc:  # reported, never hidden
            classes = {"error": repr(exc)[:200]}
        torch.cuda.empty_cache()
    train = {}
    if os.environ.get("ES_B200_BENCH_TRAIN", "1") != "0":
        for name, fixture, runs in (("c5_shape_4layers_2048tok", "llama7b_train_l4", 5),
                                    ("c5_4layers_8192tok", "llama7b_train_b8s1024_l4", 3)):
            try:
                train[name] = train_leg(rk, fixture, runs, stream)
            except Exception as exc:  # reported, never hidden
                train[name] = {"error": repr(exc)[:200]}
    km.close()

    if rank != 0:
        rk.close()
        return
    peak_tc = peaks["bf16_tflops_sustained"]
    achieved = dom["flops"] / (dom["us"] * 1e-6) / 1e12 if dom else None
    line = {
        "metric": "LLaMA-7B layer tokens/s", "value": LAYER_TOKENS / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": LAYER_WORKLOAD, "tokens_per_step": LAYER_TOKENS,
                   "placement": ("the reference's autoplace01" if placement == "autoplace01" else
                                 "tensor-parallel by hand (residual stream over the sequence, projections over heads / "
                                 "hidden / vocabulary), compiled by the reference's taskgraph and memgraph compilers; "
                                 "the autoplace01 graph is in variants"),
                   "l2": "weights (405 MB) and activations exceed the 126 MB L2; no flush",
                   "execution": "one CUDA-graph replay per step (dependency-ordered lanes), elementwise chains "
                                "folded into their readers, every attention chain one kernel; eager %.3f ms" % ms_eager,
                   "attention": att,
                   "contraction_gflop_per_step": mg["taskgraph"]["contraction_flops"] / 1e9,
                   "moves_per_step": mg["taskgraph"].get("move"), "move_bytes_per_step": mg["taskgraph"].get("move_bytes"),
                   "variants": variants},
        "clocks": clocks,
        "parity": parity,
        "device_status": status,
        "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "tensor", "kernel": "tcgen05 contraction, largest of the step: " + (dom["label"][:80] if dom else "?"),
                     "achieved": achieved, "peak": peak_tc, "unit": "TFLOP/s", "frac": achieved / peak_tc if achieved else None,
                     "peak_kind": peaks["kind"] + " (cuBLAS bf16, sustained: the kernel is timed inside the step)",
                     "duration_us": dom["us"] if dom else None,
                     "duration_by": "GPU timer read before and after the op inside one replay of the step's graph",
                     "traffic": ffn_traffic(dom), "algorithmic_flops_per_launch": dom["flops"] if dom else None,
                     "step_us_by_class": {k: round(v, 1) for k, v in sorted(by_class.items())},
                     "classes": classes},
        "c2_step": c2,
        "train": train,
        "cpu_baseline": cpu_baseline() if world == 1 else None,
    }
    print(json.dumps(line))
    rk.close()


def ffn_traffic(dom):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the step's largest contraction, from
    the committed ncu summary (profiles/traffic.json: kernel label -> bytes); None when not captured."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if dom is None or not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f)
    for key, val in table.items():
        if key in dom["label"]:
            return val
    return None


def e2e_layer(rk, r, mg, inputs, stream, steps):
    """tokens/s through the public call with host buffers: every step's input (the token embeddings; the
    weights are the resident model) crosses PCIe from pinned host memory, the graph is replayed, and the step's
    result (`scores`) is read back into pinned host memory, all inside the timed region.  The input is
    double-buffered the way a serving loop would do it: the host-to-device copy of step k + 1 runs on a copy
    stream into a staging buffer while step k is replayed, and a device-to-device copy at the top of the step
    puts it where the graph reads it.  `serial_ms_per_step` is the same with the copy in line (no overlap)."""
    torch = rk.torch
    name = "embeddings" if any(t["name"] == "embeddings" for t in mg["inputs"]) else mg["inputs"][0]["name"]
    up = r.stage_input(name, inputs[name])
    down = r.stage_output("scores")
    h2d = sum(h.numel() * h.element_size() for h, _ in up)
    d2h = sum(h.numel() * h.element_size() for h, _ in down)

    def serial_step():
        for h, d in up:
            d.copy_(h, non_blocking=True)
        r.replay(stream)
        for h, d in down:
            h.copy_(d, non_blocking=True)
    for _ in range(3):
        serial_step()
    ms_serial = timed_steps(rk, stream, serial_step, steps)

    copy_stream = torch.cuda.Stream(device=rk.dev)
    staging = [torch.empty_like(d) for _, d in up]
    arrived, consumed = torch.cuda.Event(), torch.cuda.Event()
    consumed.record(stream)

    def step():
        copy_stream.wait_event(consumed)          # the staging buffer of the step before has been read
        with torch.cuda.stream(copy_stream):
            for (h, _), sbuf in zip(up, staging):
                sbuf.copy_(h, non_blocking=True)
            arrived.record(copy_stream)
        stream.wait_event(arrived)
        for (_, d), sbuf in zip(up, staging):
            d.copy_(sbuf, non_blocking=True)
        consumed.record(stream)
        r.replay(stream)
        for h, d in down:
            h.copy_(d, non_blocking=True)
    for _ in range(3):
        step()
    ms = timed_steps(rk, stream, step, steps)
    torch.cuda.synchronize(rk.dev)
    tot_h2d, tot_d2h = sum_int(rk, h2d), sum_int(rk, d2h)
    return {"value": LAYER_TOKENS / (ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": tot_h2d,
            "d2h_bytes_per_step": tot_d2h, "ms_per_step": ms, "serial_ms_per_step": ms_serial, "steps": steps,
            "what": "input `%s` from pinned host memory every step (its copy overlaps the step before: staging buffer + "
                    "copy stream), result `scores` back to pinned host memory; weights stay resident" % name}


def sum_int(rk, v):
    if rk.world == 1:
        return v
    t = rk.torch.tensor([float(v)], dtype=rk.torch.float64, device=rk.dev)
    rk.dist.all_reduce(t)
    return int(t.item())


def train_leg(rk, fixture, runs, stream):
    """Config 5: four layers forward, the log-softmax loss, backward and the weight update as the
    reference's trainer builds them (llama/gpu_train.cc:154-322); tokens/s of the CUDA-graph replay."""
    torch = rk.torch
    path = os.path.join(ROOT, "tests", "golden", "graphs", "%s_locs%d.json.gz" % (fixture, rk.world))
    if not os.path.exists(path):
        return {"skipped": "no memgraph fixture for %d locations" % rk.world}
    from einsummable_b200.memgraph import load_memgraph
    mg = load_memgraph(path)
    need = int(max(mg["mem_sizes"])) + (8 << 30)
    free = torch.cuda.mem_get_info(rk.dev)[0]
    if free < need:
        return {"skipped": "needs %.0f GB of device memory, %.0f GB free" % (need / 1e9, free / 1e9)}
    tokens = 2048
    for t in mg["inputs"]:
        if t["name"] == "embeddings":
            tokens = int(t["shape"][0]) * int(t["shape"][1])
    r = make_runner(rk, mg, fuse=True)
    for k, v in layer_inputs(mg).items():
        r.set_input(k, v)
    r.capture()
    r.replay(stream)
    ms = timed_steps(rk, stream, lambda: r.replay(stream), runs)
    out = {"tokens": tokens, "ms": round(ms, 3), "tokens/s": round(tokens / (ms * 1e-3)),
           "contraction_TFLOP/s": round(mg["taskgraph"]["contraction_flops"] / (ms * 1e-3) / 1e12, 1),
           "nodes_folded": r.folded, "device_status": int(rk.max(r.device_status()))}
    r.graph = None
    r.close()
    del r
    torch.cuda.empty_cache()
    return out


def c2_step_leg(km, dev, stream, peaks, steps=20):
    """BASELINE config 2: f16 [8192,11008] ~ N(0,1); silu(x)*y, row max, exp(x - rowmax), row sum through
    the C ABI on one stream; algorithmic GB/s of the step and of each kernel (CUDA events between them)."""
    import torch
    from einsummable_b200 import einsummable_t, scalarop_t as S
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
    g.manual_seed(1234)
    x = torch.randn(N, dtype=torch.float16, device=dev, generator=g)
    y = torch.randn(N, dtype=torch.float16, device=dev, generator=g)
    o_silu = torch.empty(N, dtype=torch.float16, device=dev)
    o_max = torch.empty(ROWS, dtype=torch.float16, device=dev)
    o_exp = torch.empty(N, dtype=torch.float16, device=dev)
    o_sum = torch.empty(ROWS, dtype=torch.float16, device=dev)

    def step(ev=None):
        calls = ((e_silu, o_silu, [x, y]), (e_max, o_max, [x]), (e_exp, o_exp, [x, o_max]), (e_sum, o_sum, [o_exp]))
        for i, (e, o, ins) in enumerate(calls):
            if ev is not None:
                ev[i].record(stream)
            km(e, stream, o, ins, wsarg)
        if ev is not None:
            ev[4].record(stream)
    for _ in range(3):
        step()
    torch.cuda.synchronize(dev)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
    for k in range(steps):
        step(ev[k])
    torch.cuda.synchronize(dev)
    per = [float(np.mean([ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(steps)])) for i in range(4)]
    ms = float(np.mean([ev[k][0].elapsed_time(ev[k][4]) for k in range(steps)]))
    peak = peaks["hbm_gbs"]
    names = ["silu_mul", "rowmax", "exp_sub", "rowsum"]
    nbytes = [BYTES_SILU_MUL, BYTES_ROWMAX, BYTES_EXP_SUB, BYTES_ROWSUM]
    return {"workload": WORKLOAD, "ms_per_step": round(ms, 4), "GB/s": round(BYTES_STEP / (ms * 1e-3) / 1e9, 1),
            "frac_of_hbm_peak": round(BYTES_STEP / (ms * 1e-3) / 1e9 / peak, 3),
            "per_kernel_frac": {n: round(b / (t * 1e-3) / 1e9 / peak, 3) for n, t, b in zip(names, per, nbytes)},
            "silu_mul_dram_traffic_per_launch": profiled_traffic("silu_mul f16 [8192,11008]") if ROWS == 8192 else None,
            "kernels": dict(zip(names, [km.kernel_info(e).split("|")[0] for e in ops]))}


def class_fractions(classes, c2, peaks):
    """{kernel class: fraction of its roofline} for the JSON line (the full per-case numbers go to stderr)."""
    sys.stderr.write("kernel classes (timed alone, 20 launches, CUDA events):\n%s\n" % json.dumps(classes, indent=1))
    tc, hbm = peaks["bf16_tflops"], peaks["hbm_gbs"]
    out = {}
    for name, v in classes.items():
        if "TFLOP/s" in v and "attn" not in name:
            f = v["TFLOP/s"] / (tc / 2 if "f32" in name else tc)
            key = "contraction f32 3xTF32 (of half the bf16 peak, counting 1 of the 3 MMAs)" if "f32" in name else "contraction f16"
            out[key] = round(max(out.get(key, 0.0), f), 3)
        elif "attn" in name:
            out["attention contraction (HBM bound) " + name.split()[1]] = round(v["GB/s"] / hbm, 3)
        elif name.startswith("touch C3 sweep"):
            key = "touch batched " + ("add" if " add " in name else "copy")
            out[key] = round(max(out.get(key, 0.0), v["GB/s"] / hbm), 3)
        elif name.startswith("permute"):
            out["permutation"] = round(v["GB/s"] / hbm, 3)
    if c2:
        out["elementwise (C2 silu*y, exp(x-max))"] = max(c2["per_kernel_frac"]["silu_mul"], c2["per_kernel_frac"]["exp_sub"])
        out["reduction (C2 row max / row sum, inside the step)"] = max(c2["per_kernel_frac"]["rowmax"], c2["per_kernel_frac"]["rowsum"])
        out["C2 step of 4 kernels"] = c2["frac_of_hbm_peak"]
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


def run_exchange_only(args):
    """Cross-GPU copy rates of the exchange ops, two ranks (torchrun --nproc-per-node 2): rank 1 reads
    from rank 0's peer-mapped buffer with the pull op and with a touch whose input is the peer's memory
    (one-op programs, `steps` launches, CUDA events; the ~13 us floor is the program launch itself)."""
    rk = Ranks()
    torch = rk.torch
    import torch.distributed._symmetric_memory as symm_mem
    import einsummable_b200 as es
    from einsummable_b200.einsummable import touch_t
    from einsummable_b200.program import program_t
    total = (512 << 20) + 4096
    buf = symm_mem.empty(total, dtype=torch.uint8, device=rk.dev)
    buf.copy_(torch.randint(0, 255, (total,), dtype=torch.uint8, device=rk.dev))
    torch.cuda.synchronize()
    hdl = symm_mem.rendezvous(buf, rk.dist.group.WORLD)
    peers = [int(p) for p in hdl.buffer_ptrs]
    rk.barrier()
    km = es.kernel_manager_t(rk.local)
    res = {}
    if rk.rank == 1:
        dst = torch.zeros(512 << 20, dtype=torch.uint8, device=rk.dev)
        stream = torch.cuda.current_stream()
        flag = peers[0] + (512 << 20)
        for nbytes in (64 << 10, 1 << 20, 2 << 20, 8 << 20, 32 << 20, 128 << 20, 512 << 20):
            for kind in ("pull", "remote touch"):
                p = program_t(km)
                if kind == "pull":
                    p.add_pull([(peers[0], dst.data_ptr(), nbytes, None, flag)])
                else:
                    n = nbytes // 2
                    p.add_touch(touch_t([(n, n, 0, 0, n)], None, "f16"), None, dst.data_ptr(), peers[0], done_flag=flag)
                p.finalize(1)
                p.set_workspace(dst, 0)
                iters = args.steps if nbytes <= (32 << 20) else max(args.steps // 4, 2)
                ms = time_launches(lambda: p.launch(stream), stream, iters=iters, warm=args.warmup)
                res["%s %d KiB" % (kind, nbytes >> 10)] = {"us": round(ms * 1e3, 1), "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1)}
                p.close()
    rk.barrier()
    # the last op copied the first 512 MiB of rank 0's buffer: send a checksum over NCCL and compare
    chk = buf[:512 << 20].view(torch.int64).sum().reshape(1) if rk.rank == 0 else torch.zeros(1, dtype=torch.int64, device=rk.dev)
    rk.dist.broadcast(chk, src=0)
    if rk.rank == 1:
        res["checksum_matches"] = bool(int(dst.view(torch.int64).sum().item()) == int(chk.item()))
    if rk.rank == 1:
        print(json.dumps({"only": "exchange", "reference_peer_copy_GB/s": 770, "device_status": km.device_status(),
                          "sizes": res}))
    rk.close()


def run_only(args):
    """One kernel class alone, `steps` launches after `warmup`, CUDA events."""
    if args.only == "exchange":
        return run_exchange_only(args)
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
    if args.only.startswith("gemm") or args.only.startswith("attn_"):
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
    elif args.only in ("attention", "attention_noskip"):
        # the fused chain at the layer's size: Q, K, V as [batch, row, head, dim], lower-triangular mask
        from einsummable_b200.attention import attention_t
        b_, h_, s_, d_ = 4, 32, 512, 128
        q, k, v = [(torch.randn(b_, s_, h_, d_, device=dev) * 0.5).half() for _ in range(3)]
        i_, j_ = torch.arange(s_, device=dev).unsqueeze(1), torch.arange(s_, device=dev).unsqueeze(0)
        mask = torch.where(i_ >= j_, 0.0, float("-inf")).half().contiguous()
        out = torch.empty(b_, h_, s_, d_, dtype=torch.float16, device=dev)
        st = [s_ * h_ * d_, d_, h_ * d_]
        a = attention_t(b_, h_, s_, s_, d_, st, st, st, [h_ * s_ * d_, s_ * d_, d_], s_, 1 if args.only == "attention" else 0, 0)
        fn = lambda: km.attention(a, stream, out, q, k, v, mask)
        work, unit, nbytes = float(a.algorithmic_bytes()), "GB/s", a.algorithmic_bytes()
        info = "attention_tc_f16 %s: %.1f GFLOP counting every key block" % (args.only, a.flops() / 1e9)
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows of the [rows, 11008] tensors (default: the full C2 workload); "
                         "smaller values are for profiler captures only")
    ap.add_argument("--only", default=None,
                    choices=["llama_layer", "llama_layer_fused", "llama_train", "llama_train_fused", "gemm_qkv", "gemm_ffn", "gemm_f32", "gemm_nn", "gemm_tn", "attn_scores", "attn_pv", "attention", "attention_noskip", "touch", "permute", "move", "exchange"],
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
