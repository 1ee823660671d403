"""Graph level on the GPU: the reference's memgraphs (tests/golden/graphs, written
by the reference's own compilers) run node by node through the C ABI and compared
with (a) the executor-convention oracle and (b) the results of the reference's own
interpreter.  Memgraphs with several locations run here with every location as a
separate buffer on cuda:0, so moves, grouped touches and fills are all exercised on
one GPU."""
import gzip
import json
import os

import numpy as np
import pytest
import torch

import es_oracle as O
from conftest import GOLDEN_DIR, GraphArrays
from einsummable_b200.memgraph import load_memgraph, memgraph_runner_t

pytestmark = pytest.mark.gpu
GRAPHS = os.path.join(GOLDEN_DIR, "graphs")
ARR = GraphArrays()
SMALL = ["c1_n64_locs1", "c1_n64_locs2", "llama_tiny_locs1", "llama_tiny_locs2", "llama_tiny_locs4", "llama_tiny_tp_locs2", "llama_tiny_tp_locs4",
         "llama_train_tiny_locs1", "llama_train_tiny_locs2", "llama_train_adamw_tiny_locs1",
         "llama_train_adamw_tiny_locs2", "llama_train_lora_tiny_locs1", "llama_train_lora_tiny_locs2"]


def graph_path(name):
    path = os.path.join(GRAPHS, name + ".json")
    return path if os.path.exists(path) else path + ".gz"


def inputs_of(name):
    pre = name + "/in/"
    return {k[len(pre):]: ARR[k] for k in ARR.files if k.startswith(pre)}


def outputs_of(name):
    pre = name + "/out/"
    return {k[len(pre):]: ARR[k] for k in ARR.files if k.startswith(pre)}


@pytest.mark.parametrize("schedule", ["dag", "list"])
@pytest.mark.parametrize("name", SMALL)
def test_small_memgraphs_match_oracle_and_reference(name, schedule):
    """schedule "dag": the library's program executor (dependency-ordered lanes); "list": one
    stream in node order."""
    mg = load_memgraph(graph_path(name))
    ins = inputs_of(name)
    r = memgraph_runner_t(mg, schedule=schedule)
    assert (r.prog is not None) == (schedule == "dag")
    for k, v in ins.items():
        r.set_input(k, v)
    r.run()
    torch.cuda.synchronize()
    assert r.device_status() == 0
    bufs = O.memgraph_place_inputs(mg, ins)
    O.run_memgraph(mg, bufs, "executor")
    oracle = O.memgraph_collect_outputs(mg, bufs)
    for k, ref in outputs_of(name).items():
        got = r.get_output(k)
        f16 = ref.dtype == np.float16
        scale = np.abs(ref.astype(np.float64)).max()
        err_oracle = np.abs(got.astype(np.float64) - oracle[k].astype(np.float64)).max()
        err_ref = np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()
        # backward pass: gradients that are small differences of large sums move by 1e-5 of their
        # own scale with the summation order alone, hence 1e-4 for the training graphs (f32)
        tol32 = 1e-4 if name.startswith("llama_train") else 1e-5
        assert err_oracle <= (1e-2 if f16 else tol32) * scale, (name, k, err_oracle, scale)
        assert err_ref <= (2e-2 if f16 else tol32) * scale, (name, k, err_ref, scale)
    # a second run of the same program gives the same bits (groups reset per run)
    first = {k: r.get_output(k).copy() for k in outputs_of(name)}
    r.run()
    torch.cuda.synchronize()
    for k, v in first.items():
        assert r.get_output(k).tobytes() == v.tobytes()
    # and so does the replay of the run captured as one CUDA graph
    r.capture()
    r.replay()
    r.replay()
    torch.cuda.synchronize()
    assert r.device_status() == 0
    for k, v in first.items():
        assert r.get_output(k).tobytes() == v.tobytes()
    if schedule == "dag":
        prof = r.profile()
        torch.cuda.synchronize()
        assert len(prof) == len(r.units) and all(t >= 0 for _, _, t in prof)
        for k, v in first.items():
            assert r.get_output(k).tobytes() == v.tobytes()
    r.close()


@pytest.mark.parametrize("nlocs", [1, 2, 8])
def test_c1_full_size(nlocs):
    """Config 1 at full size: ij,jk->ik f32 4096^3, 2x2x2 blocks with touch
    accumulation of the partial sums, against an f64 matmul."""
    mg = load_memgraph(os.path.join(GRAPHS, "c1_n4096_locs%d.json.gz" % nlocs))
    rng = np.random.default_rng(99)
    a = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    b = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    r = memgraph_runner_t(mg)
    r.set_input("lhs", a)
    r.set_input("rhs", b)
    r.run()
    torch.cuda.synchronize()
    assert r.device_status() == 0
    got = r.get_output("out")
    want = (torch.from_numpy(a).double() @ torch.from_numpy(b).double()).numpy()
    scale = np.abs(want).max()
    assert np.abs(got.astype(np.float64) - want).max() <= 1e-5 * scale
    r.close()


FULL = np.load(os.path.join(GOLDEN_DIR, "c4_full.npz"))


@pytest.mark.parametrize("nlocs,fuse", [(1, False), (1, "elementwise"), (1, True), (8, False), (8, True), ("tp_locs8", True)])
def test_llama7b_layer_full_size_against_the_cpu_oracle(nlocs, fuse):
    """Config 4 at full size (2048 tokens, dim 4096, FFN 11008, vocabulary 32000): the reference's
    memgraph for 1 and for 8 locations (all on this GPU), as compiled, with elementwise chains
    folded, and with the attention chains as one kernel on top of that (fuse=True), against the
    scores of the CPU oracle with f64-accumulated contractions
    (tests/golden/make_c4_full.py).  f16 tolerance 1e-2 of the largest score."""
    from einsummable_b200.memgraph import synthetic_llama_inputs
    if nlocs == "tp_locs8":     # the hand-written tensor-parallel placement (tests/golden/make_tp_graphs.py)
        mg, nlocs = load_memgraph(os.path.join(GRAPHS, "llama7b_layer_tp_locs8.json.gz")), 8
    else:
        mg = load_memgraph(os.path.join(GRAPHS, "llama7b_layer_locs%d.json.gz" % nlocs))
    r = memgraph_runner_t(mg, fuse=fuse)
    # one attention chain per block of heads and rows: all of them are found
    assert r.attention_chains == (nlocs if fuse is True else 0)
    assert r.kernel_kinds().get("attention_tc_f16", 0) == r.attention_chains
    for k, v in synthetic_llama_inputs(mg, seed=7).items():
        r.set_input(k, v)
    r.run()
    torch.cuda.synchronize()
    assert r.device_status() == 0
    got = r.get_output("scores").astype(np.float64)
    want = FULL["scores"].astype(np.float64)
    assert got.shape == (4, 32000)
    scale = np.abs(want).max()
    err = np.abs(got - want).max()
    print("nlocs", nlocs, "fuse", fuse, "max err / max |score| = %.2e" % (err / scale))
    assert err <= 1e-2 * scale
    first = got.copy()
    r.capture()
    r.replay()
    torch.cuda.synchronize()
    assert r.get_output("scores").astype(np.float64).tobytes() == first.tobytes()
    if nlocs == 1 and not fuse:
        kinds = r.kernel_kinds()
        print(kinds)
        assert kinds.get("contraction_tc_f16", 0) >= 10   # every contraction of the layer is on the tensor cores
    r.close()


@pytest.mark.parametrize("fuse", [False, True])
def test_llama7b_training_graph_full_size_loss(fuse):
    """Config 5's shape at 2048 tokens (4 layers forward, loss, backward, update; 512 einsummables):
    the per-sequence loss against the CPU oracle's."""
    from einsummable_b200.memgraph import synthetic_llama_inputs
    mg = load_memgraph(os.path.join(GRAPHS, "llama7b_train_l4_locs1.json.gz"))
    r = memgraph_runner_t(mg, fuse=fuse)
    for k, v in synthetic_llama_inputs(mg, seed=7).items():
        r.set_input(k, v)
    r.run()
    torch.cuda.synchronize()
    assert r.device_status() == 0
    got = r.get_output("loss").astype(np.float64).reshape(-1)
    want = FULL["train/loss"]
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max(), (got, want)
    r.close()


@pytest.mark.parametrize("name", ["llama_tiny_locs1", "llama_train_tiny_locs1", "llama_train_adamw_tiny_locs1",
                                  "llama_train_lora_tiny_locs1", "llama_tiny_tp_locs2", "llama_tiny_tp_locs4"])
def test_fused_memgraphs_match_reference(name):
    """Elementwise producers folded into their readers (einsummable_b200/fuse.py): every fused
    join goes through the same code generator; results against the reference interpreter's."""
    mg = load_memgraph(graph_path(name))
    r = memgraph_runner_t(mg, fuse=True)
    assert r.folded > 0
    # the forward graph's attention runs as the fused kernel (head dim 32 inside a 64-wide tile); the
    # training graphs keep the softmax result for the backward pass
    # (the tensor-parallel fixtures: one chain per location, on its own heads, all locations on this GPU)
    assert r.attention_chains == {"llama_tiny_locs1": 1, "llama_tiny_tp_locs2": 2, "llama_tiny_tp_locs4": 4}.get(name, 0)
    for k, v in inputs_of(name).items():
        r.set_input(k, v)
    r.run()
    torch.cuda.synchronize()
    assert r.device_status() == 0
    for k, ref in outputs_of(name).items():
        got = r.get_output(k)
        scale = np.abs(ref.astype(np.float64)).max()
        err = np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()
        assert err <= (2e-2 if ref.dtype == np.float16 else 1e-4) * scale, (name, k, err, scale)
    r.close()


def test_llama7b_layer_fused_agrees_with_unfused():
    mg = load_memgraph(os.path.join(GRAPHS, "llama7b_layer_locs1.json.gz"))
    outs = []
    for fuse in (False, True):
        r = memgraph_runner_t(mg, fuse=fuse)
        rng = np.random.default_rng(0)
        for t in mg["inputs"]:
            shape, name = t["shape"], t["name"]
            if name == "freqs_cis":
                seq, half = shape
                ang = np.outer(np.arange(seq), 1.0 / (10000.0 ** (np.arange(half) / half)))
                v = (np.cos(ang) + 1j * np.sin(ang)).astype(np.complex64)
            elif name.endswith("norm.weight"):
                v = np.ones(shape, dtype=np.float16)
            else:
                v = (rng.standard_normal(shape).astype(np.float32) * 0.02).astype(np.float16)
            r.set_input(name, v)
        r.run()
        torch.cuda.synchronize()
        assert r.device_status() == 0
        outs.append(r.get_output("scores").astype(np.float64))
        if fuse:
            assert r.folded >= 15
        r.close()
    scale = np.abs(outs[0]).max()
    # f16 graph: the folded intermediates are no longer rounded to f16 (1e-2 of the output scale)
    assert np.abs(outs[0] - outs[1]).max() <= 1e-2 * scale


EVICT = np.load(os.path.join(GRAPHS, "graphs_evict.npz"))


@pytest.mark.parametrize("name", ["c1_n64_evict_locs1", "c1_n64_evict_locs2"])
def test_memgraphs_with_evict_and_load(name):
    """Memgraphs the reference compiled under a memory limit: 40 evicts, 50 loads and 20 inputs that
    start out in storage.  Every storage id has a fixed block of one pinned host arena; evict / load
    are copy ops of the dependency-ordered schedule.  Against the reference's
    reference_compute_memgraph with storage."""
    mg = load_memgraph(graph_path(name))
    r = memgraph_runner_t(mg)
    assert sum(1 for u in r.units if u["kind"] == "evict") > 30 and sum(1 for u in r.units if u["kind"] == "load") > 40
    pre = name + "/in/"
    for k in EVICT.files:
        if k.startswith(pre):
            r.set_input(k[len(pre):], EVICT[k])
    ref = EVICT[name + "/out/out"]
    for attempt in range(2):
        r.run()
        torch.cuda.synchronize()
        assert r.device_status() == 0
        got = r.get_output("out")
        assert np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() <= 1e-5 * np.abs(ref).max()
        # inputs that started in storage were consumed (loaded and overwritten): put them back for the next run
        for k in EVICT.files:
            if k.startswith(pre):
                r.set_input(k[len(pre):], EVICT[k])
    r.capture()                 # (its warm-up runs consume the inputs once more)
    for k in EVICT.files:
        if k.startswith(pre):
            r.set_input(k[len(pre):], EVICT[k])
    r.replay()
    torch.cuda.synchronize()
    got = r.get_output("out")
    assert np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() <= 1e-5 * np.abs(ref).max()
    r.close()


def test_storage_evict_load_through_the_c_abi():
    """es_b200_storage_* / es_b200_evict / es_b200_load: the dynamic form (ids reserved and released
    at run time, as gpu_storage_t does).  Bit-exact round trips, id reuse after a load, errors."""
    import ctypes
    import einsummable_b200 as es
    from einsummable_b200 import _lib
    lib = _lib.load()
    km = es.kernel_manager_t(0)
    sto = ctypes.c_void_p()
    _lib.check(lib.es_b200_storage_create(1 << 20, 0, ctypes.byref(sto)))
    x = torch.randn(65536, device="cuda:0")          # 256 KiB
    y = torch.zeros_like(x)
    stream = torch.cuda.current_stream().cuda_stream
    for rep in range(8):                              # 8 x 256 KiB through a 1 MiB arena: blocks must be reused
        _lib.check(lib.es_b200_evict(km._h, sto, 7, x.data_ptr(), x.numel() * 4, stream))
        _lib.check(lib.es_b200_evict(km._h, sto, 8 + rep, x.data_ptr(), 1024, stream))
        _lib.check(lib.es_b200_load(km._h, sto, 7, y.data_ptr(), y.numel() * 4, stream))
        torch.cuda.synchronize()
        assert torch.equal(x, y)
        y.zero_()
        host = np.zeros(256, np.float32)
        _lib.check(lib.es_b200_storage_read(sto, 8 + rep, host.ctypes.data_as(ctypes.c_void_p), 1024))
        assert host.tobytes() == x[:256].cpu().numpy().tobytes()
        _lib.check(lib.es_b200_storage_remove(sto, 8 + rep))
    # host-side write, then load
    w = np.arange(1024, dtype=np.float32)
    _lib.check(lib.es_b200_storage_write(sto, 3, w.ctypes.data_as(ctypes.c_void_p), 4096))
    _lib.check(lib.es_b200_load(km._h, sto, 3, y.data_ptr(), 4096, stream))
    torch.cuda.synchronize()
    assert y[:1024].cpu().numpy().tobytes() == w.tobytes()
    # errors: unknown id, id in use, wrong size, out of space
    assert lib.es_b200_load(km._h, sto, 3, y.data_ptr(), 4096, stream) == _lib.ES_BAD_ARGUMENT
    _lib.check(lib.es_b200_evict(km._h, sto, 5, x.data_ptr(), 1024, stream))
    assert lib.es_b200_evict(km._h, sto, 5, x.data_ptr(), 1024, stream) == _lib.ES_BAD_ARGUMENT
    assert lib.es_b200_load(km._h, sto, 5, y.data_ptr(), 2048, stream) == _lib.ES_BAD_ARGUMENT
    assert lib.es_b200_evict(km._h, sto, 6, x.data_ptr(), 2 << 20, stream) == _lib.ES_WORKSPACE_TOO_SMALL
    torch.cuda.synchronize()
    _lib.check(lib.es_b200_storage_destroy(sto))
    km.close()


def test_nvtx_ranges_are_opt_in_and_harmless():
    """ES_B200_NVTX=1: every launch and program op pushes / pops a named NVTX range (nothing listens here:
    the run must simply behave as before)."""
    import subprocess
    import sys
    code = (
        "import numpy as np, torch\n"
        "from einsummable_b200.memgraph import load_memgraph, memgraph_runner_t\n"
        "mg = load_memgraph(%r)\n"
        "r = memgraph_runner_t(mg)\n"
        "rng = np.random.default_rng(0)\n"
        "for t in mg['inputs']:\n"
        "    r.set_input(t['name'], rng.uniform(-1, 1, t['shape']).astype(np.float32))\n"
        "r.run(); torch.cuda.synchronize()\n"
        "assert r.device_status() == 0\n"
        "print('ok', float(np.abs(r.get_output(mg['outputs'][0]['name'])).max()))\n"
    ) % graph_path("c1_n64_locs1")
    env = dict(os.environ, ES_B200_NVTX="1")
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=root, timeout=300)
    assert res.returncode == 0 and res.stdout.startswith("ok"), res.stdout[-500:] + res.stderr[-2000:]
