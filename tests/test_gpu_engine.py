"""The reference's own GPU engine on the boundary.

oracle/_ref/engine_parity (built by oracle/Makefile where the reference tree is present; the
binary travels with the working tree) is the reference's exec graph, exec nodes, stream pool,
workspace / group / buffer managers and event loop -- src/engine/exec_graph.cc, exec_state.cc,
gpu/exec_graph.cc, ... compiled unchanged -- linked with the drop-in kernel_manager_t instead of
the reference's cuTENSOR one.  It builds the memgraph in-process with the reference's compilers,
runs exec_state_t::event_loop on it and hands back the location buffer; the saved tensors are
compared with what the reference's interpreter computed for the same inputs (tests/golden/graphs).
The same binary then runs the same memgraph_t through gpu_program_t (einsummable_b200/host/gpu_program.*,
C++ host code over the C ABI's program executor) and hands back that buffer too."""
import json
import os
import subprocess

import numpy as np
import pytest

import es_oracle as O
from conftest import GOLDEN_DIR, GraphArrays, ROOT

pytestmark = pytest.mark.gpu
BIN = os.path.join(ROOT, "oracle", "_ref", "engine_parity")
ARR = GraphArrays()

CASES = [
    ("c1_n64_locs1", "c1:64:2:1"),
    ("llama_tiny_locs1", "llama:64:2:32:128:1:2:16:0"),
]


def run_engine(spec, tmp_path, inputs=None, iters=2, fold=False):
    if not os.path.exists(BIN):
        pytest.skip("oracle/_ref/engine_parity is not built (needs the reference tree at build time)")
    # first call: only to learn the layout the reference's compilers chose (memgraph.json)
    if inputs is not None:
        res = subprocess.run([BIN, spec, str(tmp_path), "0"], capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        with open(tmp_path / "memgraph.json") as f:
            mg = json.load(f)
        bufs = O.memgraph_place_inputs(mg, inputs)
        bufs[0][:int(mg["mem_sizes"][0])].tofile(tmp_path / "in.bin")
    res = subprocess.run([BIN, spec, str(tmp_path), str(iters)] + (["fold"] if fold else []),
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    with open(tmp_path / "memgraph.json") as f:
        mg = json.load(f)
    info = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])   # the engine prints, too
    out = np.fromfile(tmp_path / "out.bin", dtype=np.uint8)
    if os.path.exists(tmp_path / "out_program.bin"):
        info["out_program"] = np.fromfile(tmp_path / "out_program.bin", dtype=np.uint8)
    if os.path.exists(tmp_path / "out_folded.bin"):
        info["out_folded"] = np.fromfile(tmp_path / "out_folded.bin", dtype=np.uint8)
    return mg, info, out


@pytest.mark.parametrize("name,spec", CASES)
def test_reference_engine_runs_memgraphs_on_the_drop_in(name, spec, tmp_path):
    pre = name + "/in/"
    inputs = {k[len(pre):]: ARR[k] for k in ARR.files if k.startswith(pre)}
    mg, info, out = run_engine(spec, tmp_path, inputs)
    assert mg["num_locs"] == 1 and info["exec_nodes"] == len(mg["nodes"])
    got = O.memgraph_collect_outputs(mg, [np.concatenate([out, np.zeros(256, np.uint8)])])
    pre = name + "/out/"
    checked = 0
    for k in ARR.files:
        if not k.startswith(pre):
            continue
        ref = ARR[k]
        g = got[k[len(pre):]]
        scale = np.abs(ref.astype(np.float64)).max()
        err = np.abs(g.astype(np.float64) - ref.astype(np.float64)).max()
        assert err <= (2e-2 if ref.dtype == np.float16 else 1e-5) * scale, (name, k, err, scale)
        checked += 1
    assert checked >= 1
    # the same memgraph_t through gpu_program_t (C++ host code only: the library's dependency-ordered
    # program instead of the event loop) gives the same saved tensors
    got2 = O.memgraph_collect_outputs(mg, [np.concatenate([info.pop("out_program"), np.zeros(256, np.uint8)])])
    assert info["program_ops"] > 0
    for k in ARR.files:
        if k.startswith(pre):
            ref = ARR[k]
            scale = np.abs(ref.astype(np.float64)).max()
            err = np.abs(got2[k[len(pre):]].astype(np.float64) - ref.astype(np.float64)).max()
            assert err <= (2e-2 if ref.dtype == np.float16 else 1e-5) * scale, ("program", name, k, err, scale)
    print(name, info)


def test_reference_engine_llama7b_layer_times(tmp_path):
    """The LLaMA-7B-shape layer (config 4) through the reference's event loop (one
    cudaStreamAddCallback round trip per node, 5 streams): every node builds and runs; the time per
    event loop is printed next to what the library's own schedule needs (see bench.py)."""
    mg, info, out = run_engine("llama:4096:32:256:32000:1:4:512:0", tmp_path, None, iters=5)
    assert info["exec_nodes"] == len(mg["nodes"])
    loops = info["event_loop_ms"]
    info.pop("out_program", None)
    print("reference engine on the drop-in, LLaMA-7B layer: build %.0f ms, event loops %s ms" % (info["build_ms"], loops))
    print("the same memgraph_t through gpu_program_t (C++ host): %d ops, eager %s ms, CUDA-graph replay %s ms"
          % (info["program_ops"], info["program_eager_ms"], info["program_replay_ms"]))
    assert min(loops) < 50.0
    # host wall clock incl. the synchronise: the program must beat the callback-driven loop clearly
    assert min(info["program_replay_ms"]) < 0.5 * min(loops)


def test_cpp_host_folds_and_runs_the_tiny_layer(tmp_path):
    """C++ host code alone: the memgraph_t folded by einsummable_b200/host/gpu_fuse.h (elementwise nodes into
    their readers, the attention chain into one node) and run by gpu_program_t -- the saved tensors against the
    reference interpreter's, at the tolerance of the graph as compiled."""
    name, spec = CASES[1]
    pre = name + "/in/"
    inputs = {k[len(pre):]: ARR[k] for k in ARR.files if k.startswith(pre)}
    mg, info, _ = run_engine(spec, tmp_path, inputs, fold=True)
    assert info["nodes_folded"] > 20 and info["attention_chains"] == 1
    assert 0 < info["folded_ops"] < info["program_ops"]
    # the same folded graph through gpu_exchange_program_t (units and order of service from gpu_exchange_plan.h;
    # one location: no exchange ops): the same kernels on the same data, so the same bits
    assert info["exchange_program_ops"] == info["folded_ops"]
    assert info["exchange_program_vs_folded_max_abs_diff"] == 0
    got = O.memgraph_collect_outputs(mg, [np.concatenate([info.pop("out_folded"), np.zeros(256, np.uint8)])])
    info.pop("out_program", None)
    pre = name + "/out/"
    checked = 0
    for k in ARR.files:
        if k.startswith(pre):
            ref = ARR[k]
            scale = np.abs(ref.astype(np.float64)).max()
            err = np.abs(got[k[len(pre):]].astype(np.float64) - ref.astype(np.float64)).max()
            assert err <= (2e-2 if ref.dtype == np.float16 else 1e-5) * scale, ("folded", k, err, scale)
            checked += 1
    assert checked >= 1
    print(name, info)


def test_cpp_host_folds_and_runs_the_llama7b_layer(tmp_path):
    """The same at full size (the buffer filled with small random f16 values): the folded graph's saved scores
    against the unfolded graph's from the same inputs, and the time of its CUDA-graph replay from C++."""
    mg, info, _ = run_engine("llama:4096:32:256:32000:1:4:512:0", tmp_path, None, iters=5, fold=True)
    info.pop("out_program", None)
    info.pop("out_folded", None)
    print("LLaMA-7B layer from C++ host code: as compiled %d ops, replay %s ms; folded %d ops (%d nodes folded, %d attention "
          "chain), replay %s ms" % (info["program_ops"], info["program_replay_ms"], info["folded_ops"], info["nodes_folded"],
                                    info["attention_chains"], info["folded_replay_ms"]))
    assert info["attention_chains"] == 1 and info["saved_finite"] and info["saved_max_abs"] > 0
    assert info["folded_vs_program_max_abs_diff"] <= 1e-2 * info["saved_max_abs"]
    assert min(info["folded_replay_ms"]) < min(info["program_replay_ms"])
    assert info["exchange_program_ops"] == info["folded_ops"]
    assert 0 <= info["exchange_program_vs_folded_max_abs_diff"] <= 1e-3 * info["saved_max_abs"]
