"""The C++ fold of elementwise nodes into their readers (einsummable_b200/host/gpu_fuse.h, compiled
against the reference's memgraph_t into oracle/_ref/libes_ref.so) on memgraphs the reference's compilers
build in-process:

  * against the Python pass (einsummable_b200/fuse.py: fuse_elementwise_chains) node by node -- the same
    nodes folded away, the same dependencies, memory regions, index maps and (after the reference's own
    parser has normalised both) the same join;
  * through the reference's interpreter: the folded graph, which is again a memgraph_t, gives the results of
    the graph as compiled."""
import ctypes
import json
import os
import sys

import numpy as np
import pytest

from conftest import ROOT
from einsummable_b200 import fuse as F

sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

LIB = os.path.join(ROOT, "oracle", "_ref", "libes_ref.so")
u64 = ctypes.c_uint64


def _lib():
    if not os.path.exists(LIB):
        pytest.skip("the reference has not been compiled here (oracle/_ref)")
    lib = ctypes.CDLL(LIB)
    if not hasattr(lib, "ref_graph_fold_elementwise"):
        pytest.skip("oracle/_ref/libes_ref.so predates the C++ fold")
    lib.ref_graph_last_error.restype = ctypes.c_char_p
    lib.ref_last_error.restype = ctypes.c_char_p
    return lib


CASES = {
    "tiny llama, 1 location": lambda L: L.ref_graph_build_llama(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 1, 0),
    "tiny llama, autoplace01, 2 locations": lambda L: L.ref_graph_build_llama(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 2, 0),
    "tiny llama, tensor-parallel, 4 locations": lambda L: L.ref_graph_build_llama_tp(u64(64), u64(4), u64(32), u64(128), 1, u64(2), u64(16), 4, 0),
    "tiny training graph, 2 locations": lambda L: L.ref_graph_build_llama_train(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 2, 1,
                                                                                 ctypes.c_double(0.01), 1, 0, 0),
}

# full size: structure only (the reference's interpreter would take hours)
LARGE = {
    "LLaMA-7B layer, tensor-parallel, 8 locations": lambda L: L.ref_graph_build_llama_tp(u64(4096), u64(32), u64(256), u64(32000), 1, u64(4),
                                                                                          u64(512), 8, 0),
    "LLaMA-7B layer, autoplace01, 2 locations": lambda L: L.ref_graph_build_llama(u64(4096), u64(32), u64(256), u64(32000), 1, u64(4),
                                                                                  u64(512), 2, 0),
}


def _json(L, h, path):
    assert L.ref_graph_write_json(h, path.encode()) >= 0, L.ref_graph_last_error().decode()
    with open(path) as f:
        return json.load(f)


def _fold(L, case, tmp_path):
    h = {**CASES, **LARGE}[case](L)
    assert h >= 0, L.ref_graph_last_error().decode()
    n = ctypes.c_int(0)
    hf = L.ref_graph_fold_elementwise(h, ctypes.byref(n))
    assert hf >= 0, L.ref_graph_last_error().decode()
    return h, hf, n.value, _json(L, h, str(tmp_path / "mg.json")), _json(L, hf, str(tmp_path / "folded.json"))


@pytest.mark.parametrize("case", list(CASES) + list(LARGE))
def test_cpp_fold_is_the_python_fold(case, tmp_path):
    L = _lib()
    _, _, n_folded, mg, got = _fold(L, case, tmp_path)
    want, want_folded = F.fuse_elementwise_chains(mg)
    assert n_folded == want_folded and n_folded > 0
    assert len(got["nodes"]) == len(want["nodes"])
    seen = {}

    def normal(text):
        if text not in seen:
            buf = ctypes.create_string_buffer(1 << 16)
            assert L.ref_scalarop_info(text.encode(), buf, len(buf)) == 0, L.ref_last_error().decode()
            seen[text] = buf.value.decode()   # the text as parsed and printed back, then its other forms
        return seen[text]

    composed = 0
    for g, w in zip(got["nodes"], want["nodes"]):
        assert g["id"] == w["id"]
        assert sorted(g["inns"]) == sorted(w["inns"]), (case, g["id"])
        if w.get("folded"):
            assert g["kind"] == "alloc", (case, g["id"], g["kind"])
            continue
        assert g["kind"] == w["kind"], (case, g["id"])
        if g["kind"] != "apply" or "einsummable" not in w:
            continue
        assert g["mems"] == w["mems"], (case, g["id"])
        ge, we = g["einsummable"], w["einsummable"]
        for key in ("join_shape", "inns", "out_rank", "castable"):
            assert ge[key] == we[key], (case, g["id"], key, ge, we)
        if ge["join"] != we["join"]:
            assert normal(ge["join"]) == normal(we["join"]), (case, g["id"], ge["join"], we["join"])
        composed += len(w["mems"]) != len(mg["nodes"][w["id"]]["mems"]) or we["join"] != mg["nodes"][w["id"]]["einsummable"]["join"]
    assert composed > 0


@pytest.mark.parametrize("case", [c for c in CASES if "autoplace01" not in c and "1 location" not in c])
def test_cpp_folded_graph_through_the_reference_interpreter(case, tmp_path):
    import make_graphs as G
    L = _lib()
    h, hf, _, mg, folded = _fold(L, case, tmp_path)
    G.L = L
    rng = np.random.default_rng(11)
    ins = G.llama_inputs(mg, rng, 0.1) if any(t["name"] == "embeddings" for t in mg["inputs"]) else None
    assert ins is not None
    if "labels" in ins:                       # one-hot rows, as the loss expects them
        labels = np.zeros(ins["labels"].shape, dtype=ins["labels"].dtype)
        labels[np.arange(labels.shape[0]), (np.arange(labels.shape[0]) * 37 + 5) % labels.shape[1]] = 1.0
        ins["labels"] = labels
    want = G.run_reference(h, mg, ins)
    got = G.run_reference(hf, folded, ins)
    assert set(got) == set(want) and want
    for k in want:
        # every to_f16 / to_f32 of a chain stays in the folded join, and the interpreter evaluates the
        # join point by point: the same roundings in the same order, so the same bits
        assert np.isfinite(got[k].astype(np.float64)).all(), k
        assert np.array_equal(got[k], want[k]), (case, k)


n_chains = {}


@pytest.mark.parametrize("case", list(CASES) + list(LARGE))
def test_cpp_attention_fold_is_the_python_one(case, tmp_path):
    """es_fuse::fold_attention on the C++-folded graph against fuse_attention on the Python-folded one: the
    same chains, the same descriptor (strides, and the lower-triangular mask recognised through the row-block
    copies and moves in front of it), the same five memories, the same dependencies on every node."""
    L = _lib()
    if not hasattr(L, "ref_graph_fold_attention"):
        pytest.skip("oracle/_ref/libes_ref.so predates the attention fold")
    _, hf, _, mg, _ = _fold(L, case, tmp_path)
    apath = str(tmp_path / "attention.json")
    ha = L.ref_graph_fold_attention(hf, apath.encode())
    assert ha >= 0, L.ref_graph_last_error().decode()
    with open(apath) as f:
        found = json.load(f)
    got = _json(L, ha, str(tmp_path / "attn_graph.json"))
    want, chains = F.fuse_attention(F.fuse_elementwise_chains(mg)[0])
    assert chains == len(found)
    n_chains[case] = chains
    for g, w in zip(got["nodes"], want["nodes"]):
        assert sorted(g["inns"]) == sorted(w["inns"]), (case, g["id"])
        if "attention" in w:
            a = found[str(w["id"])]
            assert a["attention"] == w["attention"], (case, w["id"], a["attention"], w["attention"])
            assert a["mems"] == w["mems"] and g["mems"] == w["mems"] and a["loc"] == w["loc"], (case, w["id"])
        elif w.get("folded"):
            assert g["kind"] == "alloc", (case, g["id"])
        else:
            assert g["kind"] == w["kind"], (case, g["id"])
    if "training" not in case:
        assert all(a["attention"]["skip_known"] == 1 for a in found.values())


def test_cpp_attention_fold_found_chains():
    if not n_chains:
        pytest.skip("the cases above did not run")
    assert sum(n_chains.values()) >= 3, n_chains


@pytest.mark.parametrize("case", ["tiny llama, tensor-parallel, 4 locations", "tiny training graph, 2 locations"] + list(LARGE))
def test_cpp_plan_of_the_folded_graph_is_the_python_plan(case, tmp_path):
    """Fold, attention fold, units and simulated order of service, all in C++, against the same chain in
    Python: what the C++ host launches on every rank, and in which order, is what the Python runner launches."""
    from einsummable_b200 import memgraph as M
    L = _lib()
    if not hasattr(L, "ref_graph_fold_attention"):
        pytest.skip("oracle/_ref/libes_ref.so predates the attention fold")
    _, hf, _, mg, _ = _fold(L, case, tmp_path)
    ha = L.ref_graph_fold_attention(hf, str(tmp_path / "attention.json").encode())
    assert ha >= 0, L.ref_graph_last_error().decode()
    want_mg = F.fuse_attention(F.fuse_elementwise_chains(mg)[0])[0]
    world = mg["num_locs"]
    kinds = set()
    for rank in range(world):
        upath = str(tmp_path / ("ordered%d.json" % rank))
        assert L.ref_graph_exchange_units_ordered(ha, rank, upath.encode()) >= 0, L.ref_graph_last_error().decode()
        with open(upath) as f:
            got = json.load(f)
        want = M.order_units_by_simulation(want_mg, world, rank)
        assert len(got["units"]) == len(want)
        for i, (g, w) in enumerate(zip(got["units"], want)):
            assert g["kind"] == w["kind"], (case, rank, i, g, w)
            assert g["node"] == w.get("node", -1) or w["kind"] in ("signal", "await", "pull", "wait"), (case, rank, i, g, w)
            assert g["moves"] == list(w.get("moves", [])), (case, rank, i, g, w)
            assert g["deps"] == list(w["deps"]), (case, rank, i, g, w)
            assert got["ready_us"][i] == w["sim_start_us"] and got["finish_us"][i] == w["sim_finish_us"], (case, rank, i)
            kinds.add(w["kind"])
    assert "training" in case or "attention" in kinds


# which case, nodes folded away, what it shows
HAZARDS = [
    (0, 1, "nothing in the way"),
    (1, 0, "a fill between A and B writes the memory A reads"),
    (2, 0, "B reads A's bytes under another shape"),
    (3, 0, "A's result is a saved result"),
    (4, 0, "a copy node reads A's result"),
    (5, 1, "two readers: A folds into both"),
    (6, 0, "B writes into the memory A reads"),
    (7, 1, "a later writer into the memory A read must wait for B"),
]


@pytest.mark.parametrize("which,folded,what", HAZARDS)
def test_fold_conditions_on_hand_made_graphs(which, folded, what, tmp_path):
    """One producer, its reader(s) and whatever stands in the way, built node by node with memgraph_t::insert:
    the C++ pass and the Python pass fold, or refuse, alike."""
    L = _lib()
    if not hasattr(L, "ref_graph_build_fold_case"):
        pytest.skip("oracle/_ref/libes_ref.so predates the hand-made fold cases")
    h = L.ref_graph_build_fold_case(which)
    assert h >= 0, L.ref_graph_last_error().decode()
    n = ctypes.c_int(-1)
    hf = L.ref_graph_fold_elementwise(h, ctypes.byref(n))
    assert hf >= 0, L.ref_graph_last_error().decode()
    mg = _json(L, h, str(tmp_path / "mg.json"))
    got = _json(L, hf, str(tmp_path / "folded.json"))
    if which == 3:      # the region of A's result as a saved block
        mg["outputs"] = [{"blocks": [{"loc": 0, "offset": 256, "size": 256}]}]
    want, want_folded = F.fuse_elementwise_chains(mg)
    assert n.value == folded and want_folded == folded, (what, n.value, want_folded)
    for g, w in zip(got["nodes"], want["nodes"]):
        assert sorted(g["inns"]) == sorted(w["inns"]), (what, g["id"])
        if w.get("folded"):
            assert g["kind"] == "alloc"
        elif g["kind"] == "apply":
            assert g["mems"] == w["mems"], (what, g["id"])
            assert g["einsummable"]["inns"] == w["einsummable"]["inns"], (what, g["id"])
    if which == 5:
        composed = [g for g in got["nodes"] if g["kind"] == "apply" and len(g["mems"]) == 3 and [0, 256] in g["mems"][1:]]
        assert len(composed) == 2
    if which == 7:
        fill = [g for g in got["nodes"] if g["kind"] == "constant"][0]
        reader = [g for g in got["nodes"] if g["kind"] == "apply"][0]
        assert reader["id"] in fill["inns"], (fill, reader)


def test_engine_parity_binary_loads_without_a_gpu():
    """The binary the GPU tests run (the reference's engine, gpu_program_t, gpu_exchange_program_t and the C++
    passes linked with the library) resolves all its symbols here: without arguments it prints its usage
    before any CUDA call."""
    import subprocess
    path = os.path.join(ROOT, "oracle", "_ref", "engine_parity")
    if not os.path.exists(path):
        pytest.skip("the reference has not been compiled here (oracle/_ref)")
    res = subprocess.run([path], capture_output=True, text=True, timeout=60)
    assert res.returncode == 1 and "usage: engine_parity" in res.stderr and "[fold]" in res.stderr, res.stderr[-500:]
