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


def _json(L, h, path):
    assert L.ref_graph_write_json(h, path.encode()) >= 0, L.ref_graph_last_error().decode()
    with open(path) as f:
        return json.load(f)


def _fold(L, case, tmp_path):
    h = CASES[case](L)
    assert h >= 0, L.ref_graph_last_error().decode()
    n = ctypes.c_int(0)
    hf = L.ref_graph_fold_elementwise(h, ctypes.byref(n))
    assert hf >= 0, L.ref_graph_last_error().decode()
    return h, hf, n.value, _json(L, h, str(tmp_path / "mg.json")), _json(L, hf, str(tmp_path / "folded.json"))


@pytest.mark.parametrize("case", list(CASES))
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
