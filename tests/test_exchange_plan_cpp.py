"""The C++ planner of the exchange units (einsummable_b200/host/gpu_exchange_plan.h, compiled against the
reference's memgraph_t into oracle/_ref/libes_ref.so) against the Python planner
(einsummable_b200/memgraph.py: schedule_units) on memgraphs the reference's compilers build in-process:
the same units, in the same order, with the same dependencies, on every rank."""
import ctypes
import json
import os

import pytest

from conftest import ROOT
from einsummable_b200 import memgraph as M

LIB = os.path.join(ROOT, "oracle", "_ref", "libes_ref.so")
u64 = ctypes.c_uint64


def _lib():
    if not os.path.exists(LIB):
        pytest.skip("the reference has not been compiled here (oracle/_ref)")
    lib = ctypes.CDLL(LIB)
    if not hasattr(lib, "ref_graph_exchange_units"):
        pytest.skip("oracle/_ref/libes_ref.so predates the exchange planner")
    lib.ref_graph_last_error.restype = ctypes.c_char_p
    return lib


CASES = {
    "c1 64^3 on 2 locations": lambda L: L.ref_graph_build_c1(u64(64), 2, 2, 1),
    "c1 64^3 on 2 locations with 12 KB each (evict / load)": lambda L: L.ref_graph_build_c1_evict(u64(64), 4, 2, 1, u64(12288)),
    "tiny llama, autoplace01, 2 locations": lambda L: L.ref_graph_build_llama(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 2, 0),
    "tiny llama, autoplace01, 4 locations": lambda L: L.ref_graph_build_llama(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 4, 0),
    "tiny llama, tensor-parallel, 4 locations": lambda L: L.ref_graph_build_llama_tp(u64(64), u64(4), u64(32), u64(128), 1, u64(2), u64(16), 4, 0),
    "tiny training graph, 2 locations": lambda L: L.ref_graph_build_llama_train(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 2, 1,
                                                                                 ctypes.c_double(0.01), 1, 0, 0),
    "LLaMA-7B layer, tensor-parallel, 8 locations": lambda L: L.ref_graph_build_llama_tp(u64(4096), u64(32), u64(256), u64(32000), 1, u64(4),
                                                                                          u64(512), 8, 0),
}


@pytest.mark.parametrize("case", list(CASES))
def test_cpp_and_python_planners_agree(case, tmp_path):
    L = _lib()
    h = CASES[case](L)
    assert h >= 0, L.ref_graph_last_error().decode()
    path = str(tmp_path / "mg.json")
    assert L.ref_graph_write_json(h, path.encode()) >= 0
    with open(path) as f:
        mg = json.load(f)
    n_exchange = 0
    for rank in range(mg["num_locs"]):
        upath = str(tmp_path / ("units%d.json" % rank))
        assert L.ref_graph_exchange_units(h, rank, upath.encode()) >= 0, L.ref_graph_last_error().decode()
        with open(upath) as f:
            got = json.load(f)
        want = M.schedule_units(mg, {rank}, True)
        assert len(got) == len(want), (case, rank, len(got), len(want))
        for i, (g, w) in enumerate(zip(got, want)):
            assert g["kind"] == w["kind"], (case, rank, i, g, w)
            assert g["node"] == w.get("node", -1) or w["kind"] in ("signal", "await", "pull", "wait"), (case, rank, i, g, w)
            assert g["moves"] == list(w.get("moves", [])), (case, rank, i, g, w)
            assert g["deps"] == list(w["deps"]), (case, rank, i, g, w)
            if w["kind"] in ("touch", "rtouch"):
                assert g["first"] == w["first"], (case, rank, i, g, w)
            n_exchange += w["kind"] in ("signal", "await", "pull", "rtouch", "wait")
    assert n_exchange > 0


@pytest.mark.parametrize("case", list(CASES))
def test_cpp_and_python_orders_of_simulated_service_agree(case, tmp_path):
    """es_exchange::order_units against order_units_by_simulation: the same units in the same order with
    the same renumbered dependencies, and the same simulated ready and finish times (the two run the
    same double arithmetic in the same order, so the times agree to the last bit)."""
    L = _lib()
    if not hasattr(L, "ref_graph_exchange_units_ordered"):
        pytest.skip("oracle/_ref/libes_ref.so predates the simulated order")
    h = CASES[case](L)
    assert h >= 0, L.ref_graph_last_error().decode()
    path = str(tmp_path / "mg.json")
    assert L.ref_graph_write_json(h, path.encode()) >= 0
    with open(path) as f:
        mg = json.load(f)
    world = mg["num_locs"]
    moved = 0
    for rank in range(world):
        upath = str(tmp_path / ("ordered%d.json" % rank))
        assert L.ref_graph_exchange_units_ordered(h, rank, upath.encode()) >= 0, L.ref_graph_last_error().decode()
        with open(upath) as f:
            got = json.load(f)
        want = M.order_units_by_simulation(mg, world, rank)
        plain = M.schedule_units(mg, {rank}, True)
        assert len(got["units"]) == len(want)
        for i, (g, w) in enumerate(zip(got["units"], want)):
            assert g["kind"] == w["kind"], (case, rank, i, g, w)
            assert g["node"] == w.get("node", -1) or w["kind"] in ("signal", "await", "pull", "wait"), (case, rank, i, g, w)
            assert g["moves"] == list(w.get("moves", [])), (case, rank, i, g, w)
            assert g["deps"] == list(w["deps"]), (case, rank, i, g, w)
            assert got["ready_us"][i] == w["sim_start_us"], (case, rank, i, got["ready_us"][i], w["sim_start_us"])
            assert got["finish_us"][i] == w["sim_finish_us"], (case, rank, i, got["finish_us"][i], w["sim_finish_us"])
        moved += sum(1 for w, p in zip(want, plain) if (w["kind"], w.get("node"), tuple(w.get("moves", ()))) !=
                     (p["kind"], p.get("node"), tuple(p.get("moves", ()))))
    assert moved > 0 or "c1" in case       # the simulated order differs from memgraph order somewhere


@pytest.mark.parametrize("case", ["tiny llama, tensor-parallel, 4 locations", "LLaMA-7B layer, tensor-parallel, 8 locations"])
def test_cpp_and_python_planners_agree_on_summed_remote_adds(case, tmp_path):
    """make_units' group_sum against schedule_units(group_sum=True): the remote adds of a partial-sum group as
    one `rsum` unit and one `ack` unit, in the same place, over the same touches and moves."""
    L = _lib()
    if not hasattr(L, "ref_graph_exchange_units_group_sum"):
        pytest.skip("oracle/_ref/libes_ref.so predates the summed remote adds")
    h = CASES[case](L)
    assert h >= 0, L.ref_graph_last_error().decode()
    path = str(tmp_path / "mg.json")
    assert L.ref_graph_write_json(h, path.encode()) >= 0
    with open(path) as f:
        mg = json.load(f)
    world = mg["num_locs"]
    n_rsum = 0
    for rank in range(world):
        upath = str(tmp_path / ("gs%d.json" % rank))
        assert L.ref_graph_exchange_units_group_sum(h, rank, upath.encode()) >= 0, L.ref_graph_last_error().decode()
        with open(upath) as f:
            got = json.load(f)["units"]
        want = M.order_units_by_simulation(mg, world, rank, group_sum=True)
        assert len(got) == len(want)
        for i, (g, w) in enumerate(zip(got, want)):
            assert g["kind"] == w["kind"], (case, rank, i, g, w)
            assert g["moves"] == list(w.get("moves", [])), (case, rank, i, g, w)
            assert g["deps"] == list(w["deps"]), (case, rank, i, g, w)
            assert g["nodes"] == list(w.get("nodes", [])), (case, rank, i, g, w)
            n_rsum += w["kind"] == "rsum"
    assert n_rsum > 0
