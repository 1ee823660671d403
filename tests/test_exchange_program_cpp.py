"""What the C++ host asks the library to do on every rank of a multi-location memgraph, without a GPU.

oracle/_ref/exchange_ops builds the memgraph in-process with the reference's compilers, folds it with the C++ passes
(einsummable_b200/host/gpu_fuse.h) and constructs one gpu_exchange_program_t (einsummable_b200/host/gpu_program.*) per
rank over made-up base addresses, linked with a recording stand-in of the C ABI (oracle/mock_es_b200.cc).  The recorded
ops -- kind, dependencies, every pointer, flag word, touch dimension and attention descriptor -- must be the ones the
Python runner derives from the same memgraph (fuse.py, memgraph.py: order_units_by_simulation), op for op."""
import ctypes
import json
import os
import subprocess

import pytest

from conftest import ROOT
from einsummable_b200 import fuse as F
from einsummable_b200 import memgraph as M

BIN = os.path.join(ROOT, "oracle", "_ref", "exchange_ops")
LIB = os.path.join(ROOT, "oracle", "_ref", "libes_ref.so")
CASTABLE = {None: -1, "add": 0, "mul": 1, "min": 2, "max": 3}
DTYPE = {"f16": 0, "f32": 1, "f64": 2, "c64": 3}

CASES = [
    ("llama_tp:64:4:32:128:1:2:16:0:4", 0),
    ("llama_tp:64:4:32:128:1:2:16:0:4", 1),
    ("llama:64:2:32:128:1:2:16:0:2", 0),
    ("llama:64:2:32:128:1:2:16:0:4", 0),
    ("llama_tp:4096:32:256:32000:1:4:512:0:8", 0),
    ("llama_tp:4096:32:256:32000:1:4:512:0:8", 1),
    ("llama:4096:32:256:32000:1:4:512:0:2", 0),
    ("c1_evict:64:4:1:12288:2", 0),          # config 1 under a memory limit: evict / load to host storage
    ("c1_evict:64:4:1:20480:1", 0),
    ("llama:64:2:32:128:1:2:16:0:1", 0),     # one location: gpu_program_t too
]


def ptr(loc, off):
    return ((loc + 1) << 44) + off


@pytest.mark.parametrize("spec,group_sum", CASES)
def test_cpp_exchange_program_ops_are_the_python_runners(spec, group_sum, tmp_path):
    if not os.path.exists(BIN) or not os.path.exists(LIB):
        pytest.skip("the reference has not been compiled here (oracle/_ref)")
    res = subprocess.run([BIN, spec, str(tmp_path), str(group_sum)], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    with open(tmp_path / "memgraph.json") as f:
        mg = json.load(f)
    world = mg["num_locs"]
    fused = F.fuse_attention(F.fuse_elementwise_chains(mg)[0])[0]
    nodes = fused["nodes"]
    cross = [n["id"] for n in nodes if n["kind"] == "move" and n["src_loc"] != n["dst_loc"]]
    index = {m: k for k, m in enumerate(cross)}
    lib = ctypes.CDLL(LIB)
    lib.ref_last_error.restype = ctypes.c_char_p
    seen = {}

    def normal(text):     # a join as the reference's parser prints it back (its constructor simplifies the tree)
        if text not in seen:
            buf = ctypes.create_string_buffer(1 << 16)
            assert lib.ref_scalarop_info(text.encode(), buf, len(buf)) == 0, lib.ref_last_error().decode()
            seen[text] = buf.value.decode()
        return seen[text]

    def flag(owner, kind, m):
        return ptr(owner, (1 << 40) + 4 * (kind * len(cross) + index[m]))

    kinds = set()
    programs = []
    for rank in range(world):
        with open(tmp_path / ("ops%d.json" % rank)) as f:
            programs.append((rank, json.load(f), M.order_units_by_simulation(fused, world, rank, bool(group_sum))))
    if world == 1:      # gpu_program_t: the units in memgraph order
        with open(tmp_path / "ops_program0.json") as f:
            programs.append(("gpu_program_t", json.load(f), M.schedule_units(fused, {0}, False)))
    for rank, got, units in programs:
        assert got["n_ops"] == len(units) == len(got["ops"])
        for i, (g, u) in enumerate(zip(got["ops"], units)):
            k = u["kind"]
            where = (spec, rank, i, k)
            kinds.add(k)
            assert sorted(set(g["deps"])) == list(u["deps"]), where
            if k == "einsummable":
                n = nodes[u["node"]]
                assert g["kind"] == "einsummable" and g["built_inns"] == len(n["mems"]) - 1, where
                assert g["out"] == ptr(n["loc"], n["mems"][0][0]), where
                assert g["inns"] == [ptr(n["loc"], m[0]) for m in n["mems"][1:]], where
                assert g["join"] == n["einsummable"]["join"] or normal(g["join"]) == normal(n["einsummable"]["join"]), where
            elif k == "attention":
                n = nodes[u["node"]]
                a = n["attention"]
                assert g["kind"] == "attention", where
                assert g["shape"] == [a["batch"], a["heads"], a["rows"], a["keys"], a["head_dim"]], where
                assert (g["skip_known"], g["skip_from"], g["q_stride"]) == (a["skip_known"], a["skip_from"], a["q_stride"]), where
                assert [g[x] for x in ("out", "q", "k", "v", "mask")] == [ptr(n["loc"], m[0]) for m in n["mems"]], where
            elif k in ("touch", "rtouch"):
                n = nodes[u["node"]]
                d = n["touch"]
                assert g["kind"] == k, where
                assert g["dims"] == [[int(x) for x in dim] for dim in d["selection"]], where
                assert g["castable"] == (-1 if u["first"] else CASTABLE[d["castable"]]) and g["dtype"] == DTYPE[d["dtype"]], where
                assert g["out"] == ptr(n["loc"], n["mems"][0][0]), where
                if k == "rtouch":
                    m = nodes[u["moves"][0]]
                    assert g["inn"] == ptr(m["src_loc"], m["src_offset"]), where
                    assert g["done_flag"] == flag(m["src_loc"], 1, m["id"]), where
                else:
                    assert g["inn"] == ptr(n["loc"], n["mems"][1][0]), where
            elif k == "constant":
                n = nodes[u["node"]]
                f = n["fill"]
                assert g["out"] == ptr(n["loc"], n["offset"]), where
                if f["type"] == "constant":
                    assert (g["kind"], g["dtype"], g["nelem"]) == ("fill_constant", DTYPE[f["value"]["dtype"]], f["nelem"]), where
                else:
                    assert (g["kind"], g["dtype"], g["nrow"], g["ncol"], g["start"]) == (
                        "fill_lowertri", DTYPE[f["lower"]["dtype"]], f["nrow"], f["ncol"], f["start"]), where
            elif k == "copy":
                n = nodes[u["node"]]
                s, d = (n["src_loc"], n["dst_loc"]) if n["kind"] == "move" else (n["loc"], n["loc"])
                assert (g["kind"], g["src"], g["dst"], g["bytes"]) == (
                    "copy", ptr(s, n["src_offset"]), ptr(d, n["dst_offset"]), n["size"]), where
            elif k in ("evict", "load"):
                n = nodes[u["node"]]
                assert (g["kind"], g["dev"], g["host"], g["bytes"]) == (
                    k, ptr(n["loc"], n["offset"]), (1 << 50) + 4096 * n["storage_id"], n["size"]), where
            elif k == "rsum":
                n = nodes[u["nodes"][0]]
                out = ptr(n["loc"], n["mems"][0][0])
                assert g["kind"] == "einsummable" and g["out"] == out and g["built_inns"] == len(u["moves"]) + 1, where
                assert g["inns"] == [out] + [ptr(nodes[m]["src_loc"], nodes[m]["src_offset"]) for m in u["moves"]], where
            elif k == "ack":
                assert g["kind"] == "signal" and g["flags"] == [flag(nodes[m]["src_loc"], 1, m) for m in u["moves"]], where
            elif k == "signal":
                assert g["kind"] == "signal" and g["flags"] == [flag(nodes[m]["dst_loc"], 0, m) for m in u["moves"]], where
            elif k == "await":
                assert g["kind"] == "wait" and g["flags"] == [flag(nodes[m]["dst_loc"], 0, m) for m in u["moves"]], where
            elif k == "pull":
                assert g["kind"] == "pull" and g["items"] == [
                    [ptr(nodes[m]["src_loc"], nodes[m]["src_offset"]), ptr(nodes[m]["dst_loc"], nodes[m]["dst_offset"]),
                     nodes[m]["size"], 0, flag(nodes[m]["src_loc"], 1, m)] for m in u["moves"]], where
            elif k == "wait":
                assert g["kind"] == "wait" and g["flags"] == [flag(nodes[m]["src_loc"], 1, m) for m in u["moves"]], where
            else:
                raise AssertionError(where)
    if spec.startswith("c1_evict"):
        assert {"evict", "load"} <= kinds, kinds
    if world > 1:
        assert {"signal", "await", "wait", "einsummable"} <= kinds, kinds
    if group_sum:
        assert {"rsum", "ack"} <= kinds, kinds
