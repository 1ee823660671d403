#!/usr/bin/env python3
"""Generates the storage fixture: config 1's blocked matmul compiled by the reference's
memgraph_t::make with a memory limit per location that the tensors do not fit in, so that the
memgraph holds evict / load nodes and inputs that start out in storage (the set-up of the
reference's own exps/reference.cc:89-211 test_make_memgraph_with_evict).

  tests/golden/graphs/c1_n64_evict_locs{1,2}.json   the memgraphs
  tests/golden/graphs/graphs_evict.npz                seeded inputs and the outputs of the reference's
                                                      reference_compute_memgraph with storage

Runs only where oracle/_ref/libes_ref.so was built from the reference tree.

usage: python tests/golden/make_evict_graph.py
"""
import ctypes
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "graphs")
NP = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "c64": np.complex64}
L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libes_ref.so"))
L.ref_graph_last_error.restype = ctypes.c_char_p
u64 = ctypes.c_uint64


def ok(h):
    if h < 0:
        raise RuntimeError(L.ref_graph_last_error().decode())
    return h


def blocks_of(shape, partdims):
    starts = [np.concatenate([[0], np.cumsum(p)]) for p in partdims]
    grid = [len(p) for p in partdims]
    for flat in range(int(np.prod(grid))):
        idx = np.unravel_index(flat, grid)
        yield tuple(slice(int(starts[d][i]), int(starts[d][i + 1])) for d, i in enumerate(idx))


def main():
    arrays = {}
    for nlocs, limit in ((1, 20480), (2, 12288)):
        name = "c1_n64_evict_locs%d" % nlocs
        h = ok(L.ref_graph_build_c1_evict(u64(64), 4, nlocs, 1, u64(limit)))
        path = os.path.join(OUT, name + ".json")
        ok(L.ref_graph_write_json(h, path.encode()))
        with open(path) as f:
            mg = json.load(f)
        kinds = {}
        for n in mg["nodes"]:
            kinds[n["kind"]] = kinds.get(n["kind"], 0) + 1
        assert kinds.get("evict", 0) > 0 and kinds.get("load", 0) > 0, kinds
        rng = np.random.default_rng(11)
        ins = {"lhs": rng.uniform(-1, 1, (64, 64)).astype(np.float32),
               "rhs": rng.uniform(-1, 1, (64, 64)).astype(np.float32)}
        bufs = [np.zeros(int(s) + 256, dtype=np.uint8) for s in mg["mem_sizes"]]
        for t in mg["inputs"]:
            a = ins[t["name"]].reshape(t["shape"])
            for blk, sl in zip(t["blocks"], blocks_of(t["shape"], t["partdims"])):
                raw = np.ascontiguousarray(a[sl]).view(np.uint8).reshape(-1)
                assert raw.size == blk["size"]
                if "sto_id" in blk:
                    ok(L.ref_graph_sto_write(h, blk["sto_loc"], blk["sto_id"], raw.ctypes.data_as(ctypes.c_void_p), u64(raw.size)))
                else:
                    bufs[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]] = raw
        ptrs = (ctypes.c_void_p * len(bufs))(*[b.ctypes.data for b in bufs])
        ok(L.ref_graph_run_storage(h, ptrs))
        for t in mg["outputs"]:
            out = np.zeros(t["shape"], dtype=NP[t["dtype"]])
            for blk, sl in zip(t["blocks"], blocks_of(t["shape"], t["partdims"])):
                if "sto_id" in blk:
                    raw = np.zeros(blk["size"], dtype=np.uint8)
                    ok(L.ref_graph_sto_read(h, blk["sto_loc"], blk["sto_id"], raw.ctypes.data_as(ctypes.c_void_p), u64(raw.size)))
                else:
                    raw = bufs[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]]
                out[sl] = raw.view(NP[t["dtype"]]).reshape(out[sl].shape)
            arrays["%s/out/%s" % (name, t["name"])] = out
            want = ins["lhs"].astype(np.float64) @ ins["rhs"].astype(np.float64)
            assert np.abs(out - want).max() < 1e-4, "the reference interpreter's own result is off"
        for k, v in ins.items():
            arrays["%s/in/%s" % (name, k)] = v
        print(name, "limit", limit, "mem_sizes", mg["mem_sizes"], kinds)
    np.savez_compressed(os.path.join(OUT, "graphs_evict.npz"), **arrays)


if __name__ == "__main__":
    main()
