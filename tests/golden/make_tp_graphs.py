#!/usr/bin/env python3
"""Generates the fixtures of config 4 under the hand-written tensor-parallel placement
(oracle/ref_graphs.cc: ref_graph_build_llama_tp) from the reference's own taskgraph / memgraph
compilers: tiny models on 2 and 4 locations with seeded inputs and the reference interpreter's
outputs (graphs_tp.npz), and the LLaMA-7B-shape layer on 2, 4 and 8 locations (graph only; its
result is the same `scores` as for any other placement, tests/golden/c4_full.npz).

usage: python tests/golden/make_tp_graphs.py
"""
import ctypes
import os

import numpy as np

from make_graphs import L, OUT, llama_inputs, ok, run_reference, u64, write_json


def main():
    arrays = {}
    # 2 heads on 2 locations; 4 heads on 4 locations (partial-sum groups with three remote members)
    for name, dim, heads, nlocs in (("llama_tiny_tp_locs2", 64, 2, 2), ("llama_tiny_tp_locs4", 64, 4, 4)):
        h = ok(L.ref_graph_build_llama_tp(u64(dim), u64(heads), u64(32), u64(128), 1, u64(2), u64(16), nlocs, 0))
        mg = write_json(h, name, False)
        ins = llama_inputs(mg, np.random.default_rng(11), 0.3)
        outs = run_reference(h, mg, ins)
        for k, v in ins.items():
            arrays["%s/in/%s" % (name, k)] = v
        for k, v in outs.items():
            arrays["%s/out/%s" % (name, k)] = v
        print(name, mg["taskgraph"], {k: float(np.abs(v.astype(np.float64)).max()) for k, v in outs.items()})
    np.savez_compressed(os.path.join(OUT, "graphs_tp.npz"), **arrays)
    for nlocs in (2, 4, 8):
        h = ok(L.ref_graph_build_llama_tp(u64(4096), u64(32), u64(256), u64(32000), 1, u64(4), u64(512), nlocs, 0))
        mg = write_json(h, "llama7b_layer_tp_locs%d" % nlocs, True)
        print("llama 7B layer, tensor-parallel placement,", nlocs, "locs:", mg["taskgraph"], "nodes", len(mg["nodes"]))


if __name__ == "__main__":
    main()
