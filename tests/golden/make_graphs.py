#!/usr/bin/env python3
"""Generates the graph-level fixtures under tests/golden/graphs/ from the
reference's own compilers and interpreter (oracle/_ref/libes_ref.so, built from
the reference sources by oracle/Makefile; see oracle/ref_graphs.cc).

For every case: the memgraph as JSON (what the reference's graph -> taskgraph ->
memgraph pipeline emits for that graph and placement).  For the small cases also
seeded inputs and the outputs of the reference's interpreter on them (graphs.npz):
oracle/ref_graphs.cc walks the memgraph in order with the reference's own
reference_einsummable / reference_touch / reference_fill, because
reference_compute_memgraph itself rejects constant nodes.  Runs only where the
reference tree exists.

The full-size training graphs take the reference's autoplacer and memgraph
compiler up to half an hour each (8 locations: 49003 memgraph nodes), so an
existing file is kept unless --force is given.

usage: python tests/golden/make_graphs.py [--force]
"""
import ctypes
import gzip
import json
import os
import shutil
import sys

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


def write_json(h, name, compress):
    tmp = os.path.join(OUT, name + ".json")
    ok(L.ref_graph_write_json(h, tmp.encode()))
    with open(tmp) as f:
        mg = json.load(f)
    if compress:
        with open(tmp, "rb") as f, gzip.GzipFile(tmp + ".gz", "wb", mtime=0) as g:
            shutil.copyfileobj(f, g)
        os.remove(tmp)
    return mg


def run_reference(h, mg, inputs):
    bufs = [np.zeros(int(s) + 256, dtype=np.uint8) for s in mg["mem_sizes"]]
    for t in mg["inputs"]:
        a = inputs[t["name"]].reshape(t["shape"])
        for blk, sl in zip(t["blocks"], blocks_of(t["shape"], t["partdims"])):
            raw = np.ascontiguousarray(a[sl]).view(np.uint8).reshape(-1)
            assert raw.size == blk["size"]
            bufs[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]] = raw
    ptrs = (ctypes.c_void_p * len(bufs))(*[b.ctypes.data for b in bufs])
    ok(L.ref_graph_run(h, ptrs))
    outs = {}
    for t in mg["outputs"]:
        out = np.zeros(t["shape"], dtype=NP[t["dtype"]])
        for blk, sl in zip(t["blocks"], blocks_of(t["shape"], t["partdims"])):
            raw = bufs[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]]
            out[sl] = raw.view(NP[t["dtype"]]).reshape(out[sl].shape)
        outs[t["name"]] = out
    return outs


def llama_inputs(mg, rng, weight_std):
    ins = {}
    for t in mg["inputs"]:
        shape, name = t["shape"], t["name"]
        if name == "freqs_cis":
            seq, half = shape
            theta = 1.0 / (10000.0 ** (np.arange(half) / half))
            ang = np.outer(np.arange(seq), theta)
            ins[name] = (np.cos(ang) + 1j * np.sin(ang)).astype(np.complex64)
        elif name.endswith("norm.weight"):
            ins[name] = rng.uniform(0.5, 1.5, shape).astype(NP[t["dtype"]])
        elif name == "embeddings":
            ins[name] = rng.standard_normal(shape).astype(NP[t["dtype"]])
        else:
            ins[name] = (rng.standard_normal(shape) * weight_std).astype(NP[t["dtype"]])
    return ins


def main():
    os.makedirs(OUT, exist_ok=True)
    arrays = {}

    # config 1, small (with the reference's result) and full size (graph only)
    for nlocs in (1, 2):
        h = ok(L.ref_graph_build_c1(u64(64), 2, nlocs, 1))
        mg = write_json(h, "c1_n64_locs%d" % nlocs, False)
        rng = np.random.default_rng(5)
        ins = {"lhs": rng.uniform(-1, 1, (64, 64)).astype(np.float32),
               "rhs": rng.uniform(-1, 1, (64, 64)).astype(np.float32)}
        outs = run_reference(h, mg, ins)
        for k, v in ins.items():
            arrays["c1_n64_locs%d/in/%s" % (nlocs, k)] = v
        for k, v in outs.items():
            arrays["c1_n64_locs%d/out/%s" % (nlocs, k)] = v
    for nlocs in (1, 2, 8):
        h = ok(L.ref_graph_build_c1(u64(4096), 2, nlocs, 1))
        write_json(h, "c1_n4096_locs%d" % nlocs, True)

    # config 4, tiny model through the reference's memgraph interpreter
    for nlocs in (1, 2, 4):
        h = ok(L.ref_graph_build_llama(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), nlocs, 0))
        mg = write_json(h, "llama_tiny_locs%d" % nlocs, False)
        ins = llama_inputs(mg, np.random.default_rng(11), 0.3)
        outs = run_reference(h, mg, ins)
        for k, v in ins.items():
            arrays["llama_tiny_locs%d/in/%s" % (nlocs, k)] = v
        for k, v in outs.items():
            arrays["llama_tiny_locs%d/out/%s" % (nlocs, k)] = v
        print("llama tiny", nlocs, "locs:", {k: float(np.abs(v.astype(np.float64)).max()) for k, v in outs.items()})

    # config 4, LLaMA-7B-shape layer (graph only): dim 4096, 32 heads, FFN 11008, vocab 32000, B=4, S=512
    for nlocs in (1, 2, 4, 8):
        h = ok(L.ref_graph_build_llama(u64(4096), u64(32), u64(256), u64(32000), 1, u64(4), u64(512), nlocs, 0))
        mg = write_json(h, "llama7b_layer_locs%d" % nlocs, True)
        print("llama 7B layer", nlocs, "locs:", mg["taskgraph"], "nodes", len(mg["nodes"]))

    # config 5, tiny: forward + backward + vanilla update in f32 through the reference's interpreter;
    # the gradients themselves are saved so that the comparison is not swamped by the weights
    for nlocs in (1, 2):
        h = ok(L.ref_graph_build_llama_train(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), nlocs, 1,
                                             ctypes.c_double(0.01), 1, 0, 0))
        name = "llama_train_tiny_locs%d" % nlocs
        mg = write_json(h, name, True)
        ins = llama_inputs(mg, np.random.default_rng(3), 0.3)
        labels = np.zeros((2, 128), dtype=np.float32)
        labels[0, 5] = labels[1, 77] = 1.0
        ins["labels"] = labels
        outs = run_reference(h, mg, ins)
        for k, v in ins.items():
            arrays["%s/in/%s" % (name, k)] = v
        for k, v in outs.items():
            arrays["%s/out/%s" % (name, k)] = v
        print(name, mg["taskgraph"], "loss", outs["loss"])

    # config 5, tiny, with the reference trainer's own AdamW updater (src/misc/update.cc:100-189; f32, its
    # scalar variables of iteration 1 substituted): weights, first and second moments all updated
    for nlocs in (1, 2):
        h = ok(L.ref_graph_build_llama_train(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), nlocs, 1,
                                             ctypes.c_double(0.01), 1, 1, 0))
        name = "llama_train_adamw_tiny_locs%d" % nlocs
        mg = write_json(h, name, True)
        rng = np.random.default_rng(4)
        ins = llama_inputs(mg, rng, 0.3)
        labels = np.zeros((2, 128), dtype=np.float32)
        labels[0, 9] = labels[1, 100] = 1.0
        ins["labels"] = labels
        for t in mg["inputs"]:                  # optimizer state: small positive second moments
            if t["name"].startswith("m."):
                ins[t["name"]] = (rng.standard_normal(t["shape"]) * 1e-3).astype(np.float32)
            elif t["name"].startswith("v."):
                ins[t["name"]] = (rng.uniform(1e-6, 1e-5, t["shape"])).astype(np.float32)
        outs = run_reference(h, mg, ins)
        for k, v in ins.items():
            arrays["%s/in/%s" % (name, k)] = v
        for k, v in outs.items():
            arrays["%s/out/%s" % (name, k)] = v
        print(name, mg["taskgraph"], "loss", outs["loss"])

    # config 5, tiny, the reference trainer's set-up: rank-4 LoRA adapters trained, base weights frozen
    for nlocs in (1, 2):
        h = ok(L.ref_graph_build_llama_train(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), nlocs, 1,
                                             ctypes.c_double(0.01), 1, 0, 4))
        name = "llama_train_lora_tiny_locs%d" % nlocs
        mg = write_json(h, name, True)
        ins = llama_inputs(mg, np.random.default_rng(6), 0.3)
        labels = np.zeros((2, 128), dtype=np.float32)
        labels[0, 3] = labels[1, 64] = 1.0
        ins["labels"] = labels
        outs = run_reference(h, mg, ins)
        for k, v in ins.items():
            arrays["%s/in/%s" % (name, k)] = v
        for k, v in outs.items():
            arrays["%s/out/%s" % (name, k)] = v
        print(name, mg["taskgraph"], "loss", outs["loss"], [t["name"] for t in mg["outputs"]][:6])

    # config 5, LLaMA-7B shape (graph only): 4 layers forward + backward + update, f16, at B=4, S=512 and at
    # the batch the config names, B=8, S=1024 (117 GB on one location; 8 locations: 58747 nodes, 35 minutes)
    force = "--force" in sys.argv[1:]
    for n_layers, nlocs, batch, seq in ((1, 1, 4, 512), (4, 1, 4, 512), (4, 2, 4, 512), (4, 4, 4, 512),
                                        (4, 8, 4, 512), (4, 1, 8, 1024), (4, 8, 8, 1024)):
        name = "llama7b_train_l%d_locs%d" % (n_layers, nlocs)
        if (batch, seq) != (4, 512):
            name = "llama7b_train_b%ds%d_l%d_locs%d" % (batch, seq, n_layers, nlocs)
        if os.path.exists(os.path.join(OUT, name + ".json.gz")) and not force:
            print(name, "kept")
            continue
        h = ok(L.ref_graph_build_llama_train(u64(4096), u64(32), u64(256), u64(32000), n_layers, u64(batch), u64(seq),
                                             nlocs, 0, ctypes.c_double(1e-3), 0, 0, 0))
        mg = write_json(h, name, True)
        print(name, mg["taskgraph"], "nodes", len(mg["nodes"]))

    np.savez_compressed(os.path.join(OUT, "graphs.npz"), **arrays)


if __name__ == "__main__":
    main()
