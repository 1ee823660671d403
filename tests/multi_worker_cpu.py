"""Worker of tests/test_multi_rank.py: one gloo process per location interprets its share of a
partitioned memgraph with the numpy oracle and exchanges the moves as grouped send / recv pairs,
cut into groups by einsummable_b200.memgraph.move_runs exactly as the GPU runner's NCCL transport
cuts them.  A wrong cut shows up here as ranks waiting on each other (the test has a timeout)."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import es_oracle as O  # noqa: E402
from einsummable_b200.memgraph import load_memgraph, move_runs  # noqa: E402


def main():
    name, fuse = sys.argv[1], "fuse" in sys.argv[2:]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    graphs = os.path.join(ROOT, "tests", "golden", "graphs")
    path = os.path.join(graphs, name + ".json")
    mg = load_memgraph(path if os.path.exists(path) else path + ".gz")
    assert mg["num_locs"] == world
    if fuse:
        from einsummable_b200.fuse import fuse_elementwise_chains
        mg, _ = fuse_elementwise_chains(mg)
    arr = np.load(os.path.join(graphs, "graphs_tp.npz" if "_tp_" in name else "graphs.npz"))
    pre = name + "/in/"
    ins = {k[len(pre):]: arr[k] for k in arr.files if k.startswith(pre)}
    bufs = O.memgraph_place_inputs(mg, ins)          # every location's inputs; only this rank's buffer is used
    runs = move_runs(mg)
    touched = set()
    pending, pending_run = [], None

    def flush():
        nonlocal pending, pending_run
        ops, keep = [], []
        for node in pending:
            s, d, n = node["src_loc"], node["dst_loc"], node["size"]
            if s == d:
                if s == rank:
                    bufs[rank][node["dst_offset"]:node["dst_offset"] + n] = bufs[rank][node["src_offset"]:node["src_offset"] + n].copy()
            elif s == rank:
                t = torch.from_numpy(bufs[rank][node["src_offset"]:node["src_offset"] + n].copy())
                keep.append(t)
                ops.append(dist.P2POp(dist.isend, t, d))
            elif d == rank:
                t = torch.empty(n, dtype=torch.uint8)
                keep.append((t, node["dst_offset"]))
                ops.append(dist.P2POp(dist.irecv, t, s))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        for k in keep:
            if isinstance(k, tuple):
                bufs[rank][k[1]:k[1] + k[0].numel()] = k[0].numpy()
        pending, pending_run = [], None

    for node in mg["nodes"]:
        if node["kind"] == "move":
            r = runs[node["id"]]
            if pending and r != pending_run:
                flush()
            pending.append(node)
            pending_run = r
            continue
        if node["kind"] in ("alloc", "del", "inputmem", "partialize"):
            continue
        if pending:
            flush()
        O.run_memgraph({"nodes": [node]}, bufs, "executor", groups_touched=touched, only_loc=rank)
    if pending:
        flush()

    # every block of a saved tensor lives on one rank: zero elsewhere, summed over the ranks
    for loc in range(world):
        if loc != rank:
            bufs[loc][:] = 0
    got = O.memgraph_collect_outputs(mg, bufs)
    pre = name + "/out/"
    ok = True
    for k in arr.files:
        if not k.startswith(pre):
            continue
        want = arr[k]
        t = torch.from_numpy(got[k[len(pre):]].astype(np.float64))
        dist.all_reduce(t)
        scale = np.abs(want.astype(np.float64)).max()
        err = np.abs(t.numpy() - want.astype(np.float64)).max()
        tol = 2e-2 if want.dtype == np.float16 else 1e-4
        ok = ok and err <= tol * scale
    if rank == 0:
        print(json.dumps({"name": name, "world": world, "ok": bool(ok), "runs": len(set(runs.values()))}))
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
