"""Worker of tests/test_gpu_multi.py: one process per GPU runs a memgraph whose
locations are the ranks, with moves over the chosen transport, and checks the
saved outputs against the reference interpreter's results."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from einsummable_b200.memgraph import load_memgraph, memgraph_runner_t  # noqa: E402


def log(*a):
    print("[rank %s]" % os.environ.get("RANK"), *a, file=sys.stderr, flush=True)


def main():
    name, transport = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    graphs = os.path.join(ROOT, "tests", "golden", "graphs")
    path = os.path.join(graphs, name + ".json")
    mg = load_memgraph(path if os.path.exists(path) else path + ".gz")
    arr = np.load(os.path.join(graphs, "graphs_tp.npz" if "_tp_" in name else "graphs.npz"))
    log("process group up; building runner", transport)
    r = memgraph_runner_t(mg, rank=rank, world=world, transport=transport, wait_limit_ms=2000,
                          fuse="fuse" in sys.argv[3:])
    log("runner built:", r.stats, "program ops", len(r.program))
    pre = name + "/in/"
    for k in arr.files:
        if k.startswith(pre):
            r.set_input(k[len(pre):], arr[k])
    dist.barrier()
    results = {}
    for run in range(3):        # repeated runs: flags must come back to zero every time
        r.run()
        log("run", run, "launched")
        torch.cuda.synchronize()
        log("run", run, "synchronised")
        status = r.device_status()
        assert status == 0, "rank %d: device status %#x on run %d" % (rank, status, run)
    if "capture" in sys.argv[3:]:
        log("capturing")
        r.capture()
        log("captured")
        r.replay()
        r.replay()
        torch.cuda.synchronize()
        assert r.device_status() == 0
    pre = name + "/out/"
    ok = True
    for k in arr.files:
        if not k.startswith(pre):
            continue
        want = arr[k]
        got = torch.from_numpy(r.get_output(k[len(pre):]).astype(np.float32)).cuda()
        dist.all_reduce(got)   # every block is owned by exactly one rank; the others contribute zeros
        got = got.cpu().numpy()
        scale = np.abs(want.astype(np.float64)).max()
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
        tol = 2e-2 if want.dtype == np.float16 else (1e-4 if name.startswith("llama_train") else 1e-5)
        if rank == 0:
            print(json.dumps({"output": k, "err": float(err), "scale": float(scale), "tol": tol,
                              "transport": transport, "moves": r.stats["move"]}))
        ok = ok and err <= tol * scale
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
