"""Host-side logic of the N>1 bench path on CPU: two `gloo` ranks run the
sharding arithmetic and the max-over-ranks reduction that `bench.py --gpus N`
uses (each rank owns the whole per-GPU workload; value = bytes of all ranks /
max time).  No GPU is involved."""
import os
import socket
import subprocess
import sys
import textwrap

from conftest import ROOT

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import torch, torch.distributed as dist
    import bench
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == 2
    # every rank times its own copy of the workload; the job's time is the slowest rank's
    ms = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert ms.item() == 15.0
    value = bench.BYTES_STEP * world * 4 / (ms.item() * 1e-3) / 1e9
    # weak scaling: the per-rank bytes do not depend on the world size
    assert bench.BYTES_STEP == 1262534656
    dist.barrier()
    if rank == 0:
        print(json.dumps({"value": value, "world": world}))
    dist.destroy_process_group()
""") % ROOT


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_reduce_max_time(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", env["MASTER_PORT"], str(script)],
        capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    import json
    out = json.loads(line)
    assert out["world"] == 2
    assert abs(out["value"] - 1262534656 * 2 * 4 / 15e-3 / 1e9) < 1e-6


def test_reference_arm_only_rank0_prints(tmp_path):
    """Under torchrun the reference arm runs on rank 0 alone; other ranks exit 0 silently."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
    env = dict(os.environ, RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0
    import json
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port" and line["value"] > 0


def _run_cpu_workers(nproc, name, *extra):
    worker = os.path.join(ROOT, "tests", "multi_worker_cpu.py")
    port = str(free_port())
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % nproc,
         "--master-addr", "127.0.0.1", "--master-port", port, worker, name] + list(extra),
        capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    import json
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["ok"] and out["world"] == nproc
    return out


def test_partitioned_memgraph_over_two_gloo_ranks():
    """One process per location, moves as grouped send / recv pairs cut by move_runs (the logic of
    the GPU runner's NCCL transport), results against the reference interpreter's."""
    _run_cpu_workers(2, "llama_tiny_locs2")


def test_tensor_parallel_memgraph_over_two_gloo_ranks():
    """The same model under the hand-written tensor-parallel placement (tests/golden/make_tp_graphs.py)."""
    _run_cpu_workers(2, "llama_tiny_tp_locs2")


def test_partitioned_memgraph_over_four_gloo_ranks():
    """The four-location graph is the one whose groups, cut per rank instead of from the global
    order, made the ranks wait on each other for ever."""
    _run_cpu_workers(4, "llama_tiny_locs4")


def test_folded_partitioned_training_graph_over_two_gloo_ranks():
    _run_cpu_workers(2, "llama_train_tiny_locs2", "fuse")
