"""move_t across GPUs with one process per GPU: the reference's memgraphs for 2
(and 4) locations run under torchrun, moves over NCCL send/recv and over the
peer-memory transport (symmetric memory + bounded flag kernels + SM pull copy),
checked against the reference interpreter's results."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_workers(nproc, name, transport, *extra, **env_extra):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "multi_worker.py"), name, transport] + list(extra)
    for attempt in range(3):
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=env)
        if res.returncode == 0 or "EADDRINUSE" not in res.stderr:
            break
        # the port found free a moment ago was taken by the time torchrun bound it: pick another
        cmd[cmd.index("--master-port") + 1] = str(free_port())
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("transport", ["nccl", "p2p"])
def test_two_ranks_llama_tiny(transport):
    # CUDA-graph capture is exercised with the peer-memory transport only: a process group that
    # holds captured NCCL send/recv nodes did not shut down cleanly on this stack
    out = run_workers(2, "llama_tiny_locs2", transport, *(["capture"] if transport == "p2p" else []))
    assert '"transport": "%s"' % transport in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("name", ["llama_tiny_locs2", "llama_train_tiny_locs2", "llama_tiny_tp_locs2"])
def test_two_ranks_fused(name):
    """Elementwise nodes folded into their readers inside each location (every rank folds the same
    way); the moves and their hand-shakes are those of the unfused graph."""
    run_workers(2, name, "p2p", "fuse", "capture")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_c1(tmp_path):
    run_workers(2, "c1_n64_locs2", "p2p")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("transport", ["nccl", "p2p"])
def test_four_ranks_llama_tiny(transport):
    run_workers(4, "llama_tiny_locs4", transport)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("group_sum", ["0", "1"])
def test_four_ranks_tensor_parallel_placement(group_sum):
    """The tiny model under the hand-written tensor-parallel placement on 4 locations (partial-sum groups
    with three remote members), folded, attention as one kernel, captured; with group_sum the three remote
    adds of a group run as one elementwise kernel over the peers' memory."""
    run_workers(4, "llama_tiny_tp_locs4", "p2p", "fuse", "capture", ES_B200_GROUP_SUM=group_sum)


def test_flag_kernels_single_gpu():
    """signal / wait on flags whose state already allows them to pass (no kernel waits on
    another one), and a wait that runs out: it must report, not hang or trap."""
    import einsummable_b200 as es
    km = es.kernel_manager_t(0)
    flags = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    km.flag_signal(flags[0:], None)            # 0 -> 1
    km.flag_wait(flags[0:], None)              # 1 -> 0
    km.flag_signal(flags[1:], None)
    torch.cuda.synchronize()
    assert flags.cpu().tolist() == [0, 1, 0, 0]
    assert km.device_status() == 0
    km.flag_wait(flags[2:], None, limit_ms=50)   # nothing will ever set this flag
    torch.cuda.synchronize()
    assert km.device_status() == 0x200           # wait gave up; the context is still usable
    assert flags.cpu().tolist() == [0, 1, 0, 0]
    km.flag_signal(flags[1:], None, limit_ms=50)  # flag already 1: the signal gives up too
    torch.cuda.synchronize()
    assert km.device_status() == 0x100
    x = torch.ones(8, device="cuda:0")
    assert float(x.sum().item()) == 8.0
    km.close()
