"""The peer-memory move protocol of the memgraph runner, simulated on CPU.

Every rank's launch list is built by the runner's own code (with a stand-in for the kernel
manager and made-up base addresses, so no GPU is needed) and the lists are then executed by a
small simulator with the semantics of the flag kernels: `signal` blocks until the flag is 0 and
sets it to 1, `wait` blocks until it is 1 and sets it to 0, everything else completes at once.
Checked: the ranks never all block (also over repeated runs, where the flags are reused), every
flag is back at 0 at the end, a pull happens only after the producer's signal of that very run,
and a producer writes nothing over memory a peer may still be pulling from."""
import os

import pytest
import torch

from conftest import GOLDEN_DIR
from einsummable_b200 import memgraph as M

GRAPHS = os.path.join(GOLDEN_DIR, "graphs")


class _fake_km:
    def build(self, e):
        return 0


def build_program(mg, rank, world, monkeypatch):
    r = object.__new__(M.memgraph_runner_t)
    r.mg, r.folded, r.num_locs = mg, 0, mg["num_locs"]
    r.distributed, r.transport, r.wait_limit_ms = True, "p2p", 0
    r.rank, r.devices, r.kms, r.buffers = rank, {rank: 0}, {0: _fake_km()}, {}
    r.cross_moves = [n["id"] for n in mg["nodes"] if n["kind"] == "move" and n["src_loc"] != n["dst_loc"]]
    r.move_index = {nid: k for k, nid in enumerate(r.cross_moves)}
    r.flag_off = 1 << 40
    r.peer_base = [(k + 1) << 44 for k in range(world)]      # made-up, disjoint address ranges
    real_empty = torch.empty
    monkeypatch.setattr(M.torch, "empty", lambda *a, **kw: real_empty(*a, **{k: v for k, v in kw.items() if k != "device"}))
    r._prepare()
    return r


@pytest.mark.parametrize("name,world", [("llama_tiny_locs2", 2), ("llama_tiny_locs4", 4),
                                        ("llama_train_tiny_locs2", 2), ("c1_n64_locs2", 2)])
def test_flag_protocol_never_blocks_and_resets(name, world, monkeypatch):
    path = os.path.join(GRAPHS, name + ".json")
    mg = M.load_memgraph(path if os.path.exists(path) else path + ".gz")
    runners = [build_program(mg, k, world, monkeypatch) for k in range(world)]
    programs = [r.program for r in runners]
    flags = {}
    signalled_in_run = set()
    for run in range(3):
        pc = [0] * world
        signalled_in_run.clear()
        while any(pc[k] < len(programs[k]) for k in range(world)):
            progressed = False
            for k in range(world):
                while pc[k] < len(programs[k]):
                    op = programs[k][pc[k]]
                    if op[0] == "signal":
                        if flags.get(op[1], 0) != 0:
                            break
                        flags[op[1]] = 1
                        signalled_in_run.add(op[1])
                    elif op[0] == "wait":
                        if flags.get(op[1], 0) != 1:
                            break
                        assert op[1] in signalled_in_run, "a wait consumed a signal of an earlier run"
                        flags[op[1]] = 0
                    pc[k] += 1
                    progressed = True
            assert progressed, "every rank is blocked: %r" % [
                (k, programs[k][pc[k]][:2]) for k in range(world) if pc[k] < len(programs[k])]
        assert all(v == 0 for v in flags.values()), "a flag was left set after run %d" % run
    # each cross-location move appears as signal / wait+pull+signal / wait on the two ranks
    n_cross = len(runners[0].cross_moves)
    assert sum(1 for p in programs for op in p if op[0] == "pull") == n_cross
    assert sum(1 for p in programs for op in p if op[0] == "signal") == 2 * n_cross
    assert sum(1 for p in programs for op in p if op[0] == "wait") == 2 * n_cross


@pytest.mark.parametrize("name,world", [("llama_tiny_locs2", 2), ("llama_tiny_locs4", 4), ("llama_train_tiny_locs2", 2)])
def test_producer_does_not_overwrite_a_source_before_the_acknowledgement(name, world, monkeypatch):
    """Between a producer's `signal` (data ready) and its `wait` for the consumer's acknowledgement
    the consumer may be reading the source region: the producer's own launches in that window must
    not write into it."""
    path = os.path.join(GRAPHS, name + ".json")
    mg = M.load_memgraph(path if os.path.exists(path) else path + ".gz")
    moves = [n for n in mg["nodes"] if n["kind"] == "move" and n["src_loc"] != n["dst_loc"]]
    for rank in range(world):
        r = build_program(mg, rank, world, monkeypatch)
        ready = {r._flag_ptr(n["dst_loc"], 0, r.move_index[n["id"]]): n for n in moves if n["src_loc"] == rank}
        done = {r._flag_ptr(rank, 1, r.move_index[n["id"]]): n for n in moves if n["src_loc"] == rank}
        open_moves = {}
        for op in r.program:
            kind = op[0]
            if kind == "signal" and op[1] in ready:
                n = ready[op[1]]
                open_moves[n["id"]] = (n["src_offset"], n["size"])
            elif kind == "wait" and op[1] in done:
                open_moves.pop(done[op[1]]["id"])
            else:
                written = []
                if kind == "einsummable":
                    e, offs = op[2], op[3]
                    nbytes = 1
                    for d in e.out_shape():
                        nbytes *= d
                    written.append((offs[0], nbytes * {"f16": 2, "f32": 4, "f64": 8, "c64": 8}[e.out_dtype()]))
                elif kind == "touch":
                    t, offs = op[2], op[5]
                    nbytes = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}[t.dtype]
                    for d in t.selection:
                        nbytes *= d.d_out                   # the whole destination tensor
                    written.append((offs[0], nbytes))
                elif kind == "pull":
                    written.append((op[3], op[4]))
                elif kind == "move":
                    written.append((op[4], op[5]))
                for w in written:
                    for mid, src in open_moves.items():
                        assert not (w[0] < src[0] + src[1] and src[0] < w[0] + w[1]), (rank, kind, mid)
        assert not open_moves
