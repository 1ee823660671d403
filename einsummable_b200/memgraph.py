"""Runs a memgraph (the reference's per-device program of apply / touch / fill /
move nodes) on the B200 kernel layer.

This is the caller side of the boundary, kept deliberately thin: it does what
the reference's GPU exec nodes do around the kernel manager
(src/engine/gpu/exec_graph.cc:277-467) -- pointer arithmetic on one big buffer
per location, build-once / launch-many of every einsummable, the
first-touch-of-a-group-is-a-copy rule (src/engine/gpu/exec_graph.cc:167-172,
368-378), fills and moves -- in the memgraph's own node order (a valid
topological order, src/einsummable/memgraph.h:167-173), on one stream per
process.  The memgraph itself comes from the reference's compilers as a JSON
document (oracle/ref_graphs.cc writes it); nothing here plans or partitions.

Two placements of the locations:
  * single process: every location is a buffer on a device this process can see
    (several locations may share one GPU);
  * one process per GPU (torchrun): rank r owns location r; a move between
    locations is an exchange over peer-mapped memory (or an NCCL send/recv pair).

Two schedules:
  * "dag" (default): the nodes become a program of the library's executor
    (program.py): every op waits for exactly the ops it depends on -- the
    memgraph's own edges, looked through its bookkeeping nodes -- on several
    lanes, and the whole run replays as one CUDA graph;
  * "list": one stream, the memgraph's node order (what the NCCL transport uses).
"""
import gzip
import json
import os

import numpy as np
import torch

from .attention import attention_t
from .einsummable import einsummable_t, fill_t, touch_t
from .kernel_manager import kernel_manager_t
from .program import program_t
from .scalarop import DTYPE_SIZE

NP_DTYPE = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "c64": np.complex64}


def load_memgraph(path):
    opener = gzip.open if str(path).endswith(".gz") else open
    with opener(path, "rt") as f:
        return json.load(f)


def synthetic_llama_inputs(mg, seed=7):
    """Seeded synthetic inputs for the LLaMA-shape memgraph fixtures, by input name: weights and
    embeddings ~ N(0, 0.02) rounded to f16, norm weights 1, `freqs_cis` the rotary table, `labels`
    one-hot rows.  The graph's inputs come in the same order whatever the number of locations, so
    every partitioning of one graph gets the same tensors."""
    rng = np.random.default_rng(seed)
    out = {}
    for t in mg["inputs"]:
        shape, name = t["shape"], t["name"]
        if name == "freqs_cis":
            seq, half = shape
            ang = np.outer(np.arange(seq), 1.0 / (10000.0 ** (np.arange(half) / half)))
            v = (np.cos(ang) + 1j * np.sin(ang)).astype(np.complex64)
        elif name.endswith("norm.weight"):
            v = np.ones(shape, dtype=NP_DTYPE[t["dtype"]])
        elif name == "labels":
            v = np.zeros(shape, dtype=NP_DTYPE[t["dtype"]])
            v[np.arange(shape[0]), rng.integers(0, shape[1], shape[0])] = 1.0
        else:
            v = (rng.standard_normal(shape).astype(np.float32) * 0.02).astype(np.float16).astype(NP_DTYPE[t["dtype"]])
        out[name] = v
    return out


def _scalar_from_raw(raw, dtype):
    b = bytes(raw[:DTYPE_SIZE[dtype]])
    return np.frombuffer(b, dtype=NP_DTYPE[dtype])[0]


def _blocks_of(shape, partdims):
    """Yields (slices) of every block in row-major block order (vtensor_t order)."""
    starts = [np.concatenate([[0], np.cumsum(p)]) for p in partdims]
    grid = [len(p) for p in partdims]
    for flat in range(int(np.prod(grid))):
        idx = np.unravel_index(flat, grid)
        yield tuple(slice(int(starts[d][i]), int(starts[d][i + 1])) for d, i in enumerate(idx))


def move_runs(mg):
    """Run number of every move node.  A run is a stretch of move nodes that are adjacent in the
    memgraph's global order (bookkeeping nodes aside) and do not depend on one another, so a rank
    may post its members of a run as one NCCL group.  The numbering uses the whole graph only:
    every rank cuts its groups at the same places.  (Groups that straddle a cut on one rank but
    not on its peer can wait on each other for ever.)"""
    bookkeeping = BOOKKEEPING
    moved_from = {}
    runs = {}
    run_id, members = 0, set()
    for node in mg["nodes"]:
        acc = set()
        for i in node["inns"]:
            dep = mg["nodes"][i]
            if dep["kind"] == "move":
                acc.add(i)
            elif dep["kind"] in bookkeeping:
                acc |= moved_from.get(i, set())
        moved_from[node["id"]] = acc
        if node["kind"] in bookkeeping:
            continue
        if node["kind"] != "move" or (acc & members):
            run_id += 1
            members = set()
        if node["kind"] == "move":
            members.add(node["id"])
            runs[node["id"]] = run_id
    return runs

BOOKKEEPING = ("alloc", "del", "inputmem", "inputsto", "partialize")


def node_levels(mg):
    """Earliest finish time (us) of every launching node if nothing ever waited for a free GPU or link:
    the longest chain of estimated costs (unit_cost_us) that leads to it, through all locations.  The same
    on every rank; used to tell moves that become ready early from moves that become ready late."""
    nodes = mg["nodes"]
    level = {}
    for n in nodes:
        kind = n["kind"]
        start = max((level[i] for i in n["inns"]), default=0.0)
        if kind in BOOKKEEPING:
            level[n["id"]] = start
            continue
        if kind == "apply" and "attention" in n:
            u = {"kind": "attention", "node": n["id"]}
        elif kind == "apply" and "touch" in n:
            u = {"kind": "touch", "node": n["id"], "first": True}
        elif kind == "apply":
            u = {"kind": "einsummable", "node": n["id"]}
        elif kind == "constant":
            u = {"kind": "constant", "node": n["id"]}
        elif kind == "move" and n["src_loc"] != n["dst_loc"]:
            u = {"kind": "pull", "moves": [n["id"]]}
        elif kind in ("move", "copy"):
            u = {"kind": "copy", "node": n["id"]}
        else:
            u = {"kind": kind, "node": n["id"]}
        lat, work, _ = unit_cost_us(mg, u)
        level[n["id"]] = start + lat + work + (5.0 if u["kind"] == "pull" else 0.0)   # + signal and flag
    return level


# incoming moves of one run share an await (and a pull) only when their sources are expected to be ready
# within this many microseconds of each other: a shared await is as late as its latest signal
AWAIT_SPREAD_US = 12.0


def _sides(node):
    if node["kind"] == "move":
        return (node["src_loc"], node["dst_loc"])
    return (node["loc"],)


def schedule_units(mg, owned, exchange, group_sum=False):
    """The launchable units of the locations in `owned`, in the memgraph's node order, each with
    the units it depends on.

    owned: the locations this process drives.  exchange: True when a move between two locations
    is an exchange between two processes (one process per GPU) -- the source rank gets a
    `signal` unit; the destination rank an `await` unit (waits for the signal; the incoming moves of a run
    share one only where their sources are expected to be ready together, node_levels) followed by a
    `pull` unit (copies the bytes over and acknowledges), or, when the moved block is read by
    exactly one touch, by that touch as an `rtouch` unit that reads the peer's memory directly;
    and whatever later reuses the source's memory a `wait` unit for the acknowledgement.
    False when this process drives both sides and the move is a plain copy.

    Dependencies are the memgraph's edges looked through its bookkeeping nodes (alloc, del,
    inputmem, partialize: src/einsummable/memgraph.h:189-309 -- they launch nothing but carry
    the "this memory is free again" ordering).  The incoming moves of one run (move_runs) share
    an await unit and a pull unit, each one launch; the outgoing moves of a run that wait for
    the same producers share a signal unit.  Touches of one group are chained in node order, the
    first being the copy (src/engine/gpu/exec_graph.cc:167-172,368-378).

    Units are dicts: kind in {einsummable, attention, touch, rtouch, constant, copy, evict, load, signal,
    await, pull, wait, and with group_sum: rsum, ack}, `deps` (indices of earlier units), `node` and / or
    `moves` (memgraph node ids)."""
    nodes = mg["nodes"]
    owned = set(owned)
    runs = move_runs(mg)
    run_members = {}
    for nid in sorted(runs):
        run_members.setdefault(runs[nid], []).append(nid)

    def is_cross(n):
        return exchange and n["kind"] == "move" and n["src_loc"] != n["dst_loc"]

    levels = node_levels(mg) if exchange else {}

    def ready_level(m):   # when the source of move m is expected to be ready
        return max((levels[i] for i in nodes[m]["inns"]), default=0.0)

    # real nodes a bookkeeping node stands for (nodes are in topological order)
    closure = {}
    for n in nodes:
        if n["kind"] in BOOKKEEPING:
            acc = set()
            for i in n["inns"]:
                acc |= closure[i] if nodes[i]["kind"] in BOOKKEEPING else {i}
            closure[n["id"]] = frozenset(acc)

    units, unit_of, waited, group_last = [], {}, {}, {}

    # incoming moves whose bytes are read by exactly one touch: the touch reads them in place
    remote_touch = {}
    if exchange:
        users = {}
        for n in nodes:
            if n["kind"] in BOOKKEEPING:
                continue
            for i in n["inns"]:
                if is_cross(nodes[i]):
                    users.setdefault(i, []).append(n["id"])
        for m, us in users.items():
            mv = nodes[m]
            if len(us) == 1 and mv["dst_loc"] in owned:
                t = nodes[us[0]]
                if (t["kind"] == "apply" and "touch" in t and t["loc"] == mv["dst_loc"]
                        and list(t["mems"][1]) == [mv["dst_offset"], mv["size"]]
                        and sum(1 for i in t["inns"] if is_cross(nodes[i])) == 1):
                    remote_touch[m] = t["id"]
    touch_move = {t: m for m, t in remote_touch.items()}

    # group_sum: the remote adds of a partial-sum group -- whole dense blocks that arrive from
    # several peers and are added into the same tensor one after the other -- as ONE elementwise kernel
    # out = out + r1 + ... + rk over the peers' memory (plus one launch that acknowledges the k moves),
    # instead of k dependent touches of 8-12 us each.  fused_tail[touch id] = (group key, members).
    fused_tail = {}
    if exchange and group_sum:
        members_of = {}
        for n in nodes:
            if n["kind"] == "apply" and "touch" in n and n["group"] >= 0 and n["loc"] in owned:
                members_of.setdefault((n["loc"], n["group"]), []).append(n["id"])

        def dense_add(tid):
            t = nodes[tid]["touch"]
            return (tid in touch_move and t["castable"] == "add" and t["dtype"] in ("f16", "f32")
                    and all(int(d[0]) == int(d[1]) == int(d[4]) and int(d[2]) == 0 and int(d[3]) == 0 for d in t["selection"]))

        for key, ms in members_of.items():
            # never the first member (that one is the copy); the others commute, so the remote ones may
            # be added together where the last of them stands
            tail = [tid for tid in ms[1:] if dense_add(tid)]
            if 2 <= len(tail) <= 7:
                for tid in tail:
                    fused_tail[tid] = (key, tail)
    pending_tail = {}

    def raw_deps(n, side=None):
        acc = set()
        for i in n["inns"]:
            dep = nodes[i]
            if side is not None and side not in _sides(dep):
                continue
            acc |= closure[i] if dep["kind"] in BOOKKEEPING else {i}
        return acc

    def resolve(raw):
        """Unit indices for a set of real node ids; may emit one wait unit in front."""
        deps, tokens = set(), []
        for r in sorted(raw):
            dep = nodes[r]
            if is_cross(dep):
                if dep["dst_loc"] in owned:
                    deps.add(unit_of[r])
                elif dep["src_loc"] in owned:
                    if r in waited:
                        deps.add(waited[r])
                    else:
                        tokens.append(r)
            elif r in unit_of:
                deps.add(unit_of[r])
        if tokens:
            # (the acknowledgement can only follow this rank's own signal; naming that edge keeps
            # "ordered after the wait" meaning "ordered after the signal" for whoever reads the plan)
            units.append({"kind": "wait", "moves": tokens,
                          "deps": sorted({unit_of[("signal", t)] for t in tokens if ("signal", t) in unit_of})})
            for t in tokens:
                waited[t] = len(units) - 1
            deps.add(len(units) - 1)
        return sorted(deps)

    def emit(unit):
        units.append(unit)
        return len(units) - 1

    for n in nodes:
        kind, nid = n["kind"], n["id"]
        if kind in BOOKKEEPING:
            continue
        if kind == "move" and is_cross(n):
            run = run_members[runs[nid]]
            if n["dst_loc"] in owned and nid not in unit_of:
                all_members = [m for m in run if nodes[m]["dst_loc"] in owned and nodes[m]["dst_loc"] == n["dst_loc"]
                               and is_cross(nodes[m])]
                # members in the order in which their sources are expected to be ready, cut where that
                # jumps: an early tensor must not wait behind the flag of a late one
                by_level = sorted(all_members, key=lambda m: (ready_level(m), m))
                clusters = [[by_level[0]]]
                for m in by_level[1:]:
                    if ready_level(m) - ready_level(clusters[-1][0]) > AWAIT_SPREAD_US:
                        clusters.append([])
                    clusters[-1].append(m)
                for members in clusters:
                    members = sorted(members)
                    aw = emit({"kind": "await", "moves": members, "deps": [], "loc": n["dst_loc"]})
                    copied = [m for m in members if m not in remote_touch]
                    for m in members:
                        unit_of[m] = aw
                    if copied:
                        raw = set()
                        for m in copied:
                            raw |= raw_deps(nodes[m], nodes[m]["dst_loc"])
                        deps = resolve(raw)      # may put a wait unit in front
                        idx = emit({"kind": "pull", "moves": copied, "deps": sorted(set(deps) | {aw}), "loc": n["dst_loc"]})
                        for m in copied:
                            unit_of[m] = idx
            if n["src_loc"] in owned and ("signal", nid) not in unit_of:
                members = [m for m in run if nodes[m]["src_loc"] == n["src_loc"] and is_cross(nodes[m])]
                by_deps = {}
                for m in members:
                    by_deps.setdefault(tuple(resolve(raw_deps(nodes[m], n["src_loc"]))), []).append(m)
                for deps, ms in by_deps.items():
                    idx = emit({"kind": "signal", "moves": ms, "deps": list(deps), "loc": n["src_loc"]})
                    for m in ms:
                        unit_of[("signal", m)] = idx
            continue
        loc = n["dst_loc"] if kind == "move" else n["loc"]
        if loc not in owned or (kind == "move" and n["src_loc"] not in owned):
            continue
        deps = resolve(raw_deps(n))
        if kind == "apply" and "touch" in n:
            first = True
            if n["group"] >= 0:
                key = (loc, n["group"])
                first = key not in group_last
                if not first:
                    deps = sorted(set(deps) | {group_last[key]})
            if nid in fused_tail:
                key, tail = fused_tail[nid]
                acc = pending_tail.setdefault(key, set())
                acc |= set(deps)
                if nid != tail[-1]:
                    continue                      # emitted with the last member of the tail
                idx = emit({"kind": "rsum", "nodes": list(tail), "node": tail[0], "moves": [touch_move[t] for t in tail],
                            "deps": sorted(acc), "loc": loc})
                for t in tail:
                    unit_of[t] = idx
                emit({"kind": "ack", "moves": [touch_move[t] for t in tail], "deps": [idx], "loc": loc})
                group_last[key] = idx
                continue
            if nid in touch_move:
                idx = emit({"kind": "rtouch", "node": nid, "moves": [touch_move[nid]], "deps": deps, "first": first,
                            "loc": loc})
            else:
                idx = emit({"kind": "touch", "node": nid, "deps": deps, "first": first, "loc": loc})
            if n["group"] >= 0:
                group_last[(loc, n["group"])] = idx
        elif kind == "apply" and "attention" in n:
            idx = emit({"kind": "attention", "node": nid, "deps": deps, "loc": loc})
        elif kind == "apply":
            idx = emit({"kind": "einsummable", "node": nid, "deps": deps, "loc": loc})
        elif kind == "constant":
            idx = emit({"kind": "constant", "node": nid, "deps": deps, "loc": loc})
        elif kind in ("move", "copy"):
            idx = emit({"kind": "copy", "node": nid, "deps": deps, "loc": loc})
        elif kind in ("evict", "load"):
            idx = emit({"kind": kind, "node": nid, "deps": deps, "loc": loc})
        else:
            raise ValueError("unknown memgraph node kind %r" % kind)
        unit_of[nid] = idx
    # sources nobody on this rank reused: the next run may overwrite them, so the run ends by
    # collecting their acknowledgements
    rest = [n["id"] for n in nodes if is_cross(n) and n["src_loc"] in owned and n["id"] not in waited]
    if rest:
        units.append({"kind": "wait", "moves": rest,
                      "deps": sorted({unit_of[("signal", t)] for t in rest if ("signal", t) in unit_of})})
    return units

_DSIZE = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}


def unit_cost_us(mg, u):
    """(latency_us, work_us, server) of a unit for the schedule simulation: a fixed launch latency that
    overlaps with anything, and work that occupies a server -- "gpu" (HBM / tensor time, from the
    unit's algorithmic bytes and flops at round B200 rates) or "link" (NVLink into this GPU)."""
    nodes = mg["nodes"]
    k = u["kind"]
    if k == "einsummable":
        n = nodes[u["node"]]
        e = n["einsummable"]
        nbytes = sum(m[1] for m in n["mems"])
        if (len(e["inns"]) == 2 and e["castable"] == "add" and e["out_rank"] < len(e["join_shape"])
                and e["join"].startswith("*[hole")):
            flops = 2.0
            for d in e["join_shape"]:
                flops *= d
            return 5.0, max(flops / 1.25e9, nbytes / 5.0e6), "gpu"
        return 2.5, nbytes / 5.5e6, "gpu"
    if k == "attention":
        a = nodes[u["node"]]["attention"]
        flops = 4.0 * a["batch"] * a["heads"] * a["rows"] * a["keys"] * a["head_dim"] * (0.6 if a["skip_known"] else 1.0)
        return 5.0, flops / 0.6e9, "gpu"
    if k == "touch":
        n = nodes[u["node"]]
        return 2.5, n["mems"][1][1] * (2 if u["first"] else 3) / 4.5e6, "gpu"
    if k == "rtouch":
        return 6.0, nodes[u["node"]]["mems"][1][1] / 0.65e6, "link"
    if k == "rsum":
        return 6.0, sum(nodes[t]["mems"][1][1] for t in u["nodes"]) / 0.65e6, "link"
    if k == "ack":
        return 3.0, 0.0, None
    if k == "await":
        return 3.0, 0.0, None
    if k == "constant":
        return 2.5, 0.5, "gpu"
    if k == "copy":
        return 2.5, 2 * nodes[u["node"]]["size"] / 4.5e6, "gpu"
    if k in ("evict", "load"):
        return 4.0, nodes[u["node"]]["size"] / 0.05e6, "pcie"
    if k == "signal":
        return 3.0, 0.0, None
    if k == "pull":
        return 6.0, sum(nodes[m]["size"] for m in u["moves"]) / 0.65e6, "link"
    if k == "wait":
        return 2.0, 0.0, None
    raise ValueError(k)


def simulate_schedule(mg, units_by_rank):
    """Start and finish time (us) of every unit of every rank under a simple machine model: a unit
    becomes ready when its dependencies -- and, for an await, the source ranks' signals; for a wait, the
    destination ranks' pulls or remote touches -- have finished; ready units are served first come first served; each
    rank's GPU and each rank's incoming link do one unit's work at a time, launch latencies overlap.
    Deterministic (ties by rank and index), so every rank that runs it gets the same answer.
    Returns {(rank, index): (start, finish, place in the order of service)}."""
    import heapq
    sig_of, pull_of = {}, {}
    for r, units in enumerate(units_by_rank):
        for i, u in enumerate(units):
            if u["kind"] == "signal":
                for m in u["moves"]:
                    sig_of[m] = (r, i)
            elif u["kind"] in ("pull", "rtouch", "ack"):
                for m in u["moves"]:
                    pull_of[m] = (r, i)
    preds, succs, cost = {}, {}, {}
    for r, units in enumerate(units_by_rank):
        for i, u in enumerate(units):
            p = [(r, d) for d in u["deps"]]
            if u["kind"] == "await":
                p += [sig_of[m] for m in u["moves"]]
            elif u["kind"] == "wait":
                p += [pull_of[m] for m in u["moves"]]
            preds[(r, i)] = p
            cost[(r, i)] = unit_cost_us(mg, u)
            for q in p:
                succs.setdefault(q, []).append((r, i))
    # among units that become ready at the same moment the one with the longest chain of work behind
    # it goes first (its "bottom level": three projections that are ready together are launched in
    # the order of what still hangs on each, not in node order)
    order, left = [], {k: len(p) for k, p in preds.items()}
    stack = [k for k, n in left.items() if n == 0]
    while stack:
        k = stack.pop()
        order.append(k)
        for c in succs.get(k, ()):
            left[c] -= 1
            if left[c] == 0:
                stack.append(c)
    if len(order) != len(preds):
        raise RuntimeError("simulate_schedule: the units of the ranks wait for one another in a cycle")
    bottom = {}
    for k in reversed(order):
        bottom[k] = cost[k][0] + cost[k][1] + max((bottom[c] for c in succs.get(k, ())), default=0.0)
    left = {k: len(p) for k, p in preds.items()}
    ready_at = {k: 0.0 for k in preds}
    heap = [(0.0, -bottom[k], k) for k, n in left.items() if n == 0]
    heapq.heapify(heap)
    free = {}
    times = {}
    while heap:
        t, _, k = heapq.heappop(heap)
        lat, work, server = cost[k]
        begin = t + lat
        if server is not None and work > 0:
            begin = max(begin, free.get((k[0], server), 0.0))
            free[(k[0], server)] = begin + work
        fin = begin + work
        times[k] = (t, fin, len(times))     # ready time, finish, place in the global order of service
        for c in succs.get(k, ()):
            # a flag takes about 2 us to cross NVLink
            ready_at[c] = max(ready_at[c], fin + (2.0 if c[0] != k[0] else 0.0))
            left[c] -= 1
            if left[c] == 0:
                heapq.heappush(heap, (ready_at[c], -bottom[c], c))
    return times


def order_units_by_simulation(mg, world, rank, group_sum=False):
    """The units of `rank` (schedule_units) reordered by their simulated start time, dependencies
    renumbered.  Every rank simulates all ranks, so the ranks agree on when each exchange is expected:
    the pull / wait ops, which share one in-order lane, are then served in the order in which their
    data is expected to be ready instead of the memgraph's node order.  The order stays a valid one
    on every rank and across ranks: along every dependency, also those that cross ranks, the
    simulated start times strictly increase."""
    all_units = [schedule_units(mg, {r}, True, group_sum) for r in range(world)]
    times = simulate_schedule(mg, all_units)
    units = all_units[rank]
    # the closing wait (acknowledgements nobody on this rank needs during the run) stays last
    closing = len(units) - 1 if units and units[-1]["kind"] == "wait" else -1
    order = sorted(range(len(units)), key=lambda i: (i == closing, times[(rank, i)][2]))
    new_index = {old: new for new, old in enumerate(order)}
    out = []
    for old in order:
        u = dict(units[old])
        u["deps"] = sorted(new_index[d] for d in u["deps"])
        assert all(d < len(out) for d in u["deps"])
        u["sim_start_us"], u["sim_finish_us"] = times[(rank, old)][:2]
        out.append(u)
    return out


class memgraph_runner_t:
    def __init__(self, mg, devices=None, rank=None, world=None, transport="nccl", wait_limit_ms=0, fuse=False,
                 schedule="dag", max_lanes=0, order="simulated", exchange_lanes=1, group_sum=None):
        """transport (one process per GPU only): "nccl" = send/recv pairs; "p2p" = every
        location buffer lives in symmetric memory, the destination rank pulls the bytes over
        NVLink with an SM copy kernel, and the two ranks hand-shake through bounded flag
        kernels (data ready / copy finished).
        schedule: "dag" = the library's program executor (dependency-ordered lanes, see the
        module text); "list" = one stream in node order.  The NCCL transport always runs as a list."""
        # the trailing remote adds of a partial-sum group as one kernel (schedule_units); ES_B200_GROUP_SUM=1 turns it on
        self.group_sum = (os.environ.get("ES_B200_GROUP_SUM", "0") == "1") if group_sum is None else bool(group_sum)
        self.folded = 0
        self.attention_chains = 0
        if fuse:
            # elementwise producers folded into their readers, then whole attention chains into one
            # node (fuse.py); fuse="elementwise" stops after the first pass
            from .fuse import fuse_attention, fuse_elementwise_chains
            mg, self.folded = fuse_elementwise_chains(mg)
            if fuse != "elementwise":
                mg, self.attention_chains = fuse_attention(mg)
        self.mg = mg
        self.num_locs = mg["num_locs"]
        self.distributed = rank is not None
        self.transport = transport if self.distributed else "local"
        self.schedule = "list" if self.transport == "nccl" else schedule
        if self.schedule not in ("dag", "list"):
            raise ValueError("schedule must be 'dag' or 'list'")
        self.max_lanes = max_lanes
        self.exchange_lanes = exchange_lanes
        # order of the ops of one process per GPU: "simulated" = by the start times of a simulation of
        # all ranks (order_units_by_simulation), "memgraph" = the memgraph's node order
        self.order = order
        self.prog = None
        self.wait_limit_ms = wait_limit_ms
        if self.distributed:
            if world != self.num_locs:
                raise ValueError("one process per location: world size %d != %d locations" % (world, self.num_locs))
            self.rank = rank
            dev = torch.cuda.current_device()
            self.devices = {rank: dev}
        else:
            devices = devices or [0] * self.num_locs
            self.devices = {loc: devices[loc] for loc in range(self.num_locs)}
            if len(set(self.devices.values())) > 1:
                # one process driving several GPUs: the moves synchronise the devices on the host
                self.schedule = "list"
        self.kms = {}
        for loc, dev in self.devices.items():
            if dev not in self.kms:
                self.kms[dev] = kernel_manager_t(dev)
        self.buffers = {}
        if self.transport == "p2p":
            self._alloc_symmetric()
        else:
            for loc, dev in self.devices.items():
                size = int(mg["mem_sizes"][loc]) + 256
                self.buffers[loc] = torch.zeros(size, dtype=torch.uint8, device="cuda:%d" % dev)
        self._alloc_storage()
        if self.schedule == "dag":
            self._build_program()
        else:
            if self.sto_slot:
                raise RuntimeError("memgraphs with storage (evict / load) run with the dag schedule only")
            self._prepare()

    def _alloc_storage(self):
        """Memgraphs compiled under a memory limit: one pinned host arena per process, a fixed block
        in it for every storage id of this process's locations (ids are unique within a run:
        src/einsummable/memgraph.h:311-316), so evict / load are plain copies in the static schedule."""
        self.sto_slot = {}
        off = 0
        for n in self.mg["nodes"]:
            if n["kind"] in ("inputsto", "evict") and self.owns(n["loc"]):
                key = (n["storage_loc"], n["storage_id"])
                if key not in self.sto_slot:
                    self.sto_slot[key] = (off, int(n["size"]))
                    off += (int(n["size"]) + 255) // 256 * 256
        self.sto_host = torch.zeros(max(off, 256), dtype=torch.uint8).pin_memory() if off else None

    def _sto_view(self, key):
        off, size = self.sto_slot[key]
        return self.sto_host[off:off + size]

    def _alloc_symmetric(self):
        import os
        # plain peer mappings only: the exchange uses peer loads and flags, never the NVLink
        # multicast object symmetric memory would otherwise bind the buffer to (a rank that
        # exits while bound to one disturbs its peers)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.cross_moves = [n["id"] for n in self.mg["nodes"] if n["kind"] == "move" and n["src_loc"] != n["dst_loc"]]
        self.move_index = {nid: k for k, nid in enumerate(self.cross_moves)}
        nm = len(self.cross_moves)
        self.flag_off = (int(max(self.mg["mem_sizes"])) + 256 + 255) // 256 * 256
        total = self.flag_off + 8 * nm + 256
        dev = self.devices[self.rank]
        buf = symm_mem.empty(total, dtype=torch.uint8, device="cuda:%d" % dev)
        buf.zero_()
        torch.cuda.synchronize(dev)
        hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
        self.peer_base = [int(p) for p in hdl.buffer_ptrs]
        self._symm_handle = hdl
        self.buffers[self.rank] = buf
        dist.barrier()

    def _flag_ptr(self, owner_rank, kind, k):
        """kind 0: ready flag (in the destination's buffer), 1: done flag (in the source's buffer)."""
        return self.peer_base[owner_rank] + self.flag_off + 4 * (kind * len(self.cross_moves) + k)

    def owns(self, loc):
        return loc in self.devices

    def km(self, loc):
        return self.kms[self.devices[loc]]

    def ptr(self, loc, offset):
        return self.buffers[loc].data_ptr() + int(offset)


    # ------------------------------------------------------------------ build (dag)
    def _build_program(self):
        """Translates schedule_units into ops of the library's program executor."""
        nodes = self.mg["nodes"]
        if self.transport == "p2p" and self.order == "simulated":
            self.units = order_units_by_simulation(self.mg, self.num_locs, self.rank, self.group_sum)
        elif self.num_locs == 1 and self.order == "simulated":
            self.units = order_units_by_simulation(self.mg, 1, 0)
        else:
            self.units = schedule_units(self.mg, set(self.devices), self.transport == "p2p", self.group_sum)
        dev = next(iter(self.devices.values()))
        km = self.kms[dev]
        prog = program_t(km)
        self.stats = {"einsummable": 0, "touch": 0, "move": 0, "fill": 0, "move_bytes": 0}
        self.unit_labels = []
        for u in self.units:
            kind, deps = u["kind"], u["deps"]
            if kind == "einsummable":
                node = nodes[u["node"]]
                d = node["einsummable"]
                e = einsummable_t(d["join_shape"], d["inns"], d["out_rank"], d["join"], d["castable"])
                if km.build(e) is None:
                    raise RuntimeError("build returned nullopt for %r" % (e,))
                loc = node["loc"]
                offs = [m[0] for m in node["mems"]]
                prog.add_einsummable(km._built(e)[0], self.ptr(loc, offs[0]), [self.ptr(loc, o) for o in offs[1:]], deps)
                self.stats["einsummable"] += 1
                kk = km.kernel_info(e).split("|")[0]
                self.unit_labels.append(("contraction" if kk.startswith("contraction") else
                                         ("reduction" if e.has_aggregation() else "elementwise"), repr(e)))
            elif kind == "attention":
                node = nodes[u["node"]]
                a = attention_t.from_json(node["attention"])
                loc = node["loc"]
                out, q, k, v, mask = [self.ptr(loc, m[0]) for m in node["mems"]]
                prog.add_attention(a, out, q, k, v, mask, deps)
                self.stats["einsummable"] += 1
                self.unit_labels.append(("attention", "b%d h%d rows%d keys%d d%d%s" % (
                    a.batch, a.heads, a.rows, a.keys, a.head_dim, " skip" if a.skip_known else "")))
            elif kind in ("touch", "rtouch"):
                node = nodes[u["node"]]
                d = node["touch"]
                t = touch_t(d["selection"], d["castable"], d["dtype"])
                loc = node["loc"]
                offs = [m[0] for m in node["mems"]]
                if kind == "rtouch":
                    mv = nodes[u["moves"][0]]
                    prog.add_touch(t, None if u["first"] else d["castable"], self.ptr(loc, offs[0]),
                                   self.peer_base[mv["src_loc"]] + mv["src_offset"], deps,
                                   done_flag=self._flag_ptr(mv["src_loc"], 1, self.move_index[mv["id"]]))
                    self.stats["move"] += 1
                    self.stats["move_bytes"] += mv["size"]
                else:
                    prog.add_touch(t, None if u["first"] else d["castable"], self.ptr(loc, offs[0]),
                                   self.ptr(loc, offs[1]), deps)
                self.stats["touch"] += 1
                self.unit_labels.append((kind, "%s %s %d bytes" % (d["castable"], d["dtype"], node["mems"][1][1])))
            elif kind == "rsum":
                # out = out + r1 + ... + rk, the r's read in the peers' memory (generated elementwise kernel)
                first = nodes[u["nodes"][0]]
                dt = first["touch"]["dtype"]
                nelem = first["mems"][0][1] // DTYPE_SIZE[dt]
                k = len(u["nodes"])
                join = "hole|%s@0" % dt
                for i in range(1, k + 1):
                    join = "+[%s,hole|%s@%d]" % (join, dt, i)
                e = einsummable_t([nelem], [[0]] * (k + 1), 1, join, None)
                if km.build(e) is None:
                    raise RuntimeError("build returned nullopt for %r" % (e,))
                out = self.ptr(first["loc"], first["mems"][0][0])
                srcs = [self.peer_base[nodes[m]["src_loc"]] + nodes[m]["src_offset"] for m in u["moves"]]
                prog.add_einsummable(km._built(e)[0], out, [out] + srcs, deps)
                self.stats["touch"] += k
                self.stats["move"] += k
                self.stats["move_bytes"] += sum(nodes[m]["size"] for m in u["moves"])
                self.unit_labels.append(("rsum", "%d peers x %d bytes %s" % (k, first["mems"][0][1], dt)))
            elif kind == "ack":
                prog.add_signal([self._flag_ptr(nodes[m]["src_loc"], 1, self.move_index[m]) for m in u["moves"]], deps)
                self.unit_labels.append(("signal", "ack %d" % len(u["moves"])))
            elif kind == "constant":
                node = nodes[u["node"]]
                f = node["fill"]
                out = self.ptr(node["loc"], node["offset"])
                if f["type"] == "constant":
                    dt = f["value"]["dtype"]
                    prog.add_fill_constant(fill_t.constant_t(_scalar_from_raw(f["value"]["raw"], dt), [f["nelem"]], dt),
                                           out, deps)
                else:
                    dt = f["lower"]["dtype"]
                    prog.add_fill_lowertri(fill_t.lowertri_t(_scalar_from_raw(f["lower"]["raw"], dt),
                                                             _scalar_from_raw(f["upper"]["raw"], dt),
                                                             f["nrow"], f["ncol"], f["start"], dt), out, deps)
                self.stats["fill"] += 1
                self.unit_labels.append(("fill", f["type"]))
            elif kind == "copy":
                node = nodes[u["node"]]
                if node["kind"] == "move":
                    s_loc, d_loc = node["src_loc"], node["dst_loc"]
                else:
                    s_loc = d_loc = node["loc"]
                prog.add_copy(self.ptr(s_loc, node["src_offset"]), self.ptr(d_loc, node["dst_offset"]), node["size"], deps)
                self.stats["move"] += 1
                self.stats["move_bytes"] += node["size"]
                self.unit_labels.append(("copy", str(node["size"])))
            elif kind in ("evict", "load"):
                node = nodes[u["node"]]
                host = self._sto_view((node["storage_loc"], node["storage_id"]))
                dev_ptr = self.ptr(node["loc"], node["offset"])
                if kind == "evict":
                    prog.add_evict(dev_ptr, host.data_ptr(), node["size"], deps)
                else:
                    prog.add_load(host.data_ptr(), dev_ptr, node["size"], deps)
                self.stats["move"] += 1
                self.stats["move_bytes"] += node["size"]
                self.unit_labels.append((kind, "%d bytes" % node["size"]))
            elif kind == "signal":
                prog.add_signal([self._flag_ptr(nodes[m]["dst_loc"], 0, self.move_index[m]) for m in u["moves"]], deps)
                self.stats["move"] += len(u["moves"])
                self.stats["move_bytes"] += sum(nodes[m]["size"] for m in u["moves"])
                self.unit_labels.append(("signal", str(len(u["moves"]))))
            elif kind == "pull":
                items = []
                for m in u["moves"]:
                    node = nodes[m]
                    k = self.move_index[m]
                    items.append((self.peer_base[node["src_loc"]] + node["src_offset"],
                                  self.ptr(node["dst_loc"], node["dst_offset"]), node["size"],
                                  None, self._flag_ptr(node["src_loc"], 1, k)))
                prog.add_pull(items, deps)
                self.stats["move"] += len(items)
                self.stats["move_bytes"] += sum(it[2] for it in items)
                self.unit_labels.append(("pull", "%d moves %d bytes" % (len(items), sum(it[2] for it in items))))
            elif kind == "await":
                prog.add_wait([self._flag_ptr(nodes[m]["dst_loc"], 0, self.move_index[m]) for m in u["moves"]], deps)
                self.unit_labels.append(("await", str(len(u["moves"]))))
            elif kind == "wait":
                prog.add_wait([self._flag_ptr(nodes[m]["src_loc"], 1, self.move_index[m]) for m in u["moves"]], deps)
                self.unit_labels.append(("wait", str(len(u["moves"]))))
            else:
                raise ValueError(kind)
        prog.set_exchange_lanes(self.exchange_lanes)
        need = prog.finalize(self.max_lanes)
        self.workspace = {dev: (torch.empty(max(need, 256), dtype=torch.uint8, device="cuda:%d" % dev), need)}
        prog.set_workspace(self.workspace[dev][0], max(need, 256))
        if self.wait_limit_ms:
            prog.set_wait_limit(self.wait_limit_ms)
        self.prog = prog
        self.program = self.units

    def profile(self, stream=None):
        """One run with a CUDA event pair around every op: [(class, label, milliseconds)].  For await
        and wait ops the time is time spent waiting for the peer."""
        if self.prog is None:
            raise RuntimeError("profile needs the dag schedule")
        ms = self.prog.launch_timed(stream if stream is not None else torch.cuda.current_stream())
        return [(lab[0], lab[1], t) for lab, t in zip(self.unit_labels, ms)]

    def timeline(self, stream=None):
        """One replay of the captured run with the GPU's nanosecond timer read before and after every
        op: ([(class, label, start_us, end_us)], run_us), times relative to the start of the run.  An
        op's start is when its lane was free and its dependencies had finished."""
        if self.prog is None:
            raise RuntimeError("timeline needs the dag schedule")
        spans, (t0, t1) = self.prog.replay_timed(stream if stream is not None else torch.cuda.current_stream())
        return ([(lab[0], lab[1], (a - t0) / 1e3, (b - t0) / 1e3) for lab, (a, b) in zip(self.unit_labels, spans)],
                (t1 - t0) / 1e3)

    def timeline_summary(self, tl, run_us, top=12):
        """Text summary of a timeline: time per class, how long no compute op was running, and the
        chain of ops that determined the end of the run (each with the gap since its predecessor)."""
        by = {}
        for c, _, a, b in tl:
            v = by.setdefault(c, [0, 0.0])
            v[0] += 1
            v[1] += b - a
        spin = ("await", "wait")
        iv = sorted((a, b) for c, _, a, b in tl if c not in spin)
        busy, cur_a, cur_b = 0.0, None, None
        for a, b in iv:
            if cur_b is None or a > cur_b:
                if cur_b is not None:
                    busy += cur_b - cur_a
                cur_a, cur_b = a, b
            else:
                cur_b = max(cur_b, b)
        if cur_b is not None:
            busy += cur_b - cur_a
        lines = ["run %.1f us; compute lanes busy (union) %.1f us, idle %.1f us" % (run_us, busy, run_us - busy),
                 "per class (ops / summed lane time us): " +
                 "  ".join("%s %d/%.0f" % (k, v[0], v[1]) for k, v in sorted(by.items()))]
        # critical chain
        lane_prev, last = {}, {}
        d = self.prog.describe()["ops"]
        for i, op in enumerate(d):
            lane_prev[i] = last.get(op["lane"])
            last[op["lane"]] = i
        i = max(range(len(tl)), key=lambda k: tl[k][3])
        chain = []
        while i is not None:
            preds = list(self.units[i]["deps"]) + ([lane_prev[i]] if lane_prev[i] is not None else [])
            p = max(preds, key=lambda k: tl[k][3]) if preds else None
            chain.append((i, tl[i][2] - (tl[p][3] if p is not None else 0.0)))
            i = p
        chain.reverse()
        lines.append("critical chain: %d ops; per class (ops / us on the chain, gaps included):" % len(chain))
        cc = {}
        for i, gap in chain:
            v = cc.setdefault(tl[i][0], [0, 0.0, 0.0])
            v[0] += 1
            v[1] += tl[i][3] - tl[i][2]
            v[2] += max(gap, 0.0)
        lines.append("  " + "  ".join("%s %d/%.0f (+%.0f gaps)" % (k, v[0], v[1], v[2]) for k, v in sorted(cc.items())))
        for i, gap in sorted(chain, key=lambda x: -(tl[x[0]][3] - tl[x[0]][2] + max(x[1], 0)))[:top]:
            lines.append("  at %7.1f us: %-11s %6.1f us (gap %5.1f)  %s" % (tl[i][2], tl[i][0], tl[i][3] - tl[i][2], gap,
                                                                       tl[i][1][:90]))
        return "\n".join(lines)

    # ------------------------------------------------------------------ build (list)
    def _prepare(self):
        self.program = []
        ws_need = {loc: 0 for loc in self.devices}
        self.stats = {"einsummable": 0, "touch": 0, "move": 0, "fill": 0, "move_bytes": 0}
        move_run = move_runs(self.mg) if self.transport == "nccl" else {}
        # p2p transport: a source rank must not touch memory a peer is still reading.  For every
        # node, the set of this rank's outgoing moves it depends on through chains of bookkeeping
        # nodes (del -> alloc -> ...); before such a node runs the move's "done" flag is awaited.
        self._pending_done = set()
        waits_for = {}
        if self.transport == "p2p":
            bookkeeping = ("alloc", "del", "inputmem", "partialize")
            for node in self.mg["nodes"]:
                acc = set()
                for i in node["inns"]:
                    dep = self.mg["nodes"][i]
                    if dep["kind"] == "move" and dep["src_loc"] != dep["dst_loc"] and dep["src_loc"] == self.rank:
                        acc.add(i)
                    elif dep["kind"] in bookkeeping:
                        acc |= waits_for.get(i, set())
                waits_for[node["id"]] = acc
        for node in self.mg["nodes"]:
            kind = node["kind"]
            # bookkeeping nodes do not break a run of moves
            if kind in ("alloc", "del", "inputmem", "partialize"):
                continue
            if self.transport == "p2p":
                node_loc = node.get("loc", node.get("dst_loc"))
                mine = node_loc == self.rank or (kind == "move" and node["src_loc"] == self.rank)
                if mine:
                    for mid in sorted(waits_for.get(node["id"], ())):
                        if mid in self._pending_done:
                            self.program.append(("wait", self._flag_ptr(self.rank, 1, self.move_index[mid])))
                            self._pending_done.discard(mid)
            if kind == "apply":
                loc = node["loc"]
                if not self.owns(loc):
                    continue
                if "attention" in node:
                    self.program.append(("attention", loc, attention_t.from_json(node["attention"]),
                                         [m[0] for m in node["mems"]]))
                    self.stats["einsummable"] += 1
                elif "einsummable" in node:
                    d = node["einsummable"]
                    e = einsummable_t(d["join_shape"], d["inns"], d["out_rank"], d["join"], d["castable"])
                    ws = self.km(loc).build(e)
                    if ws is None:
                        raise RuntimeError("build returned nullopt for %r" % (e,))
                    ws_need[loc] = max(ws_need[loc], ws)
                    self.program.append(("einsummable", loc, e, [m[0] for m in node["mems"]], ws))
                    self.stats["einsummable"] += 1
                else:
                    d = node["touch"]
                    t = touch_t(d["selection"], d["castable"], d["dtype"])
                    t_copy = touch_t(d["selection"], None, d["dtype"])
                    self.program.append(("touch", loc, t, t_copy, node["group"], [m[0] for m in node["mems"]]))
                    self.stats["touch"] += 1
            elif kind == "constant":
                if not self.owns(node["loc"]):
                    continue
                f = node["fill"]
                if f["type"] == "constant":
                    dt = f["value"]["dtype"]
                    fill = fill_t.constant_t(_scalar_from_raw(f["value"]["raw"], dt), [f["nelem"]], dt)
                    self.program.append(("constant_fill", node["loc"], fill, node["offset"]))
                else:
                    dt = f["lower"]["dtype"]
                    fill = fill_t.lowertri_t(_scalar_from_raw(f["lower"]["raw"], dt),
                                             _scalar_from_raw(f["upper"]["raw"], dt), f["nrow"], f["ncol"],
                                             f["start"], dt)
                    self.program.append(("lowertri_fill", node["loc"], fill, node["offset"]))
                self.stats["fill"] += 1
            elif kind == "move":
                s, d = node["src_loc"], node["dst_loc"]
                if self.owns(s) or self.owns(d):
                    mv = ("move", s, node["src_offset"], d, node["dst_offset"], node["size"])
                    if self.transport == "p2p" and s != d:
                        k = self.move_index[node["id"]]
                        if self.rank == s:
                            self.program.append(("signal", self._flag_ptr(d, 0, k)))
                            self._pending_done.add(node["id"])
                        else:
                            self.program.append(("wait", self._flag_ptr(d, 0, k)))
                            self.program.append(("pull", self.peer_base[s] + node["src_offset"], d, node["dst_offset"],
                                                 node["size"]))
                            self.program.append(("signal", self._flag_ptr(s, 1, k)))
                    # The cross-rank members of one run (move_runs) are posted as one NCCL group.
                    elif (self.distributed and s != d and self.program and self.program[-1][0] == "move_batch"
                            and self.program[-1][2] == move_run[node["id"]]):
                        self.program[-1][1].append(mv)
                    elif self.distributed and s != d:
                        self.program.append(("move_batch", [mv], move_run[node["id"]]))
                    elif (self.distributed and self.program and self.program[-1][0] == "move_batch"
                            and self.program[-1][2] == move_run.get(node["id"])):
                        # a local copy inside a run: members of a run are independent, so it goes in
                        # front of the group instead of splitting it on this rank only
                        self.program.insert(len(self.program) - 1, mv)
                    else:
                        self.program.append(mv)
                    self.stats["move"] += 1
                    self.stats["move_bytes"] += node["size"]
            elif kind == "copy":
                if self.owns(node["loc"]):
                    self.program.append(("move", node["loc"], node["src_offset"], node["loc"], node["dst_offset"],
                                         node["size"]))
            # inputmem, alloc, del, partialize: bookkeeping nodes, nothing to launch
        # outgoing moves nobody on this rank depended on: their sources may be overwritten by the next
        # run, so the run ends by collecting their "done" flags (which also leaves every flag at zero)
        for mid in sorted(self._pending_done):
            self.program.append(("wait", self._flag_ptr(self.rank, 1, self.move_index[mid])))
        self._pending_done = set()
        self.workspace = {}
        for loc, need in ws_need.items():
            dev = self.devices[loc]
            self.workspace[loc] = (torch.empty(max(need, 16), dtype=torch.uint8, device="cuda:%d" % dev), need)

    # ------------------------------------------------------------------ data
    def _tensor_desc(self, which, key):
        for t in self.mg[which]:
            if t["gid"] == key or t["name"] == key:
                return t
        raise KeyError(key)

    def set_input(self, key, array):
        t = self._tensor_desc("inputs", key)
        a = np.ascontiguousarray(array, dtype=NP_DTYPE[t["dtype"]]).reshape(t["shape"])
        for blk, sl in zip(t["blocks"], _blocks_of(t["shape"], t["partdims"])):
            if not self.owns(blk["loc"]):
                continue
            raw = np.ascontiguousarray(a[sl]).view(np.uint8).reshape(-1)
            assert raw.size == blk["size"], (raw.size, blk)
            if "sto_id" in blk:       # this block starts out in storage
                self._sto_view((blk["sto_loc"], blk["sto_id"])).copy_(torch.from_numpy(raw))
                continue
            self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]].copy_(torch.from_numpy(raw))

    def get_output(self, key):
        """The saved tensor assembled from its blocks (blocks on other ranks are left zero)."""
        t = self._tensor_desc("outputs", key)
        out = np.zeros(t["shape"], dtype=NP_DTYPE[t["dtype"]])
        for blk, sl in zip(t["blocks"], _blocks_of(t["shape"], t["partdims"])):
            if not self.owns(blk["loc"]):
                continue
            if "sto_id" in blk:       # the saved block ended up in storage (synchronise before reading)
                raw = self._sto_view((blk["sto_loc"], blk["sto_id"])).numpy().copy()
            else:
                raw = self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]].cpu().numpy()
            out[sl] = raw.view(NP_DTYPE[t["dtype"]]).reshape(out[sl].shape)
        return out

    def stage_input(self, key, array):
        """Pinned host copies of this process's blocks of input `key`, each with the device slice it
        belongs to: [(host tensor, device tensor)].  `device.copy_(host, non_blocking=True)` on the
        stream of the run then is the host-to-device copy of that input."""
        t = self._tensor_desc("inputs", key)
        a = np.ascontiguousarray(array, dtype=NP_DTYPE[t["dtype"]]).reshape(t["shape"])
        pairs = []
        for blk, sl in zip(t["blocks"], _blocks_of(t["shape"], t["partdims"])):
            if not self.owns(blk["loc"]):
                continue
            raw = np.ascontiguousarray(a[sl]).view(np.uint8).reshape(-1)
            host = torch.from_numpy(raw.copy()).pin_memory()
            pairs.append((host, self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]]))
        return pairs

    def stage_output(self, key):
        """Pinned host buffers for this process's blocks of saved tensor `key`: [(host, device)]."""
        t = self._tensor_desc("outputs", key)
        pairs = []
        for blk in t["blocks"]:
            if not self.owns(blk["loc"]):
                continue
            host = torch.empty(blk["size"], dtype=torch.uint8).pin_memory()
            pairs.append((host, self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]]))
        return pairs

    # ------------------------------------------------------------------ run
    def run(self, stream=None):
        """Launches the whole program; asynchronous on `stream` (default: torch's
        current stream of the first device)."""
        if stream is None:
            stream = torch.cuda.current_stream(next(iter(self.devices.values())))
        if self.prog is not None:
            self.prog.launch(stream)
            return
        groups_touched = set()
        for op in self.program:
            kind = op[0]
            if kind == "einsummable":
                _, loc, e, offs, ws = op
                w = self.workspace[loc]
                self.km(loc)(e, self._stream(loc, stream), self.ptr(loc, offs[0]),
                             [self.ptr(loc, o) for o in offs[1:]], (w[0], w[1]) if ws else None)
            elif kind == "attention":
                _, loc, a, offs = op
                self.km(loc).attention(a, self._stream(loc, stream), *[self.ptr(loc, o) for o in offs])
            elif kind == "touch":
                _, loc, t, t_copy, group, offs = op
                first = group < 0 or (loc, group) not in groups_touched
                if group >= 0:
                    groups_touched.add((loc, group))
                self.km(loc)(t_copy if first else t, self._stream(loc, stream), self.ptr(loc, offs[0]),
                             self.ptr(loc, offs[1]))
            elif kind == "constant_fill":
                _, loc, fill, off = op
                self.km(loc).constant_fill(fill, self._stream(loc, stream), self.ptr(loc, off))
            elif kind == "lowertri_fill":
                _, loc, fill, off = op
                self.km(loc).lowerTri_fill(fill, self._stream(loc, stream), self.ptr(loc, off))
            elif kind == "move":
                self._move(op, stream)
            elif kind == "move_batch":
                self._move_batch(op[1])
            elif kind == "signal":
                self.km(self.rank).flag_signal(op[1], stream, self.wait_limit_ms)
            elif kind == "wait":
                self.km(self.rank).flag_wait(op[1], stream, self.wait_limit_ms)
            elif kind == "pull":
                _, src_ptr, d, d_off, size = op
                self.km(d).pull(src_ptr, self.ptr(d, d_off), size, stream)

    def _stream(self, loc, stream):
        return stream

    def _move(self, op, stream):
        _, s, s_off, d, d_off, size = op
        if not self.distributed:
            if self.devices[s] != self.devices[d]:
                # single process, two GPUs, one stream per device would need events; the
                # single-process mode is for locations that share a device or for tests
                torch.cuda.synchronize(self.devices[s])
            self.km(d).move(self.devices[s], self.ptr(s, s_off), self.ptr(d, d_off), size, stream)
            if self.devices[s] != self.devices[d]:
                torch.cuda.synchronize(self.devices[d])
            return
        import torch.distributed as dist
        if s == d:
            self.km(d).move(self.devices[s], self.ptr(s, s_off), self.ptr(d, d_off), size, stream)
        elif self.rank == s:
            dist.send(self.buffers[s][s_off:s_off + size], dst=d)
        elif self.rank == d:
            dist.recv(self.buffers[d][d_off:d_off + size], src=s)

    def _move_batch(self, moves):
        import torch.distributed as dist
        ops = []
        for (_, s, s_off, d, d_off, size) in moves:
            if self.rank == s:
                ops.append(dist.P2POp(dist.isend, self.buffers[s][s_off:s_off + size], d))
            else:
                ops.append(dist.P2POp(dist.irecv, self.buffers[d][d_off:d_off + size], s))
        for w in dist.batch_isend_irecv(ops):
            w.wait()  # stream-ordered for NCCL: does not block the host

    def capture(self):
        """Captures one run of the program into a CUDA graph (after two eager warm-up
        runs): a layer is a few hundred sub-millisecond launches, so replaying a graph
        removes the per-node host round trip the reference pays through
        cudaStreamAddCallback (src/engine/gpu/exec_graph.cc:318-332)."""
        self.run()
        self.run()
        for dev in set(self.devices.values()):
            torch.cuda.synchronize(dev)
        if self.prog is not None:
            self.prog.instantiate()
            self.graph = self.prog
            return self.prog
        if self.transport == "nccl":
            # captured NCCL send / recv nodes did not shut down cleanly on this stack: replay() runs the list
            self.graph = None
            return None
        if len(set(self.devices.values())) > 1:
            raise RuntimeError("capture: one process driving several GPUs runs as a list and is not captured")
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.run(torch.cuda.current_stream())
        self.graph = g
        return g

    def replay(self, stream=None):
        if self.prog is not None:
            self.prog.replay(stream if stream is not None else torch.cuda.current_stream())
        elif self.graph is None:
            self.run(stream)
        else:
            self.graph.replay()

    def kernel_kinds(self):
        """How many einsummable ops run as which kernel kind (contraction_tc_f16, ew_vec, red_row, ...)."""
        kinds = {}
        if self.prog is not None:
            for u in self.units:
                if u["kind"] == "einsummable":
                    node = self.mg["nodes"][u["node"]]
                    d = node["einsummable"]
                    e = einsummable_t(d["join_shape"], d["inns"], d["out_rank"], d["join"], d["castable"])
                    k = self.km(node["loc"]).kernel_info(e).split("|")[0]
                    kinds[k] = kinds.get(k, 0) + 1
                elif u["kind"] == "attention":
                    kinds["attention_tc_f16"] = kinds.get("attention_tc_f16", 0) + 1
        else:
            for op in self.program:
                if op[0] == "einsummable":
                    k = self.km(op[1]).kernel_info(op[2]).split("|")[0]
                    kinds[k] = kinds.get(k, 0) + 1
                elif op[0] == "attention":
                    kinds["attention_tc_f16"] = kinds.get("attention_tc_f16", 0) + 1
        return kinds

    def device_status(self):
        return max(km.device_status() for km in self.kms.values())

    def close(self):
        if self.prog is not None:
            self.prog.close()
            self.prog = None
        for km in self.kms.values():
            km.close()
