"""The dependency-ordered schedule of the memgraph runner, checked on CPU.

schedule_units (einsummable_b200/memgraph.py) turns a memgraph into units with dependencies; the
library's program executor (es_b200_program_*, created here without a device: planning only)
assigns them to lanes and decides which events each op waits for.  Checked on the real plans:

  * every dependency of every op is implied by lane order plus the events it waits for;
  * no two ops of one process that touch overlapping memory (at least one writing) are left
    unordered -- i.e. the memgraph's edges, looked through its bookkeeping nodes, carry every
    hazard, including the reuse of freed memory;
  * exchange between ranks: a source region is not written between its `signal` and the
    acknowledgement `wait`; simulated over repeated runs with the kernels' semantics (run
    counters in the flags, the ops that wait for a peer on one in-order lane) no rank ever blocks
    for good, and every pull or in-place touch reads what the source rank signalled in that very run.
"""
import os

import pytest

from conftest import GOLDEN_DIR
from einsummable_b200 import memgraph as M
from einsummable_b200.einsummable import touch_t
from einsummable_b200.program import program_t

GRAPHS = os.path.join(GOLDEN_DIR, "graphs")
BASE = 1 << 40          # made-up buffer addresses, one range per location
FLAGS = 1 << 36         # offset of the flag words inside a location's range


def load(name):
    path = os.path.join(GRAPHS, name + ".json")
    return M.load_memgraph(path if os.path.exists(path) else path + ".gz")


def ptr(loc, off):
    return (loc + 1) * BASE + off


def plan(mg, owned, exchange, max_lanes=8, order="memgraph", exchange_lanes=1, group_sum=False):
    """(units, described schedule) of the program a runner would build for `owned`; order
    "simulated": the units of one rank sorted by the start times of the all-rank simulation."""
    nodes = mg["nodes"]
    if order == "simulated":
        (rank,) = owned
        units = M.order_units_by_simulation(mg, mg["num_locs"], rank, group_sum)
    else:
        units = M.schedule_units(mg, owned, exchange, group_sum)
    cross = [n["id"] for n in nodes if n["kind"] == "move" and n["src_loc"] != n["dst_loc"]]
    index = {m: k for k, m in enumerate(cross)}

    def flag(loc, kind, m):
        return ptr(loc, FLAGS + 4 * (kind * len(cross) + index[m]))

    prog = program_t(None)
    for u in units:
        k, deps = u["kind"], u["deps"]
        if k == "einsummable":
            n = nodes[u["node"]]
            offs = [m[0] for m in n["mems"]]
            prog.add_einsummable(0, ptr(n["loc"], offs[0]), [ptr(n["loc"], o) for o in offs[1:]], deps)
        elif k == "attention":
            from einsummable_b200.attention import attention_t
            n = nodes[u["node"]]
            prog.add_attention(attention_t.from_json(n["attention"]), *[ptr(n["loc"], m[0]) for m in n["mems"]], deps)
        elif k in ("touch", "rtouch"):
            n = nodes[u["node"]]
            d = n["touch"]
            t = touch_t(d["selection"], d["castable"], d["dtype"])
            if k == "rtouch":
                m = nodes[u["moves"][0]]
                prog.add_touch(t, None if u["first"] else d["castable"], ptr(n["loc"], n["mems"][0][0]),
                               ptr(m["src_loc"], m["src_offset"]), deps, done_flag=flag(m["src_loc"], 1, m["id"]))
            else:
                prog.add_touch(t, None if u["first"] else d["castable"], ptr(n["loc"], n["mems"][0][0]),
                               ptr(n["loc"], n["mems"][1][0]), deps)
        elif k == "constant":
            n = nodes[u["node"]]
            prog.add_copy(ptr(n["loc"], 0), ptr(n["loc"], n["offset"]), 16, deps)   # stand-in op, same deps
        elif k == "copy":
            n = nodes[u["node"]]
            s, d = (n["src_loc"], n["dst_loc"]) if n["kind"] == "move" else (n["loc"], n["loc"])
            prog.add_copy(ptr(s, n["src_offset"]), ptr(d, n["dst_offset"]), n["size"], deps)
        elif k in ("evict", "load"):
            n = nodes[u["node"]]
            host = (1 << 50) + 4096 * n["storage_id"]
            if k == "evict":
                prog.add_evict(ptr(n["loc"], n["offset"]), host, n["size"], deps)
            else:
                prog.add_load(host, ptr(n["loc"], n["offset"]), n["size"], deps)
        elif k == "rsum":
            n = nodes[u["nodes"][0]]
            out = ptr(n["loc"], n["mems"][0][0])
            prog.add_einsummable(0, out, [out] + [ptr(nodes[m]["src_loc"], nodes[m]["src_offset"]) for m in u["moves"]], deps)
        elif k == "ack":
            prog.add_signal([flag(nodes[m]["src_loc"], 1, m) for m in u["moves"]], deps)
        elif k == "signal":
            prog.add_signal([flag(nodes[m]["dst_loc"], 0, m) for m in u["moves"]], deps)
        elif k == "await":
            prog.add_wait([flag(nodes[m]["dst_loc"], 0, m) for m in u["moves"]], deps)
        elif k == "pull":
            prog.add_pull([(ptr(nodes[m]["src_loc"], nodes[m]["src_offset"]),
                            ptr(nodes[m]["dst_loc"], nodes[m]["dst_offset"]), nodes[m]["size"],
                            None, flag(nodes[m]["src_loc"], 1, m)) for m in u["moves"]], deps)
        elif k == "wait":
            prog.add_wait([flag(nodes[m]["src_loc"], 1, m) for m in u["moves"]], deps)
    prog.set_exchange_lanes(exchange_lanes)
    prog.finalize(max_lanes)
    d = prog.describe()
    prog.close()
    assert len(d["ops"]) == len(units)
    return units, d


def happens_before(d):
    """hb[i] = bitset of the ops known to be complete when op i starts."""
    ops = d["ops"]
    last, hb = {}, []
    for i, op in enumerate(ops):
        acc = 0
        pred = ([last[op["lane"]]] if op["lane"] in last else []) + op["wait_on"]
        for p in pred:
            assert p < i
            acc |= hb[p] | (1 << p)
        hb.append(acc)
        last[op["lane"]] = i
    return hb


def regions(mg, u):
    """(reads, writes) of a unit: lists of (loc, lo, hi, box) with box = (tensor key, per-dim
    (offset, size)) for a touch's destination so that touches of disjoint blocks of one tensor
    do not count as a conflict."""
    nodes = mg["nodes"]
    k = u["kind"]
    if k in ("einsummable", "attention"):
        n = nodes[u["node"]]
        mems = n["mems"]
        return ([(n["loc"], m[0], m[0] + m[1], None) for m in mems[1:]],
                [(n["loc"], mems[0][0], mems[0][0] + mems[0][1], None)])
    if k in ("touch", "rtouch"):
        n = nodes[u["node"]]
        mems, sel = n["mems"], n["touch"]["selection"]
        box = ((n["loc"], mems[0][0], tuple(s[1] for s in sel)), tuple((s[3], s[4]) for s in sel))
        out = (n["loc"], mems[0][0], mems[0][0] + mems[0][1], box)
        # an rtouch reads the source rank's memory (guarded by the signal / acknowledgement pair)
        reads = [(n["loc"], mems[1][0], mems[1][0] + mems[1][1], None)] if k == "touch" else []
        if not u["first"]:
            reads.append(out)
        return reads, [out]
    if k == "rsum":     # out += peers' blocks (read in the peers' memory under the signal / acknowledgement pair)
        n = nodes[u["nodes"][0]]
        out = (n["loc"], n["mems"][0][0], n["mems"][0][0] + n["mems"][0][1], None)
        return [out], [out]
    if k == "constant":
        n = nodes[u["node"]]
        f = n["fill"]
        size = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}[(f.get("value") or f["lower"])["dtype"]]
        nelem = f["nelem"] if f["type"] == "constant" else f["nrow"] * f["ncol"]
        return [], [(n["loc"], n["offset"], n["offset"] + nelem * size, None)]
    if k == "copy":
        n = nodes[u["node"]]
        s, d = (n["src_loc"], n["dst_loc"]) if n["kind"] == "move" else (n["loc"], n["loc"])
        return ([(s, n["src_offset"], n["src_offset"] + n["size"], None)],
                [(d, n["dst_offset"], n["dst_offset"] + n["size"], None)])
    if k in ("evict", "load"):      # the storage id's host block stands in as a region of its own
        n = nodes[u["node"]]
        dev = (n["loc"], n["offset"], n["offset"] + n["size"], None)
        sto = (("sto", n["storage_loc"]), n["storage_id"], n["storage_id"] + 1, None)
        return ([dev], [sto]) if k == "evict" else ([sto], [dev])
    if k == "pull":
        return [], [(nodes[m]["dst_loc"], nodes[m]["dst_offset"], nodes[m]["dst_offset"] + nodes[m]["size"], None)
                    for m in u["moves"]]
    if k == "signal":   # the peer reads the sources from now on
        return [(nodes[m]["src_loc"], nodes[m]["src_offset"], nodes[m]["src_offset"] + nodes[m]["size"], None)
                for m in u["moves"]], []
    return [], []


def overlap(a, b):
    if a[0] != b[0] or not (a[1] < b[2] and b[1] < a[2]):
        return False
    if a[3] is not None and b[3] is not None and a[3][0] == b[3][0]:
        return all(x[0] < y[0] + y[1] and y[0] < x[0] + x[1] for x, y in zip(a[3][1], b[3][1]))
    return True


def check_plan(mg, units, d):
    hb = happens_before(d)
    ops = d["ops"]
    for i, op in enumerate(ops):
        for dep in op["deps"]:
            assert hb[i] >> dep & 1, "op %d starts without its dependency %d" % (i, dep)
    rw = [regions(mg, u) for u in units]
    for j in range(len(units)):
        for i in range(j):
            if hb[j] >> i & 1:
                continue
            (ri, wi), (rj, wj) = rw[i], rw[j]
            for w in wi:
                for x in rj + wj:
                    assert not overlap(w, x), ("unordered hazard", i, units[i], j, units[j])
            for w in wj:
                for x in ri:
                    assert not overlap(w, x), ("unordered hazard", i, units[i], j, units[j])
    return hb


SMALL = [("c1_n64_evict_locs1", 1), ("c1_n64_evict_locs2", 2), ("c1_n64_locs2", 2), ("llama_tiny_locs2", 2), ("llama_tiny_locs4", 4), ("llama_train_tiny_locs2", 2),
         ("llama_train_adamw_tiny_locs2", 2), ("llama_tiny_tp_locs2", 2), ("llama_tiny_tp_locs4", 4)]
# the layer under the reference's autoplace01 and under the hand-written tensor-parallel placement
LARGE = [("llama7b_layer_locs1", 1), ("llama7b_layer_locs2", 2), ("llama7b_layer_locs4", 4), ("llama7b_layer_locs8", 8),
         ("llama7b_layer_tp_locs2", 2), ("llama7b_layer_tp_locs4", 4), ("llama7b_layer_tp_locs8", 8)]


@pytest.mark.parametrize("name,world", SMALL + LARGE)
@pytest.mark.parametrize("lanes", [1, 8])
def test_single_process_schedule_has_no_unordered_hazard(name, world, lanes):
    mg = load(name)
    units, d = plan(mg, set(range(world)), False, lanes)
    assert d["n_lanes"] <= lanes
    check_plan(mg, units, d)


@pytest.mark.parametrize("name,world", SMALL + LARGE)
def test_folded_graphs_stay_hazard_free_under_dependency_order(name, world):
    """The fold pass moves reads (a reader now reads its folded producer's inputs): later writers
    into that memory must have been made to wait for the reader."""
    from einsummable_b200.fuse import fuse_attention, fuse_elementwise_chains
    mg, folded = fuse_elementwise_chains(load(name))
    if not name.startswith("c1"):
        assert folded > 0
    mg, chains = fuse_attention(mg)
    if name.startswith("llama7b_layer"):
        # the five nodes of every attention block of the layer graphs become one
        assert chains == {1: 1, 2: 2, 4: 4, 8: 8}[world]
        assert sum(1 for n in mg["nodes"] if "attention" in n) == chains
    units, d = plan(mg, set(range(world)), False, 8)
    check_plan(mg, units, d)
    for rank in range(world if world > 1 else 0):
        units, d = plan(mg, {rank}, True)
        check_plan(mg, units, d)


@pytest.mark.parametrize("order", ["memgraph", "simulated"])
@pytest.mark.parametrize("name,world", SMALL[1:] + LARGE[1:])
def test_per_rank_schedules_order_every_hazard_and_protect_sources(name, world, order):
    mg = load(name)
    nodes = mg["nodes"]
    for rank in range(world):
        units, d = plan(mg, {rank}, True, order=order)
        hb = check_plan(mg, units, d)
        # the ops that wait for a peer have the exchange lane to themselves
        assert d["n_exchange_lanes"] == 1
        for u, op in zip(units, d["ops"]):
            assert (op["lane"] == 0) == (u["kind"] in ("await", "wait")), (u, op)
        # a source region: written only before its signal or after the acknowledgement
        sig, ack = {}, {}
        for i, u in enumerate(units):
            if u["kind"] == "signal":
                sig.update({m: i for m in u["moves"]})
            elif u["kind"] == "wait":
                ack.update({m: i for m in u["moves"]})
        assert set(sig) == set(ack) == {n["id"] for n in nodes if n["kind"] == "move"
                                        and n["src_loc"] == rank and n["dst_loc"] != rank}
        rw = [regions(mg, u) for u in units]
        for m, s in sig.items():
            src = (rank, nodes[m]["src_offset"], nodes[m]["src_offset"] + nodes[m]["size"], None)
            for i, (_, writes) in enumerate(rw):
                if i == s or not any(overlap(src, w) for w in writes):
                    continue
                assert (hb[s] >> i & 1) or (hb[i] >> ack[m] & 1) or i == ack[m], \
                    ("source of move %d written while a peer may read it" % m, units[i])


@pytest.mark.parametrize("exchange_lanes", [1, 4])
@pytest.mark.parametrize("order", ["memgraph", "simulated"])
@pytest.mark.parametrize("name,world", SMALL[1:] + LARGE[1:])
def test_exchange_never_blocks_over_repeated_runs(name, world, order, exchange_lanes):
    """All ranks' programs executed together with the kernels' semantics: an op starts when the
    op before it on its lane and the ops it waits for have finished; a pull finishes when every
    member's ready flag has reached the rank's run number and then raises the done flags; a wait
    finishes when its done flags have.  Also: a pull only ever sees a flag of its own run."""
    mg = load(name)
    nodes = mg["nodes"]
    plans = [plan(mg, {r}, True, order=order, exchange_lanes=exchange_lanes) for r in range(world)]
    ready, done = {}, {}
    for run in range(1, 4):
        finished = [set() for _ in range(world)]
        heads = []
        for r in range(world):
            lanes = {}
            for i, op in enumerate(plans[r][1]["ops"]):
                lanes.setdefault(op["lane"], []).append(i)
            heads.append(lanes)
        remaining = sum(len(p[0]) for p in plans)
        while remaining:
            progressed = False
            for r in range(world):
                units, d = plans[r]
                for lane, queue in heads[r].items():
                    while queue:
                        i = queue[0]
                        if not all(w in finished[r] for w in d["ops"][i]["wait_on"]):
                            break
                        u = units[i]
                        if u["kind"] == "await":
                            if not all(ready.get(m, 0) >= run for m in u["moves"]):
                                break
                            assert all(ready[m] == run for m in u["moves"]), "an await saw a flag of another run"
                        elif u["kind"] == "rsum":
                            assert all(ready.get(m, 0) == run for m in u["moves"]), "bytes read before their signal"
                        elif u["kind"] in ("pull", "rtouch", "ack"):
                            assert all(ready.get(m, 0) == run for m in u["moves"]), "bytes read before their signal"
                            for m in u["moves"]:
                                done[m] = run
                        elif u["kind"] == "wait":
                            if not all(done.get(m, 0) >= run for m in u["moves"]):
                                break
                        elif u["kind"] == "signal":
                            for m in u["moves"]:
                                assert ready.get(m, 0) == run - 1
                                ready[m] = run
                        finished[r].add(i)
                        queue.pop(0)
                        remaining -= 1
                        progressed = True
            assert progressed, "every rank is blocked in run %d" % run
        n_cross = sum(1 for n in nodes if n["kind"] == "move" and n["src_loc"] != n["dst_loc"])
        assert len(ready) == len(done) == n_cross and set(ready.values()) == set(done.values()) == {run}


def test_exchange_ops_come_in_the_same_global_order_on_every_rank():
    """pull and wait units are keyed by the memgraph node that needs them; every rank lists its
    own in increasing key order (what makes the single in-order exchange lane safe)."""
    mg = load("llama7b_layer_locs8")
    for rank in range(8):
        units = M.schedule_units(mg, {rank}, True)
        # runs in memgraph order; inside a run (its moves do not depend on one another) the awaits in the
        # order in which their sources are expected to be ready -- a function of the graph alone
        runs = M.move_runs(mg)
        levels = M.node_levels(mg)
        ready = lambda m: max((levels[i] for i in mg["nodes"][m]["inns"]), default=0.0)  # noqa: E731
        keys = [(runs[u["moves"][0]], min(ready(m) for m in u["moves"])) for u in units if u["kind"] == "await"]
        assert keys == sorted(keys)
        # an await never spans sources expected more than the spread apart
        for u in units:
            if u["kind"] == "await":
                assert max(ready(m) for m in u["moves"]) - min(ready(m) for m in u["moves"]) <= M.AWAIT_SPREAD_US
        # the incoming moves of one run share a unit where their sources come together; units never mix runs
        for u in units:
            if u["kind"] in ("await", "pull"):
                assert len({runs[m] for m in u["moves"]}) == 1
        # every incoming move is read exactly once: by a pull or by a touch in place
        read = [m for u in units if u["kind"] in ("pull", "rtouch") for m in u["moves"]]
        assert sorted(read) == sorted(n["id"] for n in mg["nodes"] if n["kind"] == "move"
                                      and n["dst_loc"] == rank and n["src_loc"] != rank)
        assert sum(1 for u in units if u["kind"] == "rtouch") >= 10


def all_ranks_stay_live(plans, world, runs=2):
    """Every rank's program executed together with the kernels' semantics for a few runs: an op starts when
    the op before it on its lane and the ops it waits for have finished; an await passes when its flags have
    reached the run number, a wait when the acknowledgements have; whoever reads a move sees the flag of the
    same run."""
    ready, done = {}, {}
    for run in range(1, runs + 1):
        finished = [set() for _ in range(world)]
        queues = []
        for r in range(world):
            lanes = {}
            for i, op in enumerate(plans[r][1]["ops"]):
                lanes.setdefault(op["lane"], []).append(i)
            queues.append(lanes)
        remaining = sum(len(p[0]) for p in plans)
        while remaining:
            progressed = False
            for r in range(world):
                units, d = plans[r]
                for lane, queue in queues[r].items():
                    while queue:
                        i = queue[0]
                        if not all(w in finished[r] for w in d["ops"][i]["wait_on"]):
                            break
                        u = units[i]
                        if u["kind"] == "await" and not all(ready.get(m, 0) >= run for m in u["moves"]):
                            break
                        if u["kind"] == "wait" and not all(done.get(m, 0) >= run for m in u["moves"]):
                            break
                        if u["kind"] in ("pull", "rtouch", "rsum", "ack"):
                            assert all(ready.get(m, 0) == run for m in u["moves"]), "bytes read before their signal"
                        if u["kind"] in ("pull", "rtouch", "ack"):
                            for m in u["moves"]:
                                done[m] = run
                        if u["kind"] == "signal":
                            for m in u["moves"]:
                                assert ready.get(m, 0) == run - 1
                                ready[m] = run
                        finished[r].add(i)
                        queue.pop(0)
                        remaining -= 1
                        progressed = True
            assert progressed, "every rank is blocked in run %d" % run
        assert set(ready.values()) == set(done.values()) == {run}


GROUP_SUM = [("llama_tiny_tp_locs4", 4), ("llama7b_layer_locs4", 4), ("llama7b_layer_locs8", 8), ("llama7b_layer_tp_locs4", 4), ("llama7b_layer_tp_locs8", 8)]


@pytest.mark.parametrize("name,world", GROUP_SUM)
def test_group_sums_keep_the_plans_hazard_free_and_the_exchange_live(name, world):
    """group_sum=True: the remote adds of a partial-sum group become one elementwise op over the peers' memory
    followed by one op that acknowledges the moves.  Same checks as for the plain plans: every hazard ordered,
    sources protected, all ranks together never block and read only what was signalled in the same run."""
    from einsummable_b200.fuse import fuse_attention, fuse_elementwise_chains
    mg = fuse_attention(fuse_elementwise_chains(load(name))[0])[0]
    nodes = mg["nodes"]
    plans = [plan(mg, {r}, True, order="simulated", group_sum=True) for r in range(world)]
    n_sums = 0
    for rank, (units, d) in enumerate(plans):
        check_plan(mg, units, d)
        sums = [u for u in units if u["kind"] == "rsum"]
        n_sums += len(sums)
        for u in sums:
            assert 2 <= len(u["moves"]) <= 7 and len(set(u["moves"])) == len(u["moves"])
            for t, m in zip(u["nodes"], u["moves"]):       # each member is the one reader of its move
                assert m in nodes[t]["inns"] and nodes[t]["touch"]["castable"] == "add"
                assert nodes[t]["mems"][0] == nodes[u["nodes"][0]]["mems"][0]
        # every incoming move is still read exactly once
        read = [m for u in units if u["kind"] in ("pull", "rtouch", "rsum") for m in u["moves"]]
        assert sorted(read) == sorted(n["id"] for n in nodes if n["kind"] == "move" and n["dst_loc"] == rank
                                      and n["src_loc"] != rank)
    assert n_sums >= 2
    all_ranks_stay_live(plans, world)


@pytest.mark.parametrize("name,world", [("llama7b_train_l4_locs2", 2), ("llama7b_train_l4_locs4", 4)])
def test_training_graphs_are_hazard_free_and_live(name, world):
    """Config 5's shape (four layers forward, loss, backward, update; 6625 / 14000 memgraph nodes), folded, one
    process per location in simulated order: every hazard ordered, the exchange never blocks."""
    from einsummable_b200.fuse import fuse_attention, fuse_elementwise_chains
    mg = fuse_attention(fuse_elementwise_chains(load(name))[0])[0]
    plans = [plan(mg, {r}, True, order="simulated") for r in range(world)]
    for units, d in plans:
        check_plan(mg, units, d)
    all_ranks_stay_live(plans, world)


def test_an_early_tensor_does_not_wait_behind_the_flag_of_a_late_one():
    """Two adjacent, independent moves from location 0 to location 1 -- one whose source exists from the
    start, one whose source is the end of a long chain -- form one run.  They must not share an await: the
    reader of the early tensor would otherwise start when the late one is ready."""
    n_el = 1 << 20                                  # 4 MiB f32 per tensor: each chain node costs microseconds
    size = 4 * n_el

    def ew(i, inns, loc, out, reads):
        return {"id": i, "inns": inns, "kind": "apply", "loc": loc, "group": -1,
                "mems": [[out, size]] + [[r, size] for r in reads],
                "einsummable": {"join_shape": [n_el], "inns": [[0] for _ in reads], "out_rank": 1,
                                "join": "exp[hole|f32@0]", "castable": None}}

    nodes = [{"id": 0, "inns": [], "kind": "inputmem", "loc": 0, "offset": 0, "size": size}]
    chain = 30                                      # x -> exp -> exp -> ... on location 0
    for k in range(chain):
        nodes.append(ew(1 + k, [k], 0, (1 + k) * size, [k * size]))
    early, late = chain + 1, chain + 2
    nodes.append({"id": early, "inns": [0], "kind": "move", "src_loc": 0, "src_offset": 0,
                  "dst_loc": 1, "dst_offset": 0, "size": size})
    nodes.append({"id": late, "inns": [chain], "kind": "move", "src_loc": 0, "src_offset": chain * size,
                  "dst_loc": 1, "dst_offset": size, "size": size})
    nodes.append(ew(chain + 3, [early], 1, 2 * size, [0]))          # reads the early tensor
    nodes.append(ew(chain + 4, [late], 1, 3 * size, [size]))        # reads the late one
    mg = {"num_locs": 2, "mem_sizes": [(chain + 1) * size, 4 * size], "taskgraph": {}, "inputs": [], "outputs": [],
          "nodes": nodes}
    assert M.move_runs(mg)[early] == M.move_runs(mg)[late]            # one run
    levels = M.node_levels(mg)
    assert levels[chain] - levels[0] > 10 * M.AWAIT_SPREAD_US
    units = M.schedule_units(mg, {1}, True)
    awaits = [u for u in units if u["kind"] == "await"]
    assert [u["moves"] for u in awaits] == [[early], [late]]
    both = [M.schedule_units(mg, {r}, True) for r in range(2)]
    times = M.simulate_schedule(mg, both)
    reader_of_early = next(i for i, u in enumerate(both[1]) if u.get("node") == chain + 3)
    signal_of_late = next(i for i, u in enumerate(both[0]) if u["kind"] == "signal" and late in u["moves"])
    assert times[(1, reader_of_early)][1] < times[(0, signal_of_late)][0]
    # sources that come together still share one await (and one pull launch)
    nodes[late]["inns"] = [0]
    nodes[late]["src_offset"] = 0
    units = M.schedule_units(mg, {1}, True)
    assert [u["moves"] for u in units if u["kind"] == "await"] == [[early, late]]
    assert [u["moves"] for u in units if u["kind"] == "pull"] == [[early, late]]


def test_simulated_order_is_the_same_on_every_rank_and_increases_along_dependencies():
    """Every rank simulates all ranks and must get the same times; along every dependency --
    local, signal -> pull, pull -> wait -- the simulated start time strictly increases, which is
    what makes one in-order exchange lane per rank safe under that order."""
    mg = load("llama7b_layer_locs4")
    all_units = [M.schedule_units(mg, {r}, True) for r in range(4)]
    times = M.simulate_schedule(mg, all_units)
    assert times == M.simulate_schedule(mg, [M.schedule_units(mg, {r}, True) for r in range(4)])
    sig, pull = {}, {}
    for r, units in enumerate(all_units):
        for i, u in enumerate(units):
            if u["kind"] == "signal":
                sig.update({m: (r, i) for m in u["moves"]})
            if u["kind"] in ("pull", "rtouch"):
                pull.update({m: (r, i) for m in u["moves"]})
    for r, units in enumerate(all_units):
        for i, u in enumerate(units):
            before = [(r, d) for d in u["deps"]]
            if u["kind"] == "await":
                before += [sig[m] for m in u["moves"]]
            if u["kind"] == "wait":
                before += [pull[m] for m in u["moves"]]
            for b in before:
                assert times[b][0] < times[b][1] <= times[(r, i)][0]
    for rank in range(4):
        units = M.order_units_by_simulation(mg, 4, rank)
        assert sorted(u["kind"] for u in units) == sorted(u["kind"] for u in all_units[rank])
        assert units[-1]["kind"] == "wait"
        starts = [u["sim_start_us"] for u in units[:-1]]
        assert starts == sorted(starts)


def test_program_rejects_bad_input():
    from einsummable_b200 import _lib
    p = program_t(None)
    a = p.add_copy(BASE, BASE + 4096, 64)
    with pytest.raises(_lib.es_error):
        p.add_copy(BASE, BASE + 4096, 64, deps=[5])          # not an earlier op
    with pytest.raises(_lib.es_error):
        p.add_pull([(BASE + 8, BASE + 4096, 64, BASE + 64, BASE + 68)])   # unaligned source
    with pytest.raises(_lib.es_error):
        p.launch()                                            # not finalized
    p.add_copy(BASE, BASE + 8192, 64, deps=[a])
    p.finalize(4)
    with pytest.raises(_lib.es_error):
        p.launch()                                            # planning only: no device
    with pytest.raises(_lib.es_error):
        p.add_copy(BASE, BASE + 4096, 64)                     # already finalized
    d = p.describe()
    assert [op["lane"] for op in d["ops"]] == [0, 0] and d["ops"][1]["wait_on"] == [] and d["n_exchange_lanes"] == 0
    p.close()


def _run_units_on_cpu(mg, units, order, inputs):
    """The units executed by the numpy oracle in the given order (the first-touch rule resolved
    statically, as the runner does): what any execution that respects only `deps` may compute."""
    import es_oracle as O
    nodes = mg["nodes"]
    storage = {}
    bufs = O.memgraph_place_inputs(mg, inputs, storage)
    for i in order:
        u = units[i]
        n = dict(nodes[u["node"]])
        if u["kind"] == "touch":
            n["group"] = -1 if u["first"] else 1
            O.run_memgraph({"nodes": [n]}, bufs, "interp", groups_touched=set() if u["first"] else {1}, storage=storage)
        else:
            O.run_memgraph({"nodes": [n]}, bufs, "interp", storage=storage)
    return O.memgraph_collect_outputs(mg, bufs, storage)


@pytest.mark.parametrize("name", ["c1_n64_evict_locs1", "c1_n64_evict_locs2", "c1_n64_locs2", "llama_tiny_locs2",
                                  "llama_train_tiny_locs2", "llama_tiny_tp_locs2"])
def test_any_order_that_respects_the_dependencies_gives_the_reference_result(name):
    """The units of a memgraph (all locations in one process) run by the oracle in random topological
    orders of their `deps`: every such order must give, bit for bit, what the memgraph's own node order
    gives (which in turn is the reference interpreter's result) -- a missing dependency shows up as a
    different result, not as a rare race."""
    import random
    import numpy as np
    mg = load(name)
    arr = np.load(os.path.join(GRAPHS, "graphs_evict.npz" if "evict" in name else ("graphs_tp.npz" if "_tp_" in name else "graphs.npz")))
    pre = name + "/in/"
    inputs = {k[len(pre):]: arr[k] for k in arr.files if k.startswith(pre)}
    pre = name + "/out/"
    want = {k[len(pre):]: arr[k] for k in arr.files if k.startswith(pre)}
    units = M.schedule_units(mg, set(range(mg["num_locs"])), False)
    rng = random.Random(7)
    base = _run_units_on_cpu(mg, units, list(range(len(units))), inputs)
    for k, ref in want.items():
        scale = np.abs(ref.astype(np.float64)).max()
        err = np.abs(base[k].astype(np.float64) - ref.astype(np.float64)).max()
        assert err <= (2e-3 if ref.dtype == np.float16 else 1e-6) * scale, (name, k, err, scale)
    for trial in range(3):
        indeg = [len(u["deps"]) for u in units]
        children = [[] for _ in units]
        for i, u in enumerate(units):
            for d in u["deps"]:
                children[d].append(i)
        ready = [i for i, d in enumerate(indeg) if d == 0]
        order = []
        while ready:
            i = ready.pop(rng.randrange(len(ready)) if trial else 0)
            order.append(i)
            for c in children[i]:
                indeg[c] -= 1
                if indeg[c] == 0:
                    ready.append(c)
        assert len(order) == len(units)
        got = _run_units_on_cpu(mg, units, order, inputs)
        for k in want:
            assert got[k].tobytes() == base[k].tobytes(), (name, trial, k)
