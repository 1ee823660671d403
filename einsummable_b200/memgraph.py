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

import numpy as np
import torch

from .einsummable import einsummable_t, fill_t, touch_t
from .kernel_manager import kernel_manager_t
from .program import program_t
from .scalarop import DTYPE_SIZE

NP_DTYPE = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "c64": np.complex64}


def load_memgraph(path):
    opener = gzip.open if str(path).endswith(".gz") else open
    with opener(path, "rt") as f:
        return json.load(f)


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
    bookkeeping = ("alloc", "del", "inputmem", "partialize")
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

BOOKKEEPING = ("alloc", "del", "inputmem", "partialize")


def _sides(node):
    if node["kind"] == "move":
        return (node["src_loc"], node["dst_loc"])
    return (node["loc"],)


def schedule_units(mg, owned, exchange):
    """The launchable units of the locations in `owned`, in the memgraph's node order, each with
    the units it depends on.

    owned: the locations this process drives.  exchange: True when a move between two locations
    is an exchange between two processes (one process per GPU) -- the source rank gets a
    `signal` unit, the destination rank a `pull` unit, and whatever later reuses the source's
    memory a `wait` unit for the destination's acknowledgement; False when this process drives
    both sides and the move is a plain copy.

    Dependencies are the memgraph's edges looked through its bookkeeping nodes (alloc, del,
    inputmem, partialize: src/einsummable/memgraph.h:189-309 -- they launch nothing but carry
    the "this memory is free again" ordering).  The incoming moves of one run (move_runs) form
    one pull unit and are served by one launch; the outgoing moves of a run that wait for the
    same producers share a signal unit.  Touches of one group are chained in node order, the
    first being the copy (src/engine/gpu/exec_graph.cc:167-172,368-378).

    Units are dicts: kind in {einsummable, touch, constant, copy, signal, pull, wait}, `deps`
    (indices of earlier units), `node` or `moves` (memgraph node ids)."""
    nodes = mg["nodes"]
    owned = set(owned)
    runs = move_runs(mg)
    run_members = {}
    for nid in sorted(runs):
        run_members.setdefault(runs[nid], []).append(nid)

    def is_cross(n):
        return exchange and n["kind"] == "move" and n["src_loc"] != n["dst_loc"]

    # real nodes a bookkeeping node stands for (nodes are in topological order)
    closure = {}
    for n in nodes:
        if n["kind"] in BOOKKEEPING:
            acc = set()
            for i in n["inns"]:
                acc |= closure[i] if nodes[i]["kind"] in BOOKKEEPING else {i}
            closure[n["id"]] = frozenset(acc)

    units, unit_of, waited, group_last = [], {}, {}, {}

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
            units.append({"kind": "wait", "moves": tokens, "deps": []})
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
                members = [m for m in run if nodes[m]["dst_loc"] in owned and nodes[m]["dst_loc"] == n["dst_loc"]
                           and is_cross(nodes[m])]
                raw = set()
                for m in members:
                    raw |= raw_deps(nodes[m], nodes[m]["dst_loc"])
                idx = emit({"kind": "pull", "moves": members, "deps": resolve(raw), "loc": n["dst_loc"]})
                for m in members:
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
            idx = emit({"kind": "touch", "node": nid, "deps": deps, "first": first, "loc": loc})
            if n["group"] >= 0:
                group_last[(loc, n["group"])] = idx
        elif kind == "apply":
            idx = emit({"kind": "einsummable", "node": nid, "deps": deps, "loc": loc})
        elif kind == "constant":
            idx = emit({"kind": "constant", "node": nid, "deps": deps, "loc": loc})
        elif kind in ("move", "copy"):
            idx = emit({"kind": "copy", "node": nid, "deps": deps, "loc": loc})
        else:
            raise ValueError("unknown memgraph node kind %r" % kind)
        unit_of[nid] = idx
    # sources nobody on this rank reused: the next run may overwrite them, so the run ends by
    # collecting their acknowledgements
    rest = [n["id"] for n in nodes if is_cross(n) and n["src_loc"] in owned and n["id"] not in waited]
    if rest:
        units.append({"kind": "wait", "moves": rest, "deps": []})
    return units


class memgraph_runner_t:
    def __init__(self, mg, devices=None, rank=None, world=None, transport="nccl", wait_limit_ms=0, fuse=False,
                 schedule="dag", max_lanes=0):
        """transport (one process per GPU only): "nccl" = send/recv pairs; "p2p" = every
        location buffer lives in symmetric memory, the destination rank pulls the bytes over
        NVLink with an SM copy kernel, and the two ranks hand-shake through bounded flag
        kernels (data ready / copy finished).
        schedule: "dag" = the library's program executor (dependency-ordered lanes, see the
        module text); "list" = one stream in node order.  The NCCL transport always runs as a list."""
        self.folded = 0
        if fuse:
            # elementwise producers folded into their readers (one location only, see fuse.py)
            from .fuse import fuse_elementwise_chains
            mg, self.folded = fuse_elementwise_chains(mg)
        self.mg = mg
        self.num_locs = mg["num_locs"]
        self.distributed = rank is not None
        self.transport = transport if self.distributed else "local"
        self.schedule = "list" if self.transport == "nccl" else schedule
        if self.schedule not in ("dag", "list"):
            raise ValueError("schedule must be 'dag' or 'list'")
        self.max_lanes = max_lanes
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
        if self.schedule == "dag":
            self._build_program()
        else:
            self._prepare()

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
        self.units = schedule_units(self.mg, set(self.devices), self.transport == "p2p")
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
            elif kind == "touch":
                node = nodes[u["node"]]
                d = node["touch"]
                t = touch_t(d["selection"], d["castable"], d["dtype"])
                loc = node["loc"]
                offs = [m[0] for m in node["mems"]]
                prog.add_touch(t, None if u["first"] else d["castable"], self.ptr(loc, offs[0]), self.ptr(loc, offs[1]), deps)
                self.stats["touch"] += 1
                self.unit_labels.append(("touch", "%s %s" % (d["castable"], d["dtype"])))
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
                                  self._flag_ptr(node["dst_loc"], 0, k), self._flag_ptr(node["src_loc"], 1, k)))
                prog.add_pull(items, deps)
                self.stats["move"] += len(items)
                self.stats["move_bytes"] += sum(it[2] for it in items)
                self.unit_labels.append(("pull", "%d moves %d bytes" % (len(items), sum(it[2] for it in items))))
            elif kind == "wait":
                prog.add_wait([self._flag_ptr(nodes[m]["src_loc"], 1, self.move_index[m]) for m in u["moves"]], deps)
                self.unit_labels.append(("wait", str(len(u["moves"]))))
            else:
                raise ValueError(kind)
        need = prog.finalize(self.max_lanes)
        self.workspace = {dev: (torch.empty(max(need, 256), dtype=torch.uint8, device="cuda:%d" % dev), need)}
        prog.set_workspace(self.workspace[dev][0], max(need, 256))
        if self.wait_limit_ms:
            prog.set_wait_limit(self.wait_limit_ms)
        self.prog = prog
        self.program = self.units

    def profile(self, stream=None):
        """One run with a CUDA event pair around every op: [(class, label, milliseconds)].  For pull
        and wait ops the time includes waiting for the peer."""
        if self.prog is None:
            raise RuntimeError("profile needs the dag schedule")
        ms = self.prog.launch_timed(stream if stream is not None else torch.cuda.current_stream())
        return [(lab[0], lab[1], t) for lab, t in zip(self.unit_labels, ms)]

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
                if "einsummable" in node:
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
            self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]].copy_(torch.from_numpy(raw))

    def get_output(self, key):
        """The saved tensor assembled from its blocks (blocks on other ranks are left zero)."""
        t = self._tensor_desc("outputs", key)
        out = np.zeros(t["shape"], dtype=NP_DTYPE[t["dtype"]])
        for blk, sl in zip(t["blocks"], _blocks_of(t["shape"], t["partdims"])):
            if not self.owns(blk["loc"]):
                continue
            raw = self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]].cpu().numpy()
            out[sl] = raw.view(NP_DTYPE[t["dtype"]]).reshape(out[sl].shape)
        return out

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
        else:
            for op in self.program:
                if op[0] == "einsummable":
                    k = self.km(op[1]).kernel_info(op[2]).split("|")[0]
                    kinds[k] = kinds.get(k, 0) + 1
        return kinds

    def device_status(self):
        return max(km.device_status() for km in self.kms.values())

    def close(self):
        if self.prog is not None:
            self.prog.close()
            self.prog = None
        for km in self.kms.values():
            km.close()
