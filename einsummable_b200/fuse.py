"""Fusion across node boundaries of a memgraph (one location): an elementwise apply node is
folded into the nodes that read its result, so the intermediate tensor never
makes its round trip through HBM.

The reference keeps such chains as separate nodes (softmax = 5 nodes, src/einsummable/gwriter.cc:830-855;
RMSNorm = 8 nodes, llama/modules.cc:126-195) and its kernel manager even splits one node into several
cuTENSOR calls; here the code generator compiles any scalarop tree, so folding a producer into its
consumer is a substitution in the join text plus a composition of the index maps.

The pass works on the memgraph as loaded from JSON and returns a new memgraph that is valid both for
in-order execution and for dependency-ordered execution: a reader that now reads A's inputs takes over
A's dependencies, and every later node that writes into memory A read (the memgraph reuses freed memory,
and the `del` that freed it only knew A as a reader) is made to depend on the readers.
A producer A is folded into its reader B when
  * A is an elementwise einsummable (no aggregation), B an einsummable that is not a plain contraction
    (those run on the tensor cores with the join x0*x1),
  * every reader of A's result qualifies (then A is folded into each of them: evaluating a
    memory-bound expression once per reader moves fewer bytes than writing and re-reading it),
    reads it in one input slot, and the result is not a saved output,
  * A and B iterate over the same number of points (nothing is recomputed), B reads A's result with
    exactly the shape and dtype A wrote it in (the taskgraph lets a node view the same bytes under
    another shape or dtype, src/einsummable/taskgraph.cc:765-793: such readers are left alone),
  * nothing between A and B in list order, and not B itself, writes memory A reads (the memgraph
    reuses memory: B now reads A's inputs later than the reference planned),
  * the folded node has at most 8 inputs.
"""
import copy
import re

MAX_INNS = 8
_DSIZE = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}
_HOLE = re.compile(r"hole\|(f16|f32|f64|c64)@(\d+)")


def _prod(v):
    r = 1
    for x in v:
        r *= int(x)
    return r


def _is_elementwise(e):
    # no aggregated mode: a castable on such a node has nothing to combine
    return e["out_rank"] == len(e["join_shape"])


def _is_plain_contraction(e):
    if e["castable"] != "add" or len(e["inns"]) != 2 or e["out_rank"] == len(e["join_shape"]):
        return False
    return re.fullmatch(r"\*\[hole\|(f16|f32|f64|c64)@0,hole\|(f16|f32|f64|c64)@1\]", e["join"]) is not None


def _overlap(a, b):
    return a[0] < b[0] + b[1] and b[0] < a[0] + a[1]


def _written_region(node, loc):
    """The (offset, size) a node writes in location `loc`'s memory, or None."""
    k = node["kind"]
    if k == "apply":
        return tuple(node["mems"][0]) if node["loc"] == loc else None
    if k == "constant":
        if node["loc"] != loc:
            return None
        f = node["fill"]
        if f["type"] == "constant":
            return (node["offset"], int(f["nelem"]) * _DSIZE[f["value"]["dtype"]])
        return (node["offset"], int(f["nrow"]) * int(f["ncol"]) * _DSIZE[f["lower"]["dtype"]])
    if k == "move":   # the destination rank pulls the bytes at the move's place in its own order
        return (node["dst_offset"], node["size"]) if node["dst_loc"] == loc else None
    if k == "copy":
        return (node["dst_offset"], node["size"]) if node["loc"] == loc else None
    if k == "load":
        return (node["offset"], node["size"]) if node["loc"] == loc else None
    return None


def _hole_dtype(join, slot):
    for m in _HOLE.finditer(join):
        if int(m.group(2)) == slot:
            return m.group(1)
    return None


def _out_dtype(join):
    """Dtype of the join's root node, by the reference's typing rules."""
    from .scalarop import scalarop_t
    return scalarop_t(join).out_dtype()


def compose(a, b, slot):
    """The einsummable that computes b with its input `slot` replaced by the expression a."""
    n_a = len(a["inns"])
    shift = n_a - 1

    def renumber_b(m):
        i = int(m.group(2))
        return "hole|%s@%d" % (m.group(1), i if i < slot else i + shift)

    def renumber_a(m):
        return "hole|%s@%d" % (m.group(1), int(m.group(2)) + slot)

    a_text = _HOLE.sub(renumber_a, a["join"])
    # substitute first (the slot's hole is unique text "hole|dt@slot"), then renumber the others
    parts = []
    pos = 0
    for m in _HOLE.finditer(b["join"]):
        parts.append(b["join"][pos:m.start()])
        parts.append(a_text if int(m.group(2)) == slot else renumber_b(m))
        pos = m.end()
    parts.append(b["join"][pos:])
    via = b["inns"][slot]                      # a's mode m is b's mode via[m]
    new_inns = b["inns"][:slot] + [[via[m] for m in inn] for inn in a["inns"]] + b["inns"][slot + 1:]
    return {"join_shape": list(b["join_shape"]), "inns": new_inns, "out_rank": b["out_rank"],
            "join": "".join(parts), "castable": b["castable"]}


def fuse_elementwise_chains(mg):
    """Returns (new memgraph, number of nodes folded away).  With several locations the same rules
    apply inside each location (every rank must fold the same way, which it does: the pass only
    reads the graph); a result that a move ships to another location is never folded."""
    mg = copy.deepcopy(mg)
    nodes = mg["nodes"]
    # (saved blocks that end up in storage have no memory region to protect)
    saved = [(blk["loc"], blk["offset"], blk["size"]) for t in mg["outputs"] for blk in t["blocks"] if "offset" in blk]
    alive = [True] * len(nodes)
    folded = 0
    for ia, a in enumerate(nodes):
        if a["kind"] != "apply" or "einsummable" not in a or not _is_elementwise(a["einsummable"]):
            continue
        out = tuple(a["mems"][0])
        loc = a["loc"]
        if any(s[0] == loc and _overlap(out, s[1:]) for s in saved):
            continue
        # readers of the result: apply nodes after A that depend on it and read exactly its region
        readers = []
        shipped = False
        for ib in range(ia + 1, len(nodes)):
            n = nodes[ib]
            if not alive[ib] or a["id"] not in n["inns"]:
                continue
            if n["kind"] in ("move", "copy", "evict"):
                shipped = True      # another location (or a copy, or the storage) reads the materialised tensor
                break
            if n["kind"] == "apply" and n["loc"] == loc and any(tuple(m) == out for m in n["mems"][1:]):
                readers.append(ib)
        if shipped or not readers:
            continue
        ea = a["einsummable"]
        a_reads = [tuple(m) for m in a["mems"][1:]]
        # with R readers the producer is evaluated R times instead of once; in bytes that is
        # R * in(A) against in(A) + (R + 1) * out(A) before, nearly always less (kernels of this
        # kind are bound by memory, not by the arithmetic)
        in_bytes = sum(m[1] for m in a_reads)
        n_r = len(readers)
        if (n_r - 1) * in_bytes > (n_r + 1) * out[1]:
            continue
        plans = []
        for ib in readers:
            b = nodes[ib]
            if "einsummable" not in b or _is_plain_contraction(b["einsummable"]):
                break
            slots = [k for k, m in enumerate(b["mems"][1:]) if tuple(m) == out]
            eb = b["einsummable"]
            if len(slots) != 1 or _prod(ea["join_shape"]) != _prod(eb["join_shape"]):
                break
            via = eb["inns"][slots[0]]
            if [int(ea["join_shape"][m]) for m in range(ea["out_rank"])] != [int(eb["join_shape"][v]) for v in via]:
                break       # the reader views the bytes under another shape
            if _out_dtype(ea["join"]) != _hole_dtype(eb["join"], slots[0]):
                break       # ... or another dtype
            if len(eb["inns"]) - 1 + len(ea["inns"]) > MAX_INNS:
                break
            if any(_overlap(tuple(b["mems"][0]), r) for r in a_reads):
                break
            plans.append((ib, slots[0]))
        if len(plans) != n_r:
            continue
        hazard = False
        for ic in range(ia + 1, readers[-1]):
            if not alive[ic]:
                continue
            w = _written_region(nodes[ic], loc)
            if w is not None and any(_overlap(w, r) for r in a_reads):
                hazard = True
                break
        if hazard:
            continue
        for ib, slot in plans:
            b = nodes[ib]
            b["einsummable"] = compose(ea, b["einsummable"], slot)
            b["mems"] = [b["mems"][0]] + b["mems"][1:1 + slot] + a["mems"][1:] + b["mems"][2 + slot:]
            b["inns"] = sorted(set(i for i in b["inns"] if i != a["id"]) | set(a["inns"]))
        # later writers into memory A read must now also wait for the readers
        reader_ids = [nodes[ib]["id"] for ib, _ in plans]
        for ic in range(readers[-1] + 1, len(nodes)):
            if not alive[ic]:
                continue
            w = _written_region(nodes[ic], loc)
            if w is not None and any(_overlap(w, r) for r in a_reads):
                nodes[ic]["inns"] = sorted(set(nodes[ic]["inns"]) | set(reader_ids))
        alive[ia] = False
        folded += 1
    # a folded node stays in the list as a bookkeeping stub so that ids keep indexing the list
    for i, n in enumerate(nodes):
        if not alive[i]:
            nodes[i] = {"id": n["id"], "inns": n["inns"], "kind": "alloc", "loc": n["loc"], "folded": True}
    return mg, folded
