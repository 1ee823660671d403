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


_X = r"to_f32\[\+\[hole\|f16@0,hole\|f16@1\]\]"
_E = r"exp\[\+\[" + _X + r",\*\[constant\{f32\|-1\},hole\|f32@2\]\]\]"
_RE_MAX = re.compile(_X)
_RE_SUM = re.compile(_E)
_RE_NORM = re.compile(r"to_f16\[\*\[" + _E + r",power\{-1\}\[hole\|f32@3\]\]\]")
_RE_MUL16 = re.compile(r"\*\[hole\|f16@0,hole\|f16@1\]")


def _row_major_strides(shape):
    st = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        st[i] = st[i + 1] * int(shape[i + 1])
    return st


def _match_attention(nodes, alive, i_s, saved):
    """The five nodes of softmax(Q K^T + mask) V that start with the scores contraction nodes[i_s]
    (after the elementwise fold): returns (indices, descriptor dict, mems [out, q, k, v, mask]) or None."""
    s = nodes[i_s]
    es = s["einsummable"]
    loc = s["loc"]
    if len(es["join_shape"]) != 5 or es["out_rank"] != 4 or not _is_plain_contraction(es) or not _RE_MUL16.fullmatch(es["join"]):
        return None
    b, h, rows, keys, d = [int(x) for x in es["join_shape"]]
    qk = {}
    for slot, modes in enumerate(es["inns"]):
        if sorted(modes) == [0, 1, 2, 4] and modes[-1] == 4:
            qk["q"] = (slot, modes)
        elif sorted(modes) == [0, 1, 3, 4] and modes[-1] == 4:
            qk["k"] = (slot, modes)
    if len(qk) != 2:
        return None

    def strides(modes, row_mode):
        st = _row_major_strides([es["join_shape"][m] for m in modes])
        at = {m: st[i] for i, m in enumerate(modes)}
        return [at[0], at[1], at[row_mode]]

    def sole_readers(ix, want):
        """Indices of the apply nodes that read node ix's result, if they are exactly `want` many, read
        it as written, and nothing ships or saves it."""
        n = nodes[ix]
        out = tuple(n["mems"][0])
        if any(sv[0] == loc and _overlap(out, sv[1:]) for sv in saved):
            return None
        got = []
        for ib in range(ix + 1, len(nodes)):
            m = nodes[ib]
            if not alive[ib] or n["id"] not in m["inns"]:
                continue
            if m["kind"] in ("move", "copy", "evict"):
                return None
            if m["kind"] == "apply":
                if m["loc"] != loc or "einsummable" not in m or not any(tuple(x) == out for x in m["mems"][1:]):
                    return None
                got.append(ib)
        return got if len(got) == want else None

    r_s = sole_readers(i_s, 3)
    if r_s is None:
        return None
    i_m, i_l, i_p = r_s
    m, l, pn = nodes[i_m], nodes[i_l], nodes[i_p]
    em, el, ep = m["einsummable"], l["einsummable"], pn["einsummable"]
    s_out = tuple(s["mems"][0])
    full = [0, 1, 2, 3]
    shape4 = [b, h, rows, keys]
    if not (em["castable"] == "max" and em["out_rank"] == 3 and [int(x) for x in em["join_shape"]] == shape4
            and em["inns"] == [full, [2, 3]] and _RE_MAX.fullmatch(em["join"]) and tuple(m["mems"][1]) == s_out):
        return None
    mask = tuple(m["mems"][2])
    m_out = tuple(m["mems"][0])
    if not (el["castable"] == "add" and el["out_rank"] == 3 and [int(x) for x in el["join_shape"]] == shape4
            and el["inns"] == [full, [2, 3], [0, 1, 2]] and _RE_SUM.fullmatch(el["join"])
            and [tuple(x) for x in l["mems"][1:]] == [s_out, mask, m_out]):
        return None
    l_out = tuple(l["mems"][0])
    if not (ep["out_rank"] == 4 and [int(x) for x in ep["join_shape"]] == shape4
            and ep["inns"] == [full, [2, 3], [0, 1, 2], [0, 1, 2]] and _RE_NORM.fullmatch(ep["join"])
            and [tuple(x) for x in pn["mems"][1:]] == [s_out, mask, m_out, l_out]):
        return None
    if sole_readers(i_m, 2) != [i_l, i_p] or sole_readers(i_l, 1) != [i_p]:
        return None
    r_p = sole_readers(i_p, 1)
    if r_p is None:
        return None
    i_o = r_p[0]
    o = nodes[i_o]
    eo = o["einsummable"]
    if not (_is_plain_contraction(eo) and _RE_MUL16.fullmatch(eo["join"]) and eo["out_rank"] == 4
            and [int(x) for x in eo["join_shape"]] == [b, h, rows, d, keys]):
        return None
    p_out = tuple(pn["mems"][0])
    v_slot = None
    for slot, modes in enumerate(eo["inns"]):
        if modes == [0, 1, 2, 4]:
            if tuple(o["mems"][1 + slot]) != p_out:
                return None
        elif sorted(modes) == [0, 1, 3, 4] and modes[-1] == 3:
            v_slot = slot
    if v_slot is None or len(eo["inns"]) != 2 or [0, 1, 2, 4] not in eo["inns"]:
        return None
    vm = eo["inns"][v_slot]
    vst = _row_major_strides([eo["join_shape"][x] for x in vm])
    vat = {x: vst[i] for i, x in enumerate(vm)}
    desc = {"batch": b, "heads": h, "rows": rows, "keys": keys, "head_dim": d,
            "q_stride": strides(qk["q"][1], 2), "k_stride": strides(qk["k"][1], 3),
            "v_stride": [vat[0], vat[1], vat[4]], "out_stride": _row_major_strides([b, h, rows, d])[:3],
            "mask_stride": keys, "skip_known": 0, "skip_from": 0}
    mems = [list(o["mems"][0]), list(s["mems"][1 + qk["q"][0]]), list(s["mems"][1 + qk["k"][0]]),
            list(o["mems"][1 + v_slot]), list(mask)]
    return [i_s, i_m, i_l, i_p, i_o], desc, mems


def _lowertri_start(nodes, alive, loc, region, before, rows, cols, depth=0):
    """If the f16 [rows, cols] tensor in `region` of location `loc`, as the node at index `before`
    reads it, is a lower-triangular fill -- 0 where column <= row - start, -inf elsewhere -- returns
    start, else None.  Looks through what the compilers put between the fill and its readers: copies of
    row blocks (touches without a castable) and moves of whole tensors."""
    if depth > 4 or region[1] != rows * cols * 2:
        return None
    covered, start = [], None
    for ic in range(before - 1, -1, -1):
        n = nodes[ic]
        if not alive[ic]:
            continue
        w = _written_region(n, loc)
        if w is None or not _overlap(w, region):
            continue
        if n["kind"] == "constant":
            f = n["fill"]
            if (covered or w != region or f["type"] != "lowertri" or f["lower"]["dtype"] != "f16"
                    or int(f["nrow"]) != rows or int(f["ncol"]) != cols
                    or list(f["upper"]["raw"][:2]) != [0, 252] or list(f["lower"]["raw"][:2]) != [0, 0]
                    or abs(int(f["start"])) >= (1 << 30)):
                return None
            return int(f["start"])
        if n["kind"] == "move":
            if covered or w != region:
                return None
            src = (n["src_offset"], n["size"])
            return _lowertri_start(nodes, alive, n["src_loc"], src, ic, rows, cols, depth + 1)
        if n["kind"] == "apply" and "touch" in n:
            t = n["touch"]
            sel = t["selection"]
            if w != region or t["dtype"] != "f16" or t["castable"] is not None or len(sel) != 2:
                return None
            (ri, ro, oi, oo, sz), (ci, co, coi, coo, csz) = [[int(x) for x in d] for d in sel]
            if ro != rows or (ci, co, coi, coo, csz) != (cols, cols, 0, 0, cols):
                return None
            if any(oo < hi and lo < oo + sz for lo, hi in covered):
                return None                  # an older lifetime of the memory shows through
            sub = _lowertri_start(nodes, alive, loc, tuple(n["mems"][1]), ic, ri, cols, depth + 1)
            if sub is None:
                return None
            s_here = sub + oo - oi           # row r of the block is row r - oo + oi of the source
            if start is not None and s_here != start:
                return None
            start = s_here
            covered.append((oo, oo + sz))
            if sum(hi - lo for lo, hi in covered) == rows:
                return start
            continue
        return None
    return None


def fuse_attention(mg):
    """Replaces every softmax(Q K^T + mask) V chain -- scores contraction, max, sum of exponentials,
    normalisation, contraction with V, as they stand after fuse_elementwise_chains -- by one apply node
    with an "attention" descriptor (einsummable_b200/attention.py), placed where the last of the five
    stood.  Returns (new memgraph, number of chains replaced).  The same conditions as for folding
    apply: the four intermediate results have no other reader and are not saved or shipped, and
    nothing between the first and the last node writes memory the chain reads; later writers into
    that memory are made to wait for the new node."""
    from .attention import attention_t
    mg = copy.deepcopy(mg)
    nodes = mg["nodes"]
    saved = [(blk["loc"], blk["offset"], blk["size"]) for t in mg["outputs"] for blk in t["blocks"] if "offset" in blk]
    alive = [not n.get("folded", False) for n in nodes]
    fused = 0
    for i_s, s in enumerate(nodes):
        if not alive[i_s] or s["kind"] != "apply" or "einsummable" not in s:
            continue
        got = _match_attention(nodes, alive, i_s, saved)
        if got is None:
            continue
        idx, desc, mems = got
        if not attention_t.from_json(desc).eligible() or any(m[0] % 16 for m in mems):
            continue
        i_o = idx[-1]
        loc = s["loc"]
        reads = [tuple(m) for m in mems[1:]]
        if any(_overlap(tuple(mems[0]), r) for r in reads):
            continue
        # Q and K are now read where the last node stands instead of the first, the mask instead of
        # where the max node stood (V is read where it always was)
        hazard = False
        mask = tuple(mems[4])
        for ic in range(i_s + 1, i_o):
            if not alive[ic] or ic in idx:
                continue
            w = _written_region(nodes[ic], loc)
            if w is None:
                continue
            if any(_overlap(w, r) for r in reads[:2]) or (ic > idx[1] and _overlap(w, mask)):
                hazard = True
                break
        if hazard:
            continue
        # a mask that is a lower-triangular fill (0 / -inf): the kernel computes it and skips the key
        # blocks above the diagonal
        tri = _lowertri_start(nodes, alive, loc, mask, idx[1], desc["rows"], desc["keys"])
        if tri is not None:
            desc["skip_known"], desc["skip_from"] = 1, tri
        removed = set(nodes[i]["id"] for i in idx[:-1])
        deps = set()
        for i in idx:
            deps |= set(nodes[i]["inns"])
        o = nodes[i_o]
        nodes[i_o] = {"id": o["id"], "inns": sorted(deps - removed - {o["id"]}), "kind": "apply", "loc": loc,
                      "group": -1, "attention": desc, "mems": mems}
        for ic in range(i_o + 1, len(nodes)):
            if not alive[ic]:
                continue
            w = _written_region(nodes[ic], loc)
            if w is not None and any(_overlap(w, r) for r in reads):
                nodes[ic]["inns"] = sorted(set(nodes[ic]["inns"]) | {o["id"]})
        for i in idx[:-1]:
            n = nodes[i]
            alive[i] = False
            nodes[i] = {"id": n["id"], "inns": n["inns"], "kind": "alloc", "loc": n["loc"], "folded": True}
        fused += 1
    return mg, fused


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
