"""Interchange formats of the callers either side of the hot path (host only).

  * memgraph_to_wire / memgraph_from_wire: a memgraph as the reference sends it between processes
    -- the protobuf message MemGraph of src/proto/einsummable.proto:199-320, written by
    memgraph_t::to_wire and read by memgraph_t::from_wire (src/einsummable/memgraph.cc:258-457) --
    to and from the dict form the memgraph runner takes.  The message holds the nodes only; where
    the graph's inputs and saved tensors live travels separately in the reference too
    (src/server/base.h), so `inputs` / `outputs` are not part of it.
  * wire_to_json / wire_from_json: any message of that .proto by name, JSON with the .proto's
    field names (the library's schema-driven codec, csrc/wire.cc; no protobuf package involved).
  * weight files (llama/from_pth2.py:27-35, llama/reader.cc:42-110): list, read, append.
"""
import ctypes
import json

import numpy as np

from . import _lib


def wire_to_json(message, data):
    lib = _lib.load()
    need = ctypes.c_uint64(0)
    buf = ctypes.create_string_buffer(bytes(data), len(data)) if len(data) else None
    _lib.check(lib.es_b200_wire_to_json(message.encode(), buf, len(data), None, 0, ctypes.byref(need)))
    out = ctypes.create_string_buffer(need.value)
    _lib.check(lib.es_b200_wire_to_json(message.encode(), buf, len(data), out, need.value, None))
    return json.loads(out.value.decode())


def wire_from_json(message, obj):
    lib = _lib.load()
    text = json.dumps(obj).encode()
    need = ctypes.c_uint64(0)
    _lib.check(lib.es_b200_wire_from_json(message.encode(), text, None, 0, ctypes.byref(need)))
    out = ctypes.create_string_buffer(max(need.value, 1))
    _lib.check(lib.es_b200_wire_from_json(message.encode(), text, out, need.value, None))
    return out.raw[:need.value]


# ------------------------------------------------------------------ memgraph <-> MemGraph message
def _einsummable_to_proto(e):
    p = {"join_shape": [int(x) for x in e["join_shape"]], "inns": [{"idxs": [int(i) for i in inn]} for inn in e["inns"]],
         "out_rank": int(e["out_rank"]), "join": e["join"]}
    if e.get("castable") is not None:
        p["castable"] = e["castable"]
    return p


def _einsummable_from_proto(p):
    return {"join_shape": p["join_shape"], "inns": [x["idxs"] for x in p["inns"]], "out_rank": p["out_rank"],
            "join": p["join"], "castable": p.get("castable")}


def _fill_to_proto(f):
    if f["type"] == "constant":
        return {"constant": {"value": f["value"]["text"], "shape": [int(f["nelem"])]}}
    return {"lowertri": {"lower": f["lower"]["text"], "upper": f["upper"]["text"], "ncol": int(f["ncol"]),
                         "nrow": int(f["nrow"]), "start": int(f["start"])}}


_SIZE = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}
_NP = {"f16": np.float16, "f32": np.float32, "f64": np.float64}


def _scalar_from_text(text):
    """"f32|-inf" -> {"dtype", "raw", "text"} (scalar_t's operator<<, src/einsummable/scalarop.cc)."""
    dtype, _, val = text.partition("|")
    val = {"INF": "inf", "NINF": "-inf", "NAN": "nan"}.get(val, val)
    if dtype == "c64":
        re_, im_ = val.strip("()").split(",")
        raw = np.complex64(complex(float(re_), float(im_))).tobytes()
    else:
        raw = _NP[dtype](float(val)).tobytes()
    return {"dtype": dtype, "raw": list(raw) + [0] * (8 - len(raw)), "text": text}


def _fill_from_proto(p):
    if "constant" in p:
        c = p["constant"]
        n = 1
        for d in c["shape"]:
            n *= d
        return {"type": "constant", "value": _scalar_from_text(c["value"]), "nelem": n}
    t = p["lowertri"]
    return {"type": "lowertri", "lower": _scalar_from_text(t["lower"]), "upper": _scalar_from_text(t["upper"]),
            "nrow": t["nrow"], "ncol": t["ncol"], "start": t["start"]}


def memgraph_to_proto(mg):
    nodes = []
    for n in mg["nodes"]:
        k = n["kind"]
        if k in ("alloc", "del", "partialize") and "offset" not in n:
            raise ValueError("this memgraph dict carries no offsets for its %s nodes (an older dump)" % k)
        if k == "inputmem":
            body = {"inputmem": {"loc": n["loc"], "offset": n["offset"], "size": n["size"]}}
        elif k == "inputsto":
            body = {"inputsto": {"storage_loc": n["storage_loc"], "storage_id": n["storage_id"], "size": n["size"]}}
        elif k == "constant":
            body = {"constant": {"loc": n["loc"], "offset": n["offset"], "fill": _fill_to_proto(n["fill"])}}
        elif k == "apply":
            a = {"loc": n["loc"], "mems_offset": [m[0] for m in n["mems"]], "mems_size": [m[1] for m in n["mems"]],
                 "group": n["group"]}
            if "einsummable" in n:
                a["einsummable"] = _einsummable_to_proto(n["einsummable"])
            else:
                t = n["touch"]
                a["touch"] = {"selection": [dict(zip(("d_inn", "d_out", "offset_inn", "offset_out", "size"), s))
                                            for s in t["selection"]], "dtype": t["dtype"]}
                if t.get("castable") is not None:
                    a["touch"]["castable"] = t["castable"]
            body = {"apply": a}
        elif k == "move":
            body = {"move": {kk: n[kk] for kk in ("src_loc", "src_offset", "dst_loc", "dst_offset", "size")}}
        elif k == "copy":
            body = {"copy": {kk: n[kk] for kk in ("loc", "size", "src_offset", "dst_offset")}}
        elif k in ("evict", "load"):
            body = {k: {"storage_loc": n["storage_loc"], "storage_id": n["storage_id"], "loc": n["loc"],
                        "offset": n["offset"], "size": n["size"]}}
        elif k in ("alloc", "del", "partialize"):
            body = {k: {"loc": n["loc"], "offset": n["offset"], "size": n["size"]}}
        else:
            raise ValueError("unknown memgraph node kind %r" % k)
        body["inns"] = list(n["inns"])
        nodes.append(body)
    return {"num_compute_locs": mg["num_locs"], "num_storage_locs": mg["num_storage_locs"],
            "storage_locs": list(mg["storage_locs"]), "nodes": nodes}


def memgraph_from_proto(p):
    nodes = []
    mem_sizes = [0] * p["num_compute_locs"]

    def grow(loc, end):
        mem_sizes[loc] = max(mem_sizes[loc], int(end))

    for i, b in enumerate(p["nodes"]):
        (kind, x), = [(k, v) for k, v in b.items() if k != "inns"]
        n = {"id": i, "inns": b.get("inns", []), "kind": kind}
        if kind == "apply":
            n.update(loc=x["loc"], group=x["group"], mems=[[o, s] for o, s in zip(x["mems_offset"], x["mems_size"])])
            for o, s in n["mems"]:
                grow(x["loc"], o + s)
            if "einsummable" in x:
                n["einsummable"] = _einsummable_from_proto(x["einsummable"])
            else:
                t = x["touch"]
                n["touch"] = {"dtype": t["dtype"], "castable": t.get("castable"),
                              "selection": [[s["d_inn"], s["d_out"], s["offset_inn"], s["offset_out"], s["size"]]
                                            for s in t["selection"]]}
        elif kind == "constant":
            n.update(loc=x["loc"], offset=x["offset"], fill=_fill_from_proto(x["fill"]))
        elif kind == "inputsto":
            n.update(loc=x["storage_loc"], **x)
        else:
            n.update(x)
            if kind == "move":
                grow(x["src_loc"], x["src_offset"] + x["size"])
                grow(x["dst_loc"], x["dst_offset"] + x["size"])
            elif "offset" in x and "loc" in x:
                grow(x["loc"], x["offset"] + x["size"])
        nodes.append(n)
    return {"num_locs": p["num_compute_locs"], "num_storage_locs": p["num_storage_locs"],
            "storage_locs": p["storage_locs"], "mem_sizes": mem_sizes, "taskgraph": {}, "inputs": [], "outputs": [],
            "nodes": nodes}


def memgraph_to_wire(mg):
    """memgraph_t::to_wire: the serialized MemGraph message."""
    return wire_from_json("MemGraph", memgraph_to_proto(mg))


def memgraph_from_wire(data):
    """memgraph_t::from_wire, as the dict the memgraph runner takes (no inputs / outputs: see above)."""
    return memgraph_from_proto(wire_to_json("MemGraph", data))


# ------------------------------------------------------------------ weight files
def weight_file_list(path):
    """[(tensor name, element count)] of a weight file, in file order."""
    lib = _lib.load()
    count = ctypes.c_int(0)
    _lib.check(lib.es_b200_weight_file_list(path.encode(), None, 0, None, 0, ctypes.byref(count)))
    n = count.value
    names = ctypes.create_string_buffer(51 * n + 1)
    nelems = (ctypes.c_uint64 * max(n, 1))()
    _lib.check(lib.es_b200_weight_file_list(path.encode(), names, len(names), nelems, n, ctypes.byref(count)))
    return list(zip(names.value.decode().split("\n")[:n], list(nelems)[:n]))


def weight_file_read(path, name):
    """The named tensor's values (f16, flat)."""
    lib = _lib.load()
    nelem = ctypes.c_uint64(0)
    _lib.check(lib.es_b200_weight_file_read(path.encode(), name.encode(), None, 0, ctypes.byref(nelem)))
    out = np.empty(nelem.value, dtype=np.float16)
    _lib.check(lib.es_b200_weight_file_read(path.encode(), name.encode(), out.ctypes.data_as(ctypes.c_void_p),
                                            out.nbytes, None))
    return out


def weight_file_append(path, name, array):
    a = np.ascontiguousarray(array, dtype=np.float16).reshape(-1)
    _lib.check(_lib.load().es_b200_weight_file_append(path.encode(), name.encode(),
                                                      a.ctypes.data_as(ctypes.c_void_p), a.size))
