#!/usr/bin/env python3
"""Generates tests/golden/wire/: serialized protobuf messages the library's own wire codec
(csrc/wire.cc) is pinned against.

The bytes come from Google's protobuf runtime (the `protobuf` Python package), with message classes
built at run time from the reference's own src/proto/einsummable.proto (parsed here: `protoc` is not
installed).  The memgraphs are built by the reference's compilers (oracle/_ref/libes_ref.so) and
dumped as JSON by oracle/ref_graphs.cc; einsummable_b200.wire.memgraph_to_proto maps that dict to
the message's fields.  Needs the reference tree (ES_REFERENCE_ROOT or ../reference).

  <name>.json      the memgraph dict (nodes with offsets for alloc / del / partialize)
  <name>.bin       MemGraph message serialized by the protobuf runtime
  extras.json      a few small messages of other types: {message name: [json, hex bytes]}

usage: python tests/golden/make_wire.py
"""
import ctypes
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "wire")
sys.path.insert(0, ROOT)

from google.protobuf import descriptor_pb2, descriptor_pool, json_format, message_factory  # noqa: E402

from einsummable_b200.wire import memgraph_to_proto  # noqa: E402

REF = os.environ.get("ES_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
TYPES = {"int32": 5, "int64": 3, "uint64": 4, "bool": 8, "string": 9}
LABELS = {"optional": 1, "required": 2, "repeated": 3}


def file_descriptor():
    """einsummable.proto -> FileDescriptorProto (flat messages, scalar / message fields, oneofs)."""
    text = open(os.path.join(REF, "src", "proto", "einsummable.proto")).read()
    text = re.sub(r"//[^\n]*", "", text)
    fd = descriptor_pb2.FileDescriptorProto(name="einsummable.proto", package="es_proto", syntax="proto2")
    for name, body in re.findall(r"message\s+(\w+)\s*\{((?:[^{}]|\{[^{}]*\})*)\}", text):
        msg = fd.message_type.add(name=name)
        oneofs = re.findall(r"oneof\s+(\w+)\s*\{([^{}]*)\}", body)
        plain = re.sub(r"oneof\s+\w+\s*\{[^{}]*\}", "", body)
        for label, typ, fname, num in re.findall(r"(optional|required|repeated)\s+(\w+)\s+(\w+)\s*=\s*(\d+)", plain):
            f = msg.field.add(name=fname, number=int(num), label=LABELS[label])
            if typ in TYPES:
                f.type = TYPES[typ]
            else:
                f.type, f.type_name = 11, ".es_proto." + typ
        for k, (oname, obody) in enumerate(oneofs):
            msg.oneof_decl.add(name=oname)
            for typ, fname, num in re.findall(r"(\w+)\s+(\w+)\s*=\s*(\d+)", obody):
                f = msg.field.add(name=fname, number=int(num), label=1, oneof_index=k)
                if typ in TYPES:
                    f.type = TYPES[typ]
                else:
                    f.type, f.type_name = 11, ".es_proto." + typ
    return fd


def main():
    os.makedirs(OUT, exist_ok=True)
    pool = descriptor_pool.DescriptorPool()
    pool.Add(file_descriptor())
    cls = lambda name: message_factory.GetMessageClass(pool.FindMessageTypeByName("es_proto." + name))

    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libes_ref.so"))
    L.ref_graph_last_error.restype = ctypes.c_char_p
    u64 = ctypes.c_uint64

    def ok(h):
        if h < 0:
            raise RuntimeError(L.ref_graph_last_error().decode())
        return h

    graphs = {
        "c1_n64_locs2": lambda: L.ref_graph_build_c1(u64(64), 2, 2, 1),
        "c1_n64_evict_locs2": lambda: L.ref_graph_build_c1_evict(u64(64), 4, 2, 1, u64(12288)),
        "llama_tiny_locs2": lambda: L.ref_graph_build_llama(u64(64), u64(2), u64(32), u64(128), 1, u64(2), u64(16), 2, 0),
    }
    for name, build in graphs.items():
        h = ok(build())
        path = os.path.join(OUT, name + ".json")
        ok(L.ref_graph_write_json(h, path.encode()))
        with open(path) as f:
            mg = json.load(f)
        msg = json_format.ParseDict(memgraph_to_proto(mg), cls("MemGraph")())
        data = msg.SerializeToString()
        with open(os.path.join(OUT, name + ".bin"), "wb") as f:
            f.write(data)
        print(name, len(mg["nodes"]), "nodes ->", len(data), "bytes")

    extras = {
        "Einsummable": {"join_shape": [4, 5, 3], "inns": [{"idxs": [0, 2]}, {"idxs": [2, 1]}], "out_rank": 2,
                        "join": "*[hole|f32@0,hole|f32@1]", "castable": "+"},
        "Touch": {"selection": [{"d_inn": 4, "d_out": 3, "offset_inn": 1, "offset_out": 0, "size": 2}], "dtype": "f16"},
        "Fill": {"lowertri": {"lower": "f16|0", "upper": "f16|-inf", "ncol": 512, "nrow": 512, "start": -3}},
        "Placement": {"partition": {"partdims": [{"spans": [2048, 4096]}, {"spans": [11008]}]}, "locations": [0, 7]},
        "TaskGraphNode": {"move": {"src": 1, "dst": 0, "inn": 17, "size": 1 << 33}, "is_save": False},
        "MemLoc": {"offset": (1 << 40) + 16, "size": 0, "loc": -1},
    }
    out = {}
    for name, obj in extras.items():
        msg = json_format.ParseDict(obj, cls(name)())
        out[name] = [obj, msg.SerializeToString().hex()]
    with open(os.path.join(OUT, "extras.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
