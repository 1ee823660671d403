"""The interchange formats (csrc/wire.cc): the protobuf wire codec against bytes serialized by
Google's protobuf runtime from the reference's own .proto (tests/golden/make_wire.py), and the
weight file format of llama/from_pth2.py / llama/reader.cc."""
import json
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN_DIR
from einsummable_b200 import _lib, wire

WIRE = os.path.join(GOLDEN_DIR, "wire")
GRAPHS = ["c1_n64_locs2", "c1_n64_evict_locs2", "llama_tiny_locs2"]


def load(name):
    with open(os.path.join(WIRE, name + ".json")) as f:
        mg = json.load(f)
    with open(os.path.join(WIRE, name + ".bin"), "rb") as f:
        return mg, f.read()


@pytest.mark.parametrize("name", GRAPHS)
def test_memgraph_to_wire_is_byte_identical_to_protobuf(name):
    mg, data = load(name)
    assert wire.memgraph_to_wire(mg) == data


@pytest.mark.parametrize("name", GRAPHS)
def test_memgraph_from_wire_recovers_every_node(name):
    mg, data = load(name)
    back = wire.memgraph_from_wire(data)
    assert back["num_locs"] == mg["num_locs"] and back["storage_locs"] == mg["storage_locs"]
    assert len(back["nodes"]) == len(mg["nodes"])
    for a, b in zip(back["nodes"], mg["nodes"]):
        assert a["kind"] == b["kind"] and a["inns"] == b["inns"]
        for k, v in b.items():
            if k == "fill":
                for part in ("value", "lower", "upper"):
                    if part in v:
                        assert a["fill"][part]["raw"] == v[part]["raw"], (a, b)
                assert {kk: vv for kk, vv in a["fill"].items() if kk not in ("value", "lower", "upper")} == \
                    {kk: vv for kk, vv in v.items() if kk not in ("value", "lower", "upper")}
            else:
                assert a[k] == v, (k, a, b)
    assert back["mem_sizes"] == [int(x) for x in mg["mem_sizes"]] or all(
        x <= int(y) for x, y in zip(back["mem_sizes"], mg["mem_sizes"]))
    # and the decoded graph serializes to the same bytes again
    assert wire.memgraph_to_wire(back) == data


def test_a_decoded_memgraph_is_what_the_schedule_builder_takes():
    from einsummable_b200.memgraph import schedule_units
    mg, data = load("llama_tiny_locs2")
    units_a = schedule_units(mg, {0, 1}, False)
    units_b = schedule_units(wire.memgraph_from_wire(data), {0, 1}, False)
    assert [(u["kind"], u["deps"]) for u in units_a] == [(u["kind"], u["deps"]) for u in units_b]


def test_other_messages_and_edge_values():
    with open(os.path.join(WIRE, "extras.json")) as f:
        extras = json.load(f)
    for name, (obj, hexbytes) in extras.items():
        data = bytes.fromhex(hexbytes)
        assert wire.wire_from_json(name, obj) == data, name
        assert wire.wire_to_json(name, data) == obj, name
    # negative int32 / int64 travel as ten-byte varints; packed repeated scalars are accepted on input
    assert wire.wire_to_json("EsInn", bytes([0x0A, 0x03, 0x01, 0x02, 0x03])) == {"idxs": [1, 2, 3]}
    assert wire.wire_to_json("MemLoc", wire.wire_from_json("MemLoc", {"offset": 1, "size": 2, "loc": -5}))["loc"] == -5
    # unknown fields are skipped, the last occurrence of a scalar wins
    assert wire.wire_to_json("Mem", bytes([0x08, 0x01, 0x08, 0x07, 0x78, 0x05, 0x10, 0x02])) == {"offset": 7, "size": 2}


def test_wire_errors():
    with pytest.raises(_lib.es_error):
        wire.wire_to_json("NoSuchMessage", b"")
    with pytest.raises(_lib.es_error):
        wire.wire_to_json("Mem", bytes([0x08]))                 # truncated varint
    with pytest.raises(_lib.es_error):
        wire.wire_to_json("Einsummable", bytes([0x22, 0x7F]))   # string longer than the message
    with pytest.raises(_lib.es_error):
        wire.wire_from_json("Mem", {"offset": 1, "bogus": 2})
    with pytest.raises(_lib.es_error):
        wire.wire_from_json("Mem", {"offset": "one"})


def test_weight_file_round_trip_and_layout(tmp_path):
    path = str(tmp_path / "weights_00")
    rng = np.random.default_rng(3)
    tensors = {"tok_embeddings.weight": rng.standard_normal(300).astype(np.float16),
               "layers.0.attention.wq.weight": rng.standard_normal(4096).astype(np.float16),
               "norm.weight": np.ones(7, np.float16)}
    for k, v in tensors.items():
        wire.weight_file_append(path, k, v)
    # byte layout as llama/from_pth2.py writes it: 50-byte padded name, int64 count, f16 values
    with open(path, "rb") as f:
        raw = f.read()
    first = "tok_embeddings.weight"
    assert raw[:50] == first.ljust(50).encode() and struct.unpack("<q", raw[50:58])[0] == 300
    assert raw[58:58 + 600] == tensors[first].tobytes()
    assert len(raw) == sum(58 + 2 * v.size for v in tensors.values())
    assert wire.weight_file_list(path) == [(k, v.size) for k, v in tensors.items()]
    for k, v in tensors.items():
        assert wire.weight_file_read(path, k).tobytes() == v.tobytes()
    with pytest.raises(_lib.es_error):
        wire.weight_file_read(path, "missing.weight")
    with pytest.raises(_lib.es_error):
        wire.weight_file_append(path, "x" * 51, np.zeros(1, np.float16))
    with open(path, "ab") as f:
        f.write(b"truncated")
    with pytest.raises(_lib.es_error):
        wire.weight_file_list(path)
