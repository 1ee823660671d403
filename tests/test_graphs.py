"""Graph level on CPU: the oracle's memgraph interpreter against the results the
reference's own interpreter produced for the same memgraphs (tests/golden/graphs)."""
import json
import os

import numpy as np
import pytest

import es_oracle as O
from conftest import GOLDEN_DIR, GraphArrays

GRAPHS = os.path.join(GOLDEN_DIR, "graphs")
ARR = GraphArrays()
SMALL = ["c1_n64_locs1", "c1_n64_locs2", "llama_tiny_locs1", "llama_tiny_locs2", "llama_tiny_locs4", "llama_tiny_tp_locs2", "llama_tiny_tp_locs4",
         "llama_train_tiny_locs1", "llama_train_tiny_locs2", "llama_train_adamw_tiny_locs1",
         "llama_train_adamw_tiny_locs2", "llama_train_lora_tiny_locs1", "llama_train_lora_tiny_locs2"]


def load(name):
    path = os.path.join(GRAPHS, name + ".json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    import gzip
    with gzip.open(path + ".gz", "rt") as f:
        return json.load(f)


def inputs_of(name):
    pre = name + "/in/"
    return {k[len(pre):]: ARR[k] for k in ARR.files if k.startswith(pre)}


def outputs_of(name):
    pre = name + "/out/"
    return {k[len(pre):]: ARR[k] for k in ARR.files if k.startswith(pre)}


@pytest.mark.parametrize("name", SMALL)
def test_oracle_memgraph_interp_matches_reference(name):
    mg = load(name)
    bufs = O.memgraph_place_inputs(mg, inputs_of(name))
    O.run_memgraph(mg, bufs, "interp")
    got = O.memgraph_collect_outputs(mg, bufs)
    for k, want in outputs_of(name).items():
        g = got[k]
        assert g.shape == want.shape and g.dtype == want.dtype
        scale = np.abs(want.astype(np.float64)).max()
        err = np.abs(g.astype(np.float64) - want.astype(np.float64)).max()
        # f16 trees with exp / pow differ from half.hpp in the last place here and there
        tol = 4e-3 if want.dtype == np.float16 else 1e-6
        if name.startswith("llama_train"):
            # numpy's exp / log / power differ from libm's in the last place of f32; the backward
            # pass carries that into gradients that are small differences of larger terms (the
            # attention gradients of these fixtures are 1e-9 .. 1e-12)
            tol = 2e-5
        assert err <= tol * scale, (name, k, err, scale)


@pytest.mark.parametrize("name", SMALL)
def test_oracle_memgraph_executor_mode_close(name):
    mg = load(name)
    bufs = O.memgraph_place_inputs(mg, inputs_of(name))
    O.run_memgraph(mg, bufs, "executor")
    got = O.memgraph_collect_outputs(mg, bufs)
    for k, want in outputs_of(name).items():
        scale = np.abs(want.astype(np.float64)).max()
        err = np.abs(got[k].astype(np.float64) - want.astype(np.float64)).max()
        # a whole layer chains ~15 f16 ops; the interpreter additionally accumulates every
        # contraction in f16, so the two conventions drift apart by about 1e-2 of the output scale
        tol = 2e-2 if want.dtype == np.float16 else 1e-5
        if name.startswith("llama_train"):
            # the attention gradients (1e-9) are what is left of sums of terms a thousand times
            # larger: summation order alone moves them by 1e-5 of their own scale in f32
            tol = 1e-4
        assert err <= tol * scale, (name, k, err, scale)


def test_llama7b_layer_statistics():
    import gzip
    want = {1: (0, 0), 2: (29, 189059072), 4: (145, 541472768), 8: (429, 675930112)}
    for n, (moves, nbytes) in want.items():
        with gzip.open(os.path.join(GRAPHS, "llama7b_layer_locs%d.json.gz" % n), "rt") as f:
            mg = json.load(f)
        assert mg["num_locs"] == n
        assert mg["taskgraph"]["move"] == moves and mg["taskgraph"]["move_bytes"] == nbytes
        assert abs(mg["taskgraph"]["contraction_flops"] - 847.157e9) < 1e7


@pytest.mark.parametrize("name", ["llama_tiny_locs2", "llama_tiny_locs4", "c1_n64_locs2", "llama_tiny_tp_locs2"])
def test_move_runs_cut_groups_the_same_way_on_every_rank(name):
    """The NCCL transport posts a rank's members of one run as one group.  Runs must come from
    the global order alone: no non-move node inside a run, no dependency between two members."""
    from einsummable_b200.memgraph import move_runs
    mg = load(name)
    runs = move_runs(mg)
    moves = [n for n in mg["nodes"] if n["kind"] == "move"]
    assert sorted(runs) == sorted(n["id"] for n in moves)
    bookkeeping = ("alloc", "del", "inputmem", "partialize")
    last_run, broken = None, True
    for n in mg["nodes"]:
        if n["kind"] in bookkeeping:
            continue
        if n["kind"] != "move":
            broken = True
            continue
        r = runs[n["id"]]
        assert last_run is None or r >= last_run
        if r == last_run:
            assert not broken, "a compute node sits inside run %d" % r
        last_run, broken = r, False
    # no member of a run reaches another member through bookkeeping nodes
    by_id = {n["id"]: n for n in mg["nodes"]}

    def move_ancestors(i, seen):
        for j in by_id[i]["inns"]:
            k = by_id[j]["kind"]
            if k == "move":
                seen.add(j)
            elif k in bookkeeping:
                move_ancestors(j, seen)
        return seen

    for n in moves:
        for j in move_ancestors(n["id"], set()):
            assert runs[j] != runs[n["id"]]


def test_compose_substitutes_and_renumbers():
    from einsummable_b200.fuse import compose
    a = {"join_shape": [4, 8], "inns": [[0, 1], [1]], "out_rank": 2,
         "join": "+[hole|f32@0,*[constant{f32|-1},hole|f32@1]]", "castable": None}      # x[a,b] - m[b]
    b = {"join_shape": [8, 4], "inns": [[1, 0], [0, 1]], "out_rank": 1,                   # sum_b y[a',b'] * A^T
         "join": "*[hole|f32@1,exp[hole|f32@0]]", "castable": "add"}
    c = compose(a, b, 0)
    # a's modes (0, 1) are b's modes (1, 0); b's other input moves behind a's two inputs
    assert c["inns"] == [[1, 0], [0], [0, 1]]
    assert c["join"] == "*[hole|f32@2,exp[+[hole|f32@0,*[constant{f32|-1},hole|f32@1]]]]"
    assert c["castable"] == "add" and c["out_rank"] == 1 and c["join_shape"] == [8, 4]


@pytest.mark.parametrize("name", ["llama_tiny_locs1", "llama_train_tiny_locs1", "c1_n64_locs1", "llama_tiny_locs2", "llama_tiny_tp_locs2",
                                  "llama_tiny_locs4", "llama_train_tiny_locs2", "llama_train_adamw_tiny_locs1",
                                  "llama_train_adamw_tiny_locs2", "llama_train_lora_tiny_locs1",
                                  "llama_train_lora_tiny_locs2"])
def test_fused_memgraph_still_matches_reference(name):
    """Folding elementwise producers into their readers must not change the results beyond the
    rounding of the intermediates that are no longer written (none in f32 beyond reassociation)."""
    from einsummable_b200.fuse import fuse_elementwise_chains
    mg = load(name)
    fused, n = fuse_elementwise_chains(mg)
    assert n > 0 or name.startswith("c1")
    assert len(fused["nodes"]) == len(mg["nodes"])          # ids keep indexing the list
    for mode in ("interp", "executor"):
        bufs = O.memgraph_place_inputs(fused, inputs_of(name))
        O.run_memgraph(fused, bufs, mode)
        got = O.memgraph_collect_outputs(fused, bufs)
        for k, want in outputs_of(name).items():
            scale = np.abs(want.astype(np.float64)).max()
            err = np.abs(got[k].astype(np.float64) - want.astype(np.float64)).max()
            tol = 2e-2 if want.dtype == np.float16 else 1e-4
            assert err <= tol * scale, (name, mode, k, err, scale)


def test_attention_chain_becomes_one_node_and_still_matches_reference():
    """fuse_attention replaces scores / max / sum / normalise / values by one node; the oracle computes
    that node as the reference's five einsummables, so the result is, bit for bit, the folded graph's."""
    from einsummable_b200.fuse import fuse_attention, fuse_elementwise_chains
    name = "llama_tiny_locs1"
    mg = load(name)
    assert fuse_attention(mg)[1] == 0            # the pattern is the folded one
    folded, _ = fuse_elementwise_chains(mg)
    fused, n = fuse_attention(folded)
    assert n == 1 and len(fused["nodes"]) == len(mg["nodes"])
    (node,) = [x for x in fused["nodes"] if "attention" in x]
    a = node["attention"]
    assert (a["batch"], a["heads"], a["rows"], a["keys"], a["head_dim"]) == (2, 2, 16, 16, 32)
    assert (a["skip_known"], a["skip_from"]) == (1, 0)       # the mask is the lower-triangular fill
    # Q and K are [batch, row, head, dim] tensors, the result [batch, head, row, dim]
    assert a["q_stride"] == [16 * 64, 32, 64] and a["k_stride"] == a["q_stride"] and a["out_stride"] == [1024, 512, 32]
    gone = sum(1 for x, y in zip(folded["nodes"], fused["nodes"]) if x["kind"] == "apply" and y.get("folded"))
    assert gone == 4
    results = []
    for g in (folded, fused):
        bufs = O.memgraph_place_inputs(g, inputs_of(name))
        O.run_memgraph(g, bufs, "interp")
        results.append(O.memgraph_collect_outputs(g, bufs))
    for k, want in outputs_of(name).items():
        assert np.array_equal(results[0][k], results[1][k]), k
        scale = np.abs(want.astype(np.float64)).max()
        assert np.abs(results[1][k].astype(np.float64) - want.astype(np.float64)).max() <= 2e-2 * scale
    # the training graphs keep the softmax result for the backward pass: nothing to replace
    t, _ = fuse_elementwise_chains(load("llama_train_tiny_locs1"))
    assert fuse_attention(t)[1] == 0


def test_fusion_never_folds_a_tensor_that_a_move_ships():
    from einsummable_b200.fuse import fuse_elementwise_chains
    mg = load("llama_tiny_locs2")
    fused, n = fuse_elementwise_chains(mg)
    assert n > 0
    folded = {x["id"] for x in fused["nodes"] if x.get("folded")}
    for node in fused["nodes"]:
        if node["kind"] == "move":
            assert not (set(node["inns"]) & folded)
    # the moves themselves are untouched, so every rank still sees the same exchange steps
    assert [x for x in fused["nodes"] if x["kind"] == "move"] == [x for x in mg["nodes"] if x["kind"] == "move"]


def _mini(nodes, outputs=()):
    """A hand-made one-location memgraph: only what the fusion pass reads."""
    return {"num_locs": 1, "mem_sizes": [1 << 20], "taskgraph": {}, "inputs": [],
            "outputs": [{"blocks": [{"loc": 0, "offset": o, "size": s}]} for o, s in outputs], "nodes": nodes}


def _ew(i, inns, out, reads, join="hole|f32@0", n=64, castable=None, rank2=False):
    shape = [8, 8] if rank2 else [n]
    idx = [0, 1] if rank2 else [0]
    return {"id": i, "inns": inns, "kind": "apply", "loc": 0, "group": -1,
            "mems": [list(out)] + [list(r) for r in reads],
            "einsummable": {"join_shape": shape, "inns": [idx for _ in reads], "out_rank": len(shape),
                            "join": join, "castable": castable}}


def test_fusion_hazards_on_hand_made_graphs():
    from einsummable_b200.fuse import fuse_elementwise_chains
    X, A, B, C = (0, 256), (256, 256), (512, 256), (768, 256)
    sq = "power{2}[hole|f32@0]"
    exp = "exp[hole|f32@0]"
    # plain chain: exp(x^2) in one node
    mg = _mini([_ew(0, [], A, [X], sq), _ew(1, [0], B, [A], exp)], outputs=[B])
    f, n = fuse_elementwise_chains(mg)
    assert n == 1 and f["nodes"][1]["einsummable"]["join"] == "exp[power{2}[hole|f32@0]]"
    assert f["nodes"][1]["mems"] == [list(B), list(X)] and f["nodes"][0].get("folded")
    # the producer's result is itself saved: it has to be written
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), _ew(1, [0], B, [A], exp)], outputs=[A, B]))[1] == 0
    # a node between the two overwrites what the producer read: the reader cannot read it later
    clobber = _ew(1, [], X, [C], sq)
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), clobber, _ew(2, [0], B, [A], exp)], outputs=[B]))[1] == 0
    # the reader's own output lies on the producer's input
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), _ew(1, [0], X, [A], exp)], outputs=[X]))[1] == 0
    # the reader uses the result in two slots
    two = _ew(1, [0], B, [A, A], "*[hole|f32@0,hole|f32@1]")
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), two], outputs=[B]))[1] == 0
    # a plain contraction keeps its operands materialised (it runs on the tensor cores)
    mm = {"id": 1, "inns": [0], "kind": "apply", "loc": 0, "group": -1, "mems": [list(B), list(A), list(C)],
          "einsummable": {"join_shape": [8, 8, 8], "inns": [[0, 2], [2, 1]], "out_rank": 2,
                          "join": "*[hole|f32@0,hole|f32@1]", "castable": "add"}}
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq, rank2=True), mm], outputs=[B]))[1] == 0
    # two readers: folded into both, evaluated twice
    r1, r2 = _ew(1, [0], B, [A], exp), _ew(2, [0], C, [A], "log[hole|f32@0]")
    f, n = fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), r1, r2], outputs=[B, C]))
    assert n == 1 and [x["mems"][1] for x in f["nodes"][1:]] == [list(X), list(X)]
    # a reduction as the reader keeps its castable and output rank
    red = {"id": 1, "inns": [0], "kind": "apply", "loc": 0, "group": -1, "mems": [[2048, 32], list(A)],
           "einsummable": {"join_shape": [8, 8], "inns": [[0, 1]], "out_rank": 1, "join": "hole|f32@0", "castable": "add"}}
    f, n = fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq, rank2=True), red], outputs=[(2048, 32)]))
    assert n == 1 and f["nodes"][1]["einsummable"] == {"join_shape": [8, 8], "inns": [[0, 1]], "out_rank": 1,
                                                       "join": sq, "castable": "add"}


def test_fusion_leaves_readers_that_view_the_bytes_differently():
    """The taskgraph lets a node read the same bytes under another shape (squeeze) or dtype (a
    complex view of float pairs), src/einsummable/taskgraph.cc:765-793: a producer is never folded
    into such a reader, and a later writer into memory the folded producer read waits for the reader."""
    from einsummable_b200.fuse import fuse_elementwise_chains
    X, A, B, C = (0, 256), (256, 256), (512, 256), (768, 256)
    sq = "power{2}[hole|f32@0]"
    # producer writes [64]; the reader takes the same 256 bytes as [8, 8]
    reader = _ew(1, [0], B, [A], "exp[hole|f32@0]", rank2=True)
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), reader], outputs=[B]))[1] == 0
    # ... and the other way round (more modes in the producer than in the reader's slot)
    reader = _ew(1, [0], B, [A], "exp[hole|f32@0]")
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq, rank2=True), reader], outputs=[B]))[1] == 0
    # producer writes 64 f32; the reader takes them as 32 c64
    cview = _ew(1, [0], B, [A], "conj[hole|c64@0]", n=32)
    assert fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), cview], outputs=[B]))[1] == 0
    # producer converts to f16, the reader's hole is f32 over half as many... same count, other dtype
    conv = _ew(0, [], A, [X], "to_f16[hole|f32@0]")
    assert fuse_elementwise_chains(_mini([conv, _ew(1, [0], B, [A], "exp[hole|f32@0]")], outputs=[B]))[1] == 0
    # same shape and dtype: folded, and the later writer into X now depends on the reader
    writer = _ew(2, [], X, [C], sq)
    f, n = fuse_elementwise_chains(_mini([_ew(0, [], A, [X], sq), _ew(1, [0], B, [A], "exp[hole|f32@0]"), writer],
                                         outputs=[B]))
    assert n == 1 and f["nodes"][2]["inns"] == [1]


@pytest.mark.parametrize("accumulate", ["f32", "f64"])
@pytest.mark.parametrize("name", ["c1_n64_locs2", "llama_tiny_locs1", "llama_tiny_locs4", "llama_train_tiny_locs2",
                                  "llama_train_adamw_tiny_locs1", "llama_train_lora_tiny_locs2"])
def test_cpu_engine_matches_reference(name, accumulate):
    """oracle/cpu_engine.py (the timed CPU baseline and the full-size oracle) against the reference
    interpreter's results on the graphs small enough for the interpreter, same tolerances as the GPU runner."""
    from cpu_engine import cpu_engine_t
    mg = load(name)
    eng = cpu_engine_t(mg, accumulate=accumulate, threads=2)
    for k, v in inputs_of(name).items():
        eng.set_input(k, v)
    eng.run()
    for k, ref in outputs_of(name).items():
        got = eng.get_output(k)
        scale = np.abs(ref.astype(np.float64)).max()
        err = np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()
        tol = 2e-2 if ref.dtype == np.float16 else (1e-4 if name.startswith("llama_train") else 1e-5)
        assert err <= tol * scale, (name, k, err, scale)
    eng.run()       # groups reset per run
    for k, ref in outputs_of(name).items():
        assert np.isfinite(eng.get_output(k).astype(np.float64)).all()


def test_full_size_fixture_is_present_and_sane():
    z = np.load(os.path.join(GOLDEN_DIR, "c4_full.npz"))
    assert z["scores"].shape == (4, 32000) and z["scores"].dtype == np.float16
    assert np.isfinite(z["scores"].astype(np.float32)).all() and np.abs(z["scores"]).max() > 1
    assert z["train/loss"].shape == (4,) and np.isfinite(z["train/loss"]).all()


EVICT = np.load(os.path.join(GRAPHS, "graphs_evict.npz"))


@pytest.mark.parametrize("name", ["c1_n64_evict_locs1", "c1_n64_evict_locs2"])
def test_oracle_runs_memgraphs_with_evict_and_load(name):
    """Memgraphs the reference compiled under a memory limit (evict / load nodes, inputs that start
    out in storage): the oracle's interpreter against the reference's reference_compute_memgraph
    with storage, bit for bit in interp mode."""
    mg = load(name)
    kinds = {n["kind"] for n in mg["nodes"]}
    assert {"evict", "load", "inputsto"} <= kinds
    pre = name + "/in/"
    ins = {k[len(pre):]: EVICT[k] for k in EVICT.files if k.startswith(pre)}
    storage = {}
    bufs = O.memgraph_place_inputs(mg, ins, storage)
    O.run_memgraph(mg, bufs, "interp", storage=storage)
    got = O.memgraph_collect_outputs(mg, bufs, storage)
    ref = EVICT[name + "/out/out"]
    assert got["out"].tobytes() == ref.tobytes()
