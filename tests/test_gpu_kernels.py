"""Parity of the CUDA path against the reference fixtures and the oracle,
through the C ABI.  Every test here needs a B200."""
import numpy as np
import pytest
import torch

import einsummable_b200 as es
import es_oracle as O
from einsummable_b200 import _lib, einsummable_t, fill_t, scalarop_t, touch_t
from conftest import golden
from gpu_util import NP, TORCH, assert_close, run_einsummable, to_dev, to_host

pytestmark = pytest.mark.gpu
G = golden()
S = scalarop_t


@pytest.fixture(scope="module")
def km():
    k = es.kernel_manager_t(0)
    yield k
    k.close()


def case_einsummable(case):
    return einsummable_t(case["join_shape"], case["inns"], case["out_rank"], case["join"], case["castable"])


def is_pure_copy(case):
    return case["castable"] is None and case["join"].startswith("hole|")


@pytest.mark.parametrize("case", G.meta["einsummable"], ids=lambda c: c["name"])
def test_einsummable_matches_reference_fixture(km, case):
    e = case_einsummable(case)
    got = run_einsummable(km, e, G.es_inputs(case))
    want = G.es_output(case)
    assert got.dtype == want.dtype and got.shape == want.shape
    if is_pure_copy(case) or case["castable"] in ("min", "max") and case["join"].startswith("hole|"):
        # permutation / broadcast / min-max selection move bits, never round
        assert got.tobytes() == want.tobytes(), case["name"]
    else:
        assert_close(got, want, case["out_dtype"], case["name"],
                     normwise=case["castable"] in ("add", "mul"))


@pytest.mark.parametrize("case", [c for c in G.meta["einsummable"] if c["name"] in (
    "silu_mul_f16", "add_ab_b_f32", "sum_ab_a_f32", "max_ab_a_f16", "rope_c64", "exp_sub_rowmax_f32",
    "to_f32", "softmax_v3_sum_f32", "add_f64")], ids=lambda c: c["name"])
def test_unaligned_pointers_use_scalar_twin(km, case):
    e = case_einsummable(case)
    item = min(np.dtype(NP[d]).itemsize for d in list(e.join.hole_dtypes.values()) + [e.out_dtype()])
    widest = max(np.dtype(NP[d]).itemsize for d in list(e.join.hole_dtypes.values()) + [e.out_dtype()])
    got = run_einsummable(km, e, G.es_inputs(case), misalign=widest)
    assert_close(got, G.es_output(case), case["out_dtype"], case["name"],
                 normwise=case["castable"] in ("add", "mul"))


@pytest.mark.parametrize("case", G.meta["touch"], ids=lambda c: c["name"])
def test_touch_bit_exact(km, case):
    t = touch_t(case["selection"], case["castable"], case["dtype"])
    inn = to_dev(G.arrays["touch/%s/inn" % case["name"]])
    out = to_dev(G.arrays["touch/%s/out0" % case["name"]])
    km(t, None, out, inn)
    torch.cuda.synchronize()
    assert to_host(out).tobytes() == G.arrays["touch/%s/out" % case["name"]].tobytes()


def test_touch_batch_bit_exact(km):
    cases = [c for c in G.meta["touch"] if c["dtype"] == "f32"]
    touches, outs, inns, wants = [], [], [], []
    for c in cases:
        touches.append(touch_t(c["selection"], c["castable"], c["dtype"]))
        inns.append(to_dev(G.arrays["touch/%s/inn" % c["name"]]))
        outs.append(to_dev(G.arrays["touch/%s/out0" % c["name"]]))
        wants.append(G.arrays["touch/%s/out" % c["name"]])
    items = torch.empty(len(cases) * 256, dtype=torch.uint8, device="cuda:0")
    km.touch_batch(touches, None, outs, inns, items)
    torch.cuda.synchronize()
    for o, w, c in zip(outs, wants, cases):
        assert to_host(o).tobytes() == w.tobytes(), c["name"]
    # prepared form: copy touches are idempotent, so a second launch must leave the same bits
    copies = [i for i, c in enumerate(cases) if c["castable"] is None]
    outs2 = [to_dev(G.arrays["touch/%s/out0" % cases[i]["name"]]) for i in copies]
    prepared = km.prepare_touch_batch([touches[i] for i in copies], None, outs2, [inns[i] for i in copies], items)
    km.launch_prepared_touch_batch(prepared, None)
    km.launch_prepared_touch_batch(prepared, None)
    torch.cuda.synchronize()
    for o, i in zip(outs2, copies):
        assert to_host(o).tobytes() == wants[i].tobytes(), cases[i]["name"]


@pytest.mark.parametrize("i", range(len(G.meta["fill"])))
def test_lowertri_fill_bit_exact(km, i):
    c = G.meta["fill"][i]
    conv = {"INF": float("inf"), "NINF": float("-inf")}

    def val(s):
        if s in conv:
            return conv[s]
        if s.startswith("("):
            a, b = s.strip("()").split(",")
            return complex(float(a), float(b))
        return float(s)
    out = torch.zeros(c["nrow"] * c["ncol"], dtype=TORCH[c["dtype"]], device="cuda:0")
    km.lowerTri_fill(fill_t.lowertri_t(val(c["lower"]), val(c["upper"]), c["nrow"], c["ncol"], c["start"],
                                       c["dtype"]), None, out)
    torch.cuda.synchronize()
    assert to_host(out).tobytes() == G.arrays["fill/%d" % i].tobytes()


@pytest.mark.parametrize("dtype,value,n", [("f16", 1.5, 1000), ("f32", -2.25, 4099), ("f64", 3.0, 17),
                                            ("c64", 1 - 2j, 333), ("f16", float("-inf"), 7)])
def test_constant_fill_bit_exact(km, dtype, value, n):
    raw = torch.zeros(n + 3, dtype=TORCH[dtype], device="cuda:0")
    out = raw[1:n + 1]                       # odd start: exercises the scalar head/tail
    km.constant_fill(fill_t.constant_t(value, [n], dtype), None, out)
    torch.cuda.synchronize()
    got = to_host(raw)
    want = O.reference_fill_constant(value, n, dtype)
    assert got[1:n + 1].tobytes() == want.tobytes()
    assert got[0] == 0 and got[n + 1] == 0 and got[n + 2] == 0   # canaries untouched


def test_move_same_device_bit_exact(km):
    for nbytes in (16, 4096 + 16, (5 << 20) + 48, 1000):
        src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda:0")
        dst = torch.zeros(nbytes + 32, dtype=torch.uint8, device="cuda:0")
        km.move(0, src, dst[16:], nbytes, None)
        torch.cuda.synchronize()
        d = to_host(dst)
        assert d[16:16 + nbytes].tobytes() == O.reference_move(to_host(src)).tobytes()
        assert not d[:16].any() and not d[16 + nbytes:].any()


# ---- larger shapes against the executor-convention oracle ----
def test_c2_silu_mul_f16_rows(km):
    rng = np.random.default_rng(1)
    n = 64 * 11008
    x = rng.standard_normal(n).astype(np.float16)
    y = rng.standard_normal(n).astype(np.float16)
    e = einsummable_t([n], [[0], [0]], 1, S.combine(S.make_mul("f16"), [S.make_silu("f16"), S.make_identity("f16")]))
    got = run_einsummable(km, e, [x, y])
    want = O.reference_einsummable([n], [[0], [0]], 1, e.join.text, None, [x, y], "executor")
    assert_close(got, want, "f16", "silu_mul")


@pytest.mark.parametrize("castable", ["max", "add"])
@pytest.mark.parametrize("dtype,shape", [("f16", (96, 11008)), ("f32", (128, 4096)), ("f32", (4096, 512)),
                                         ("f32", (3, 70000)), ("f16", (2, 1 << 20))])
def test_c2_row_reductions(km, castable, dtype, shape):
    rng = np.random.default_rng(2)
    x = rng.standard_normal(shape[0] * shape[1]).astype(NP[dtype])
    e = einsummable_t(list(shape), [[0, 1]], 1, S.make_identity(dtype), castable)
    got = run_einsummable(km, e, [x])
    xf = x.reshape(shape).astype(np.float64)
    want = (xf.max(axis=1) if castable == "max" else xf.sum(axis=1)).astype(NP[dtype])
    if castable == "max":
        assert got.tobytes() == want.tobytes()
    else:
        # sums of N(0,1): compare at the scale of the partial sums, not of a cancelling total
        scale = np.sqrt(shape[1])
        rtol = 1e-2 if dtype == "f16" else 1e-5
        assert np.abs(got.astype(np.float64) - xf.sum(axis=1)).max() <= rtol * scale


def test_c2_exp_sub_rowmax_and_fused_sum(km):
    rng = np.random.default_rng(3)
    a, b = 64, 11008
    x = rng.standard_normal(a * b).astype(np.float32)
    m = x.reshape(a, b).max(axis=1)
    join = S.combine(S.make_exp("f32"), [S.make_sub("f32")])
    e = einsummable_t([a, b], [[0, 1], [0]], 2, join)
    got = run_einsummable(km, e, [x, m])
    want = np.exp(x.reshape(a, b).astype(np.float64) - m[:, None].astype(np.float64)).reshape(-1)
    assert_close(got, want.astype(np.float32), "f32", "exp(x-rowmax)")
    e2 = einsummable_t([a, b], [[0, 1], [0]], 1, join, "add")
    got2 = run_einsummable(km, e2, [x, m])
    assert_close(got2, want.reshape(a, b).sum(axis=1).astype(np.float32), "f32", "sum exp(x-rowmax)")


def test_c3_permutation_bhsd_bshd_bit_exact(km):
    rng = np.random.default_rng(4)
    shape = (4, 64, 8, 128)  # b s h d
    for dtype in ("f16", "f32"):
        x = rng.uniform(-1, 1, int(np.prod(shape))).astype(NP[dtype])
        # out[b,h,s,d] = in[b,s,h,d]: join modes (b,h,s,d), input holds (b,s,h,d) -> acbd->abcd
        e = einsummable_t([4, 8, 64, 128], [[0, 2, 1, 3]], 4, S.make_identity(dtype))
        got = run_einsummable(km, e, [x])
        want = np.ascontiguousarray(x.reshape(shape).transpose(0, 2, 1, 3)).reshape(-1)
        assert got.tobytes() == want.tobytes()


def test_transposes_bit_exact(km):
    rng = np.random.default_rng(5)
    for dtype, (a, b) in [("f16", (300, 257)), ("f32", (1000, 33)), ("f64", (65, 64)), ("c64", (40, 100))]:
        x = rng.uniform(-1, 1, a * b).astype(NP[dtype])
        e = einsummable_t([a, b], [[1, 0]], 2, S.make_identity(dtype))   # ba->ab
        got = run_einsummable(km, e, [x])
        assert got.tobytes() == np.ascontiguousarray(x.reshape(b, a).T).reshape(-1).tobytes()


def test_column_reductions(km):
    rng = np.random.default_rng(6)
    for (a, b) in [(4096, 300), (37, 5000), (3, 100000)]:
        x = rng.standard_normal(a * b).astype(np.float32)
        e = einsummable_t([a, b], [[1, 0]], 1, S.make_identity("f32"), "add")   # ba->a
        got = run_einsummable(km, e, [x])
        want = x.reshape(b, a).astype(np.float64).sum(axis=0)
        assert np.abs(got - want).max() <= 1e-5 * np.sqrt(b) * 4


def test_touch_c1_partial_sum_group(km):
    """C1's pattern: the first touch of a group is a copy, the second accumulates
    (src/engine/gpu/exec_graph.cc:368-378); 2 partials, so the result is order independent."""
    rng = np.random.default_rng(7)
    n = 2048 * 2048
    p0 = rng.uniform(-1, 1, n).astype(np.float32)
    p1 = rng.uniform(-1, 1, n).astype(np.float32)
    out = torch.full((n,), 7.0, dtype=torch.float32, device="cuda:0")
    sel = [(n, n, 0, 0, n)]
    km(touch_t(sel, None, "f32"), None, out, to_dev(p0))
    km(touch_t(sel, "add", "f32"), None, out, to_dev(p1))
    torch.cuda.synchronize()
    assert to_host(out).tobytes() == (p0 + p1).tobytes()


def test_touch_c3_subregions(km):
    """C3: blocks of a [b,h,s,d] tensor copied / accumulated into a destination
    with a different split, f16 and f32."""
    rng = np.random.default_rng(8)
    full = (8, 64, 8, 128)
    for dtype in ("f16", "f32"):
        src_block = rng.uniform(-1, 1, (4, 32, 4, 64)).astype(NP[dtype])   # one source block (p=2)
        dst = rng.uniform(-1, 1, full).astype(NP[dtype])
        for castable in (None, "add", "max"):
            sel = [(4, 8, 1, 2, 3), (32, 64, 0, 16, 32), (4, 8, 2, 5, 2), (64, 128, 0, 64, 64)]
            want = dst.copy().reshape(-1)
            O.reference_touch(sel, castable, want, src_block.reshape(-1))
            d_out = to_dev(dst.reshape(-1))
            km(touch_t(sel, castable, dtype), None, d_out, to_dev(src_block.reshape(-1)))
            torch.cuda.synchronize()
            assert to_host(d_out).tobytes() == want.tobytes(), (dtype, castable)


# ---- error behaviour through the C ABI ----
def test_launch_without_build_throws(km):
    e = einsummable_t([123], [[0]], 1, S.make_exp("f32"))
    with pytest.raises(es.es_error) as ei:
        km(e, None, 0, [0])
    assert ei.value.status == _lib.ES_NOT_BUILT


def test_wrong_input_count_and_workspace(km):
    e = einsummable_t([2, 1 << 22], [[0, 1]], 1, S.make_identity("f32"), "add")
    ws = km.build(e)
    assert ws and ws > 0 and "red_split" in km.kernel_info(e)
    x = torch.zeros(2 << 22, dtype=torch.float32, device="cuda:0")
    out = torch.zeros(2, dtype=torch.float32, device="cuda:0")
    with pytest.raises(es.es_error) as ei:
        km(e, None, out, [x, x])
    assert ei.value.status == _lib.ES_BAD_ARGUMENT
    with pytest.raises(es.es_error) as ei:
        km(e, None, out, [x])                      # workspace missing
    assert ei.value.status == _lib.ES_WORKSPACE_TOO_SMALL
    small = torch.zeros(16, dtype=torch.uint8, device="cuda:0")
    with pytest.raises(es.es_error) as ei:
        km(e, None, out, [x], (small, 16))
    assert ei.value.status == _lib.ES_WORKSPACE_TOO_SMALL


def test_touch_rejects_out_of_bounds_region(km):
    x = torch.zeros(100, dtype=torch.float32, device="cuda:0")
    with pytest.raises(es.es_error) as ei:
        km(touch_t([(10, 10, 5, 0, 6)], None, "f32"), None, x, x)
    assert ei.value.status == _lib.ES_BAD_DESCRIPTOR
    with pytest.raises(es.es_error):
        km(touch_t([(10, 10, 0, 0, 10)], "max", "c64"), None, x, x)


def test_build_is_idempotent(km):
    e = einsummable_t([64, 64], [[0, 1], [1]], 2, S.make_add("f32"))
    km.build(e)
    first = km._ids[km._key(e)]
    km.build(einsummable_t([64, 64], [[0, 1], [1]], 2, S.make_add("f32")))
    assert km._ids[km._key(e)] == first
    # an un-merged spelling of the same op maps to the same kernel
    e2 = einsummable_t([8, 8, 64], [[0, 1, 2], [2]], 3, S.make_add("f32"))
    km.build(e2)
    assert km._ids[km._key(e2)][0] == first[0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_move_between_two_gpus_bit_exact(km):
    """move_t across GPUs (one process, peer access), small (pull kernel) and large (copy engine)."""
    for nbytes in (4096, (3 << 20) + 16, (9 << 20)):
        src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda:1")
        dst = torch.zeros(nbytes + 32, dtype=torch.uint8, device="cuda:0")
        torch.cuda.synchronize(1)
        km.move(1, src, dst[16:], nbytes, None)
        torch.cuda.synchronize(0)
        d = to_host(dst)
        assert d[16:16 + nbytes].tobytes() == to_host(src).tobytes()
        assert not d[:16].any() and not d[16 + nbytes:].any()
