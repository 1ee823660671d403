"""The C restatement (oracle/es_oracle.c, the timed CPU baseline) against the
fixtures produced by the reference's interpreter."""
import ctypes
import os

import numpy as np
import pytest

from conftest import ROOT, golden, ulp_distance

G = golden()
LIB = os.path.join(ROOT, "oracle", "libes_oracle.so")
pytestmark = pytest.mark.skipif(not os.path.exists(LIB), reason="oracle/libes_oracle.so not built (make -C oracle)")


@pytest.fixture(scope="module")
def lib():
    return ctypes.CDLL(LIB)


def p(a):
    return ctypes.c_void_p(a.ctypes.data)


def case(name):
    return next(c for c in G.meta["einsummable"] if c["name"] == name)


def u64(v):
    return ctypes.c_uint64(v)


def test_silu_mul(lib):
    for name, fn in (("silu_mul_f16", lib.oracle_silu_mul_f16), ("silu_mul_f32", lib.oracle_silu_mul_f32)):
        c = case(name)
        x, y = G.es_inputs(c)
        out = np.zeros_like(x)
        fn(u64(x.size), p(out), p(x), p(y))
        assert ulp_distance(out, G.es_output(c)) <= 4, name


def test_exp_sub(lib):
    for name, fn in (("exp_sub_rowmax_f16", lib.oracle_exp_sub_ab_a_f16),
                     ("exp_sub_rowmax_f32", lib.oracle_exp_sub_ab_a_f32)):
        c = case(name)
        x, m = G.es_inputs(c)
        out = np.zeros_like(x)
        fn(u64(c["join_shape"][0]), u64(c["join_shape"][1]), p(out), p(x), p(m))
        assert ulp_distance(out, G.es_output(c)) <= 2, name


@pytest.mark.parametrize("name,fn,code", [
    ("sum_ab_a_f32", "oracle_reduce_ab_a_f32", 0), ("sum_ab_a_f16", "oracle_reduce_ab_a_f16", 0),
    ("max_ab_a_f32", "oracle_reduce_ab_a_f32", 3), ("max_ab_a_f16", "oracle_reduce_ab_a_f16", 3),
    ("min_ab_a_f64", "oracle_reduce_ab_a_f64", 2), ("prod_ab_a_f32", "oracle_reduce_ab_a_f32", 1)])
def test_reductions(lib, name, fn, code):
    c = case(name)
    (x,) = G.es_inputs(c)
    want = G.es_output(c)
    out = np.zeros_like(want)
    getattr(lib, fn)(code, u64(c["join_shape"][0]), u64(c["join_shape"][1]), p(out), p(x))
    if code >= 2:
        assert out.tobytes() == want.tobytes()
    else:
        # f64 running total (CPU executor) vs the interpreter's accumulation in the tensor dtype
        rtol = 1e-2 if want.dtype == np.float16 else 1e-5
        scale = np.abs(x.astype(np.float64)).reshape(c["join_shape"]).sum(axis=1)
        assert (np.abs(out.astype(np.float64) - want.astype(np.float64)) <= rtol * scale).all()


def test_reduce_exp_sub(lib):
    c = case("exp_sub_sum_f32")
    x, m = G.es_inputs(c)
    out = np.zeros(c["join_shape"][0], dtype=np.float32)
    lib.oracle_reduce_exp_sub_f32(u64(c["join_shape"][0]), u64(c["join_shape"][1]), p(out), p(x), p(m))
    np.testing.assert_allclose(out, G.es_output(c), rtol=1e-5)


@pytest.mark.parametrize("c", G.meta["touch"], ids=lambda c: c["name"])
def test_touch_bit_exact(lib, c):
    code = {"f16": 0, "f32": 1, "f64": 2, "c64": 3}[c["dtype"]]
    cast = {None: -1, "add": 0, "mul": 1, "min": 2, "max": 3}[c["castable"]]
    sel = c["simplified"]
    dims = (ctypes.c_uint64 * (5 * len(sel)))(*[v for s in sel for v in s])
    out = G.arrays["touch/%s/out0" % c["name"]].copy()
    inn = G.arrays["touch/%s/inn" % c["name"]]
    assert lib.oracle_touch(len(sel), dims, cast, code, p(out), p(inn)) == 0
    assert out.tobytes() == G.arrays["touch/%s/out" % c["name"]].tobytes()


def test_matmul_f32(lib):
    c = case("mm_ss_f32")
    a, b = G.es_inputs(c)
    ni, nk, nj = c["join_shape"]
    out = np.zeros(ni * nk, dtype=np.float32)
    lib.oracle_matmul_f32(u64(ni), u64(nj), u64(nk), p(out), p(a), p(b))
    np.testing.assert_allclose(out, G.es_output(c), rtol=1e-5, atol=1e-5)


def test_fill_lowertri(lib):
    for i, c in enumerate(G.meta["fill"]):
        want = G.arrays["fill/%d" % i]
        eb = want.dtype.itemsize
        out = np.zeros_like(want)
        lo = want.reshape(c["nrow"], c["ncol"])
        # take the two values from the fixture's meta
        conv = {"INF": float("inf"), "NINF": float("-inf")}

        def val(s):
            if s in conv:
                return conv[s]
            if s.startswith("("):
                a, b = s.strip("()").split(",")
                return complex(float(a), float(b))
            return float(s)
        l = np.array([val(c["lower"])], dtype=want.dtype)
        u = np.array([val(c["upper"])], dtype=want.dtype)
        lib.oracle_fill_lowertri(eb, p(l), p(u), ctypes.c_int64(c["nrow"]), ctypes.c_int64(c["ncol"]),
                                 ctypes.c_int64(c["start"]), p(out))
        assert out.tobytes() == want.tobytes()
