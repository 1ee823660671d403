"""Tensor-core contractions (tcgen05 / TMEM / TMA) against the executor-convention
oracle (f64 accumulation from the input values, rounded once), through the C ABI.
Tolerances: f16 1e-2, f32 (3xTF32) 1e-5, both relative to the largest output
value (sums with cancellation have no per-element relative error); the opt-in
single-TF32 policy is checked at 2e-3."""
import numpy as np
import pytest
import torch

import einsummable_b200 as es
import es_oracle as O
from einsummable_b200 import einsummable_t, scalarop_t
from gpu_util import NP, assert_close, run_einsummable

pytestmark = pytest.mark.gpu
S = scalarop_t


@pytest.fixture(scope="module")
def km():
    k = es.kernel_manager_t(0)
    yield k
    assert k.device_status() == 0, "a bounded wait inside a tensor-core kernel expired"
    k.close()


def contraction(spec, extents, dtype):
    return einsummable_t.from_str(spec, extents, S.make_mul(dtype), "add")


def check(km, spec, extents, dtype, expect_tc=True, rtol=None, misalign=0, seed=0):
    e = contraction(spec, extents, dtype)
    rng = np.random.default_rng(seed)
    ins = [rng.uniform(-1, 1, int(np.prod(e.inn_shape(k)))).astype(NP[dtype]) for k in range(2)]
    got = run_einsummable(km, e, ins, misalign=misalign)
    info = km.kernel_info(e)
    if expect_tc:
        assert info.startswith("contraction_tc"), info
    want = O.reference_einsummable(e.join_shape, e.inns, e.out_rank, e.join.text, "add", ins, "executor")
    assert km.device_status() == 0
    if rtol is None:
        assert_close(got, want, dtype, spec + " " + info, normwise=True)
    else:
        scale = np.abs(want.astype(np.float64)).max()
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
        assert err <= rtol * scale, (spec, err, scale)
    return info


@pytest.mark.parametrize("spec,extents", [
    ("ij,kj->ik", dict(i=256, j=128, k=128)),           # both K-major, one tile
    ("ij,kj->ik", dict(i=128, j=64, k=64)),             # smallest: one k-block, bn=64
    ("ij,kj->ik", dict(i=512, j=1024, k=768)),          # many k-blocks, bn=256, ring wraps
    ("ij,kj->ik", dict(i=200, j=200, k=136)),           # ragged M, N and K (zero-filled tails)
    ("ij,jk->ik", dict(i=256, j=192, k=384)),           # B MN-major
    ("ji,kj->ik", dict(i=256, j=192, k=128)),           # A MN-major
    ("ji,jk->ik", dict(i=384, j=320, k=256)),           # both MN-major
    ("ij,jk->ik", dict(i=136, j=72, k=200)),            # ragged, MN-major B
    ("bij,bkj->bik", dict(b=3, i=256, j=128, k=128)),   # batched
    ("acbe,adbe->abcd", dict(a=2, b=4, c=256, d=256, e=128)),   # attention scores
    ("abce,aebd->abcd", dict(a=2, b=4, c=256, d=128, e=256)),   # attention P.V
    ("aebf,cdef->abcd", dict(a=2, b=256, c=4, d=128, e=4, f=128)),  # WO (merges to adbe,cde->abc)
    ("ij,kj->ik", dict(i=4, j=512, k=1024)),            # few rows: operands swapped
])
def test_f16_contractions(km, spec, extents):
    check(km, spec, extents, "f16")


@pytest.mark.parametrize("spec,extents,big,small", [
    ("ij,kj->ik", dict(i=2048, j=1024, k=4096), 128, 0),     # every row pair is one 256-row item
    ("ij,kj->ik", dict(i=2176, j=1024, k=2816), 88, 11),     # odd number of 128-row tiles: last row alone
    ("ij,kj->ik", dict(i=2048, j=1024, k=5632), 148, 56),    # one wave of 256-row items, 128-row tail
    ("ij,kj->ik", dict(i=2000, j=1032, k=4100), 136, 0),     # ragged M, N and K
    ("ji,kj->ik", dict(i=2048, j=1024, k=4096), 128, 0),     # A MN-major: two copies per half
    ("ij,jk->ik", dict(i=2048, j=1024, k=4096), 128, 0),     # B MN-major
    ("bij,bkj->bik", dict(b=2, i=1024, j=1024, k=2560), 80, 0),   # batched
])
def test_f16_contractions_256_row_items(km, spec, extents, big, small):
    """Large f16 contractions schedule 256-row items (two 128-row halves sharing one B tile in
    shared memory) first and 128-row items for the tail; both kinds in one launch."""
    info = check(km, spec, extents, "f16")
    assert "items256=%d,items128=%d" % (big, small) in info, info


@pytest.mark.parametrize("spec,extents", [
    ("ij,jk->ik", dict(i=256, j=256, k=256)),
    ("ij,kj->ik", dict(i=128, j=512, k=256)),
    ("ji,jk->ik", dict(i=256, j=160, k=128)),
    ("ij,jk->ik", dict(i=200, j=100, k=72)),
    ("acbe,adbe->abcd", dict(a=1, b=2, c=128, d=128, e=64)),
])
def test_f32_contractions_3xtf32(km, spec, extents):
    info = check(km, spec, extents, "f32")
    assert "3xtf32" in info


def test_f32_single_tf32_policy():
    km = es.kernel_manager_t(0)
    km.set_f32_policy("tf32")
    info = check(km, "ij,jk->ik", dict(i=256, j=256, k=256), "f32", rtol=2e-3)
    assert info.startswith("contraction_tc_tf32")
    km.close()


def test_c1_block_2048_f32(km):
    """One block product of config 1 (ij,jk->ik f32, 2048^3), full size."""
    check(km, "ij,jk->ik", dict(i=2048, j=2048, k=2048), "f32")


def test_llama_ffn_shape_f16(km):
    check(km, "ij,kj->ik", dict(i=2048, j=4096, k=1376), "f16")


def test_unaligned_operands_fall_back_to_simt(km):
    # pointers offset by 2 bytes cannot be addressed by TMA: the generated kernel runs instead
    check(km, "ij,kj->ik", dict(i=64, j=64, k=64), "f16", expect_tc=False, misalign=2)


def test_shapes_tma_cannot_describe_fall_back(km):
    info = check(km, "ij,kj->ik", dict(i=33, j=30, k=17), "f16", expect_tc=False)
    assert not info.startswith("contraction_tc")
    info = check(km, "ij,jk->ik", dict(i=16, j=24, k=20), "f64", expect_tc=False)
    assert not info.startswith("contraction_tc")


def test_linearity_at_full_llama_size(km):
    """Size-independent property at a full LLaMA shape (2048 x 4096 x 4096):
    with B = identity-like selector the product reproduces A's columns exactly."""
    i, j, k = 2048, 4096, 4096
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, i * j).astype(np.float16)
    perm = rng.permutation(j)[:k]
    b = np.zeros((k, j), dtype=np.float16)
    b[np.arange(k), perm] = 1.0
    e = einsummable_t.from_matmul_st(i, j, k, "f16")
    got = run_einsummable(km, e, [a, b.reshape(-1)])
    assert km.kernel_info(e).startswith("contraction_tc")
    want = a.reshape(i, j)[:, perm].reshape(-1)
    assert got.tobytes() == want.tobytes()


def test_clock_trace_is_absent_from_the_product_library(km):
    """The kernel's clock trace only exists in the library built with -DES_B200_TRACE
    (python -m einsummable_b200.build --trace); the product library says so."""
    from einsummable_b200 import _lib
    with pytest.raises(_lib.es_error) as exc:
        km.debug_trace(16)
    assert "ES_B200_TRACE" in str(exc.value)
