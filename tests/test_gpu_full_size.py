"""The configurations at their full sizes, checked through properties that need no CPU pass over
the whole tensor: planted extrema, constant rows, selection by exact comparison on the device,
block-wise round trips.  (The oracle checks the same kernels element by element at reduced sizes
in test_gpu_kernels.py.)"""
import numpy as np
import pytest
import torch

import einsummable_b200 as es
from einsummable_b200 import einsummable_t, scalarop_t, touch_t

pytestmark = pytest.mark.gpu
S = scalarop_t
ROWS, COLS = 8192, 11008


@pytest.fixture(scope="module")
def km():
    k = es.kernel_manager_t(0)
    yield k
    assert k.device_status() == 0
    k.close()


def run(km, e, ins, out):
    ws = km.build(e)
    w = torch.empty(max(ws or 0, 16), dtype=torch.uint8, device="cuda:0")
    km(e, None, out, ins, (w, ws) if ws else None)
    torch.cuda.synchronize()


def test_c2_row_max_full_size_is_a_selection(km):
    """max is a selection: bit-exact against the device's own amax, and a planted value wins."""
    g = torch.Generator(device="cuda:0").manual_seed(11)
    x = torch.randn(ROWS, COLS, dtype=torch.float16, device="cuda:0", generator=g)
    cols = torch.randint(0, COLS, (ROWS,), device="cuda:0", generator=g)
    x[torch.arange(ROWS, device="cuda:0"), cols] = 9.5   # above any N(0,1) draw of this size
    out = torch.empty(ROWS, dtype=torch.float16, device="cuda:0")
    run(km, einsummable_t([ROWS, COLS], [[0, 1]], 1, S.make_identity("f16"), "max"), [x.reshape(-1)], out)
    assert torch.equal(out, torch.full_like(out, 9.5))
    x[:, 0] = -1.0
    x[5, :] = -3.0
    run(km, einsummable_t([ROWS, COLS], [[0, 1]], 1, S.make_identity("f16"), "min"), [x.reshape(-1)], out)
    assert torch.equal(out, x.amin(dim=1))


def test_c2_row_sum_full_size_linearity(km):
    """sum is linear: constant rows give cols * c exactly (in f16: 11008 * 2^-6 = 172),
    and sum(x) + sum(-x) cancels to zero within the rounding of the two results."""
    out = torch.empty(ROWS, dtype=torch.float16, device="cuda:0")
    e = einsummable_t([ROWS, COLS], [[0, 1]], 1, S.make_identity("f16"), "add")
    c = torch.full((ROWS * COLS,), 2.0 ** -6, dtype=torch.float16, device="cuda:0")
    run(km, e, [c], out)
    assert torch.equal(out, torch.full_like(out, COLS * 2.0 ** -6))
    g = torch.Generator(device="cuda:0").manual_seed(12)
    x = torch.randn(ROWS * COLS, dtype=torch.float16, device="cuda:0", generator=g)
    neg = torch.empty_like(out)
    run(km, e, [x], out)
    run(km, e, [-x], neg)
    assert torch.equal(out, -neg)                      # same order of additions, opposite signs
    want = x.reshape(ROWS, COLS).double().sum(dim=1)
    # tolerance 1e-2 relative to the scale of the partial sums (sqrt(cols) for N(0,1) terms)
    assert (out.double() - want).abs().max().item() <= 1e-2 * np.sqrt(COLS)


def test_c2_elementwise_full_size_against_f32_math(km):
    """silu(x)*y and exp(x - m) on the whole tensor against the same expressions in f32 on the
    device, rounded once: at most 1 ulp of f16 apart (fast exp / reciprocal inside the kernel)."""
    g = torch.Generator(device="cuda:0").manual_seed(13)
    x = torch.randn(ROWS * COLS, dtype=torch.float16, device="cuda:0", generator=g)
    y = torch.randn(ROWS * COLS, dtype=torch.float16, device="cuda:0", generator=g)
    out = torch.empty_like(x)
    e = einsummable_t([ROWS * COLS], [[0], [0]], 1, S.combine(S.make_mul("f16"), [S.make_silu("f16"), S.make_identity("f16")]))
    run(km, e, [x, y], out)
    xf, yf = x.float(), y.float()
    want = (xf / (1.0 + torch.exp(-xf)) * yf)
    err = (out.float() - want).abs()
    ulp = torch.maximum(want.abs(), torch.tensor(2.0 ** -14, device="cuda:0")) * 2.0 ** -10
    assert (err <= 1.01 * ulp).all()
    del want, err, ulp, xf, yf
    m = x.reshape(ROWS, COLS).amax(dim=1)
    e2 = einsummable_t([ROWS, COLS], [[0, 1], [0]], 2, S.combine(S.make_exp("f16"), [S.make_sub("f16")]))
    run(km, e2, [x, m], out)
    want = torch.exp(x.reshape(ROWS, COLS).float() - m.float()[:, None]).reshape(-1)
    err = (out.float() - want).abs()
    ulp = torch.maximum(want.abs(), torch.tensor(2.0 ** -14, device="cuda:0")) * 2.0 ** -10
    assert (err <= 1.01 * ulp).all()
    assert out.reshape(ROWS, COLS).amax(dim=1).eq(1.0).all()    # exp(0) at every row's maximum


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("pdim", [2, 4, 8])
def test_c3_full_sweep_round_trip(km, dtype, pdim):
    """[32,512,32,128] cut into pdim blocks per dim: every block copied out of the tensor into a
    packed buffer and copied back into an empty tensor reproduces it bit for bit; accumulating the
    blocks a second time doubles it exactly (x + x is exact)."""
    full = (32, 512, 32, 128)
    tdt = torch.float16 if dtype == "f16" else torch.float32
    g = torch.Generator(device="cuda:0").manual_seed(14)
    src = (torch.rand(int(np.prod(full)), dtype=torch.float32, device="cuda:0", generator=g) * 2 - 1).to(tdt)
    bs = [f // pdim for f in full]
    blk = int(np.prod(bs))
    nblk = pdim ** 4
    packed = torch.zeros(nblk * blk, dtype=tdt, device="cuda:0")
    back = torch.zeros_like(src)
    gather, scatter, accumulate, outs_g, inns_g, outs_s, inns_s = [], [], [], [], [], [], []
    for b in range(nblk):
        idx = np.unravel_index(b, (pdim,) * 4)
        # block (idx) of the full tensor -> packed block b, and back
        gather.append(touch_t([(full[d], bs[d], int(idx[d]) * bs[d], 0, bs[d]) for d in range(4)], None, dtype))
        scatter.append(touch_t([(bs[d], full[d], 0, int(idx[d]) * bs[d], bs[d]) for d in range(4)], None, dtype))
        accumulate.append(touch_t([(bs[d], full[d], 0, int(idx[d]) * bs[d], bs[d]) for d in range(4)], "add", dtype))
        outs_g.append(packed[b * blk:(b + 1) * blk])
        inns_g.append(src)
        outs_s.append(back)
        inns_s.append(packed[b * blk:(b + 1) * blk])
    items = torch.empty(nblk * 256, dtype=torch.uint8, device="cuda:0")
    for touches, outs, inns in ((gather, outs_g, inns_g), (scatter, outs_s, inns_s)):
        km.touch_batch(touches, None, outs, inns, items)
        torch.cuda.synchronize()
    assert torch.equal(back, src)
    km.touch_batch(accumulate, None, outs_s, inns_s, items)
    torch.cuda.synchronize()
    assert torch.equal(back, src + src)
