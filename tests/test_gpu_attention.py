"""The fused attention kernel (es_b200_launch_attention) through the C ABI against a plain PyTorch
fp32 restatement of the chain with the reference's roundings (scores and probabilities are f16
tensors in the reference's graph), and, at small sizes, against the oracle, which computes the node as
the reference's five einsummables.

Tolerance: 1e-2 of the largest output value -- the f16 tolerance of the contraction tests; the
kernel normalises after the second contraction instead of before it, so its probabilities are
rounded to f16 at a different scale than the reference's."""
import os
import sys

import numpy as np
import pytest
import torch

import einsummable_b200 as es
from einsummable_b200 import _lib
from einsummable_b200.attention import attention_t

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle"))
import es_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
NEG_INF = float("-inf")


def torch_reference(q, k, v, mask):
    """q [b,h,rows,d], k / v [b,h,keys,d], mask [rows,keys] or None: CPU tensors, f16."""
    s = torch.einsum("bhid,bhjd->bhij", q.float(), k.float()).half()
    x = (s + mask).float() if mask is not None else s.float()
    p = torch.softmax(x, dim=-1).half()
    return torch.einsum("bhij,bhjd->bhid", p.float(), v.float()).half()


def causal_mask(rows, keys, start=0):
    i = torch.arange(rows).unsqueeze(1)
    j = torch.arange(keys).unsqueeze(0)
    return torch.where(i - start >= j, torch.tensor(0.0), torch.tensor(NEG_INF)).half()


def make(b, h, rows, keys, d, layout, seed):
    """Random operands; layout "bshd": [batch, row, head, dim] as the llama graphs hold Q, K, V;
    "bhsd": heads outside the rows.  Returns the storage tensors and [b,h,n,d] views of them."""
    g = torch.Generator().manual_seed(seed)

    def one(n):
        shape = (b, n, h, d) if layout == "bshd" else (b, h, n, d)
        t = (torch.randn(shape, generator=g) * 0.5).half()
        return t, (t.permute(0, 2, 1, 3) if layout == "bshd" else t)

    return one(rows), one(keys), one(keys)


def strides_of(view):
    st = view.stride()
    assert st[3] == 1
    return [st[0], st[1], st[2]]


def run(km, qv, kv, vv, mask, skip=None, stream=None):
    b, h, rows, d = qv.shape
    keys = kv.shape[2]
    dev = "cuda:0"
    # the views share storage with contiguous tensors: move the storage, rebuild the views
    def to_dev(view):
        base = view._base if view._base is not None else view
        dbase = base.to(dev)
        return dbase, dbase.as_strided(view.shape, view.stride(), view.storage_offset())
    qb, qd = to_dev(qv)
    kb, kd = to_dev(kv)
    vb, vd = to_dev(vv)
    out = torch.full((b, h, rows, d), float("nan"), dtype=torch.float16, device=dev)
    md = mask.to(dev).contiguous() if mask is not None else None
    a = attention_t(b, h, rows, keys, d, strides_of(qd), strides_of(kd), strides_of(vd), strides_of(out),
                    keys, 0 if skip is None else 1, skip or 0)
    km.attention(a, stream, out, qd, kd, vd, md)
    torch.cuda.synchronize()
    assert km.device_status() == 0
    return out.cpu()


def check(got, want, what):
    scale = want.float().abs().max().item()
    err = (got.float() - want.float()).abs().max().item()
    assert np.isfinite(got.float().numpy()).all(), what
    assert err <= 1e-2 * scale, (what, err, scale)


CASES = [
    # b, h, rows, keys, d, layout, mask
    (1, 1, 128, 64, 128, "bhsd", "zero"),        # one key block: no rescaling
    (1, 2, 128, 128, 128, "bshd", "random"),     # two blocks
    (1, 2, 128, 320, 128, "bshd", "random"),     # five blocks
    (2, 3, 200, 150, 64, "bshd", "random"),      # ragged rows and keys, one 64-wide block of the head dim
    (2, 2, 16, 16, 32, "bshd", "causal"),        # the tiny llama fixture's shape: head dim 32 of a 64-wide tile
    (2, 1, 16, 16, 16, "bshd", "causal"),        # one of four heads of the tiny tensor-parallel fixture: head dim 16
    (1, 2, 130, 70, 96, "bhsd", "causal"),       # head dim 96 of a 128-wide tile
    (2, 4, 256, 512, 128, "bshd", "causal"),
    (1, 3, 64, 64, 128, "bhsd", None),           # no mask
]


@pytest.mark.parametrize("b,h,rows,keys,d,layout,mask_kind", CASES)
def test_attention_matches_fp32_reference_and_oracle(b, h, rows, keys, d, layout, mask_kind):
    km = es.kernel_manager_t(0)
    (_, qv), (_, kv), (_, vv) = make(b, h, rows, keys, d, layout, seed=rows * 7 + keys)
    if mask_kind == "zero":
        mask = torch.zeros(rows, keys).half()
    elif mask_kind == "random":
        g = torch.Generator().manual_seed(5)
        mask = torch.randn(rows, keys, generator=g).half()
        mask[torch.rand(rows, keys, generator=g) < 0.2] = NEG_INF
        mask[:, 0] = 0.0                         # no row without a finite entry
    elif mask_kind == "causal":
        mask = causal_mask(rows, keys)
    else:
        mask = None
    got = run(km, qv, kv, vv, mask)
    check(got, torch_reference(qv, kv, vv, mask), "fp32 reference")
    if mask is not None and b * h * rows * keys * d <= (1 << 22):
        a = {"batch": b, "heads": h, "rows": rows, "keys": keys, "head_dim": d,
             "q_stride": strides_of(qv), "k_stride": strides_of(kv), "v_stride": strides_of(vv)}
        base = lambda v: (v._base if v._base is not None else v).numpy().reshape(-1)  # noqa: E731
        want = O.reference_attention(a, base(qv), base(kv), base(vv), mask.numpy())
        check(got, torch.from_numpy(want.reshape(b, h, rows, d)), "oracle")
    km.close()


@pytest.mark.parametrize("start", [0, -256, 100])
def test_skipping_masked_key_blocks_changes_nothing(start):
    """With a lower-triangular mask the kernel may be told which keys are -inf; the blocks it then
    leaves out contribute exact zeros, so the result is bit for bit the one without the hint."""
    km = es.kernel_manager_t(0)
    b, h, rows, keys, d = 2, 4, 256, 512, 128
    (_, qv), (_, kv), (_, vv) = make(b, h, rows, keys, d, "bshd", seed=3)
    mask = causal_mask(rows, keys, start)
    if start > 0:
        mask[:start, 0] = 0.0                    # rows above the diagonal's start would be all -inf
    plain = run(km, qv, kv, vv, mask)
    hinted = run(km, qv, kv, vv, mask, skip=start) if start <= 0 else plain
    assert torch.equal(plain.view(torch.int16), hinted.view(torch.int16))
    check(plain, torch_reference(qv, kv, vv, mask), "fp32 reference")
    km.close()


def test_llama7b_attention_block_full_size():
    """The block of the LLaMA-7B layer: 4 x 32 heads, 512 x 512, head dim 128, Q / K / V as
    [batch, row, head, dim], the lower-triangular mask with the skip hint -- on a side stream."""
    km = es.kernel_manager_t(0)
    b, h, rows, keys, d = 4, 32, 512, 512, 128
    (_, qv), (_, kv), (_, vv) = make(b, h, rows, keys, d, "bshd", seed=11)
    mask = causal_mask(rows, keys)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        got = run(km, qv, kv, vv, mask, skip=0, stream=side)
    check(got, torch_reference(qv, kv, vv, mask), "fp32 reference")
    km.close()


def test_attention_as_an_op_of_a_program_and_replayed():
    from einsummable_b200.program import program_t
    km = es.kernel_manager_t(0)
    b, h, rows, keys, d = 1, 4, 256, 256, 128
    (_, qv), (_, kv), (_, vv) = make(b, h, rows, keys, d, "bhsd", seed=2)
    mask = causal_mask(rows, keys)
    dev = "cuda:0"
    qd, kd, vd, md = qv.to(dev), kv.to(dev), vv.to(dev), mask.to(dev)
    out = torch.zeros(b, h, rows, d, dtype=torch.float16, device=dev)
    a = attention_t(b, h, rows, keys, d, strides_of(qd), strides_of(kd), strides_of(vd), strides_of(out), keys, 1, 0)
    p = program_t(km)
    fill = p.add_copy(md, md, 16)                 # any earlier op: the attention op waits for it
    p.add_attention(a, out, qd, kd, vd, md, deps=[fill])
    ws = p.finalize(2)
    p.set_workspace(torch.empty(max(ws, 256), dtype=torch.uint8, device=dev), max(ws, 256))
    want = torch_reference(qv, kv, vv, mask)
    stream = torch.cuda.current_stream()
    p.launch(stream)
    torch.cuda.synchronize()
    check(out.cpu(), want, "eager")
    out.zero_()
    p.instantiate()
    p.replay(stream)
    torch.cuda.synchronize()
    check(out.cpu(), want, "replay")
    assert km.device_status() == 0
    p.close()
    km.close()


def test_attention_rejects_what_the_kernel_cannot_serve():
    km = es.kernel_manager_t(0)
    x = torch.zeros(1 << 16, dtype=torch.float16, device="cuda:0")
    ok = dict(batch=1, heads=1, rows=16, keys=16, head_dim=64, q_stride=[1024, 1024, 64], k_stride=[1024, 1024, 64],
              v_stride=[1024, 1024, 64], out_stride=[1024, 1024, 64], mask_stride=16)
    for change, status in ((dict(head_dim=136), _lib.ES_NOT_SUPPORTED), (dict(head_dim=60), _lib.ES_NOT_SUPPORTED),
                           (dict(q_stride=[1024, 1024, 60]), _lib.ES_NOT_SUPPORTED),
                           (dict(mask_stride=8), _lib.ES_BAD_DESCRIPTOR), (dict(rows=0), _lib.ES_BAD_DESCRIPTOR)):
        a = attention_t(**{**ok, **change})
        with pytest.raises(es.es_error) as ei:
            km.attention(a, None, x, x, x, x, x)
        assert ei.value.status == status, change
    with pytest.raises(es.es_error):
        km.attention(attention_t(**ok), None, x, x[1:], x, x, x)    # 2-byte aligned operand
    km.close()
