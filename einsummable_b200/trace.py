"""Clock trace of the tensor-core contraction kernel.

    python -m einsummable_b200.build --trace
    python -m einsummable_b200.trace gemm 2048 4096 4096 [f16|f32]      # ij,kj->ik, M N K
    python -m einsummable_b200.trace scores | pv | nn | tn
    python -m einsummable_b200.trace attention [noskip]                 # the fused attention chain, layer size

Loads lib/libes_b200_trace.so (the library compiled with -DES_B200_TRACE: CTA 0 records
clock64() at the role boundaries, see csrc/contraction.cu), launches one contraction a few
times and prints, in SM cycles of CTA 0: the producer's time per k-iteration and how much of
it was spent waiting for a free stage, the MMA issuer's time per k-iteration and its wait for a
full stage, and the epilogue's waits and durations.  This is how the bound of each kernel
variant was found (producer lane, tensor pipe or epilogue); ncu's counters do not show it.
"""
import os
import sys

import numpy as np


def attention_trace(torch, kernel_manager_t, skip):
    """Cycles per key block of the traced CTA (last query tile of head 0, batch 0): where the
    softmax warp and the issuing lane spend them."""
    from .attention import attention_t
    b, h, s, d = 4, 32, 512, 128
    q, k, v = [(torch.randn(b, s, h, d, device="cuda") * 0.5).half() for _ in range(3)]
    i, j = torch.arange(s, device="cuda").unsqueeze(1), torch.arange(s, device="cuda").unsqueeze(0)
    mask = torch.where(i >= j, 0.0, float("-inf")).half().contiguous()
    out = torch.empty(b, h, s, d, dtype=torch.float16, device="cuda")
    st = [s * h * d, d, h * d]
    a = attention_t(b, h, s, s, d, st, st, st, [h * s * d, s * d, d], s, 1 if skip else 0, 0)
    km = kernel_manager_t(0)
    for _ in range(5):
        km.attention(a, None, out, q, k, v, mask)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        km.attention(a, None, out, q, k, v, mask)
    e1.record()
    torch.cuda.synchronize()
    print("%.1f us per launch (with the trace compiled in), device status %d" % (e0.elapsed_time(e1) / 20 * 1e3, km.device_status()))
    raw = np.array(km.debug_trace(8512 + 4096)[8000:], dtype=np.int64)
    cta = raw[512:].reshape(1024, 4)[:b * h * ((s + 127) // 128)]
    t0 = cta[:, 1].min()
    print("CTAs: %d, first start to last end %.1f us; duration by key blocks:" % (len(cta), (cta[:, 2].max() - t0) / 1e3),
          {int(nb): "%.1f us (n=%d)" % ((cta[cta[:, 3] == nb, 2] - cta[cta[:, 3] == nb, 1]).mean() / 1e3, (cta[:, 3] == nb).sum())
           for nb in sorted(set(cta[:, 3]))})
    starts = np.sort(cta[:, 1] - t0) / 1e3
    print("start times (us), every 32nd CTA in start order:", np.round(starts[::32], 1))
    for sm in (0, 1, 73, 147):
        mine = cta[cta[:, 0] == sm]
        order = np.argsort(mine[:, 1])
        print("  SM %3d:" % sm, ["%.1f-%.1f (%d blocks)" % ((r[1] - t0) / 1e3, (r[2] - t0) / 1e3, r[3]) for r in mine[order]])
    tr = raw[:512].reshape(16, 32)
    n = 0
    while n < 32 and tr[6, n] != 0:
        n += 1
    np.set_printoptions(linewidth=220)
    print("key blocks of the traced CTA:", n)
    names = ["wait for the scores", "read + pack the scores", "mask + maximum", "wait for P V of the block before (+ rescale)",
             "exponentials + store P", "fence + arrive"]
    print("softmax warp 0, cycles per block:", np.diff(tr[0, :n]))
    for x, name in enumerate(names):
        print("  %-46s" % name, tr[x + 1, :n] - tr[x, :n])
    names = ["wait for K, issue the next block's scores", "wait for this block's scores, copy K", "wait for P",
             "wait for V, issue P V", "wait for P V", "copy V"]
    print("issuing lane, cycles per block  :", np.diff(tr[8, :n]))
    for x, name in enumerate(names):
        print("  %-46s" % name, tr[9 + x, :n] - tr[8 + x, :n])
    print("softmax start - issuer start      :", tr[0, :n] - tr[8, :n])
    print("setup: entry -> TMEM allocated %d -> after the CTA barrier %d -> first block starts %d" % (
        tr[7, 1] - tr[7, 0], tr[7, 2] - tr[7, 0], tr[0, 0] - tr[7, 0]))
    print("end: last arrive -> last P V seen %d -> result stored %d -> after the CTA barrier %d -> TMEM freed %d" % (
        tr[15, 0] - tr[6, n - 1], tr[15, 1] - tr[6, n - 1], tr[15, 2] - tr[6, n - 1], tr[15, 3] - tr[6, n - 1]))
    km.close()


def main(argv):
    import torch
    from . import _lib
    from .build import TRACE_LIB
    if not os.path.exists(TRACE_LIB):
        raise SystemExit("build the trace library first: python -m einsummable_b200.build --trace")
    _lib.LIB_PATH = TRACE_LIB
    from . import einsummable_t, kernel_manager_t, scalarop_t as S
    which = argv[0] if argv else "gemm"
    if which == "attention":
        return attention_trace(torch, kernel_manager_t, "noskip" not in argv)
    dt = "f16"
    if which == "gemm":
        m, n, k = [int(v) for v in argv[1:4]] if len(argv) >= 4 else (2048, 4096, 4096)
        dt = argv[4] if len(argv) > 4 else "f16"
        e = einsummable_t.from_matmul_st(m, k, n, dt)          # (i, j, k) of ij,kj->ik: j is contracted
    elif which == "scores":
        e = einsummable_t.from_str("acbe,adbe->abcd", dict(a=4, b=32, c=512, d=512, e=128), S.make_mul(dt), "add")
    elif which == "pv":
        e = einsummable_t.from_str("abce,aebd->abcd", dict(a=4, b=32, c=512, d=128, e=512), S.make_mul(dt), "add")
    elif which == "nn":
        e = einsummable_t.from_str("ij,jk->ik", dict(i=2048, j=4096, k=4096), S.make_mul(dt), "add")
    elif which == "tn":
        e = einsummable_t.from_str("ji,jk->ik", dict(i=4096, j=2048, k=4096), S.make_mul(dt), "add")
    else:
        raise SystemExit(__doc__)
    km = kernel_manager_t(0)
    ws = km.build(e)
    tdt = torch.float16 if dt == "f16" else torch.float32
    ins = [torch.randn(int(np.prod(e.inn_shape(i))), dtype=tdt, device="cuda") for i in range(2)]
    out = torch.empty(e.out_nelem(), dtype=tdt, device="cuda")
    work = torch.empty(max(ws or 0, 16), dtype=torch.uint8, device="cuda")
    wsarg = (work, ws) if ws else None
    for _ in range(5):
        km(e, None, out, ins, wsarg)
    torch.cuda.synchronize()
    s, t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(20):
        km(e, None, out, ins, wsarg)
    t.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(t) / 20
    print("%s\n%.1f us per launch, %.0f TFLOP/s (with the trace compiled in)" % (
        km.kernel_info(e), ms * 1e3, 2.0 * float(np.prod(e.join_shape)) / ms / 1e9))
    tr = np.array(km.debug_trace(), dtype=np.int64).reshape(8, 1000)
    t0 = tr[0, 0]
    np.set_printoptions(linewidth=200)

    def recorded(row, lo, hi):      # entries CTA 0 reached (zero = never written)
        m = 0
        while lo + m < hi and tr[row, lo + m] != 0:
            m += 1
        return m

    n = min(24, recorded(0, 0, 1000), recorded(4, 0, 1000))
    nt = min(8, recorded(0, 500, 1000), recorded(1, 500, 1000))
    ne = min(8, recorded(5, 0, 1000), recorded(7, 0, 1000))
    print("producer, cycles per k-iteration :", np.diff(tr[0, :n]))
    print("  of which waiting for a stage   :", tr[1, :n] - tr[0, :n])
    print("MMA issuer, cycles per k-iteration:", np.diff(tr[4, :n]))
    print("  of which waiting for operands  :", tr[3, :n] - tr[2, :n])
    print("  issue + commit                 :", tr[4, :n] - tr[3, :n])
    print("tile tops (producer)             :", tr[0, 500:500 + nt] - t0)
    print("  coordinates ready after        :", tr[1, 500:500 + nt] - tr[0, 500:500 + nt])
    print("epilogue: wait begins            :", tr[5, :ne] - t0)
    print("  accumulator ready              :", tr[6, :ne] - t0)
    print("  released                       :", tr[7, :ne] - t0)
    print("  drain cycles                   :", tr[7, :ne] - tr[6, :ne])
    km.close()


if __name__ == "__main__":
    main(sys.argv[1:])
