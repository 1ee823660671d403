"""Clock trace of the tensor-core contraction kernel.

    python -m einsummable_b200.build --trace
    python -m einsummable_b200.trace gemm 2048 4096 4096 [f16|f32]      # ij,kj->ik, M N K
    python -m einsummable_b200.trace scores | pv | nn | tn

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


def main(argv):
    import torch
    from . import _lib
    from .build import TRACE_LIB
    if not os.path.exists(TRACE_LIB):
        raise SystemExit("build the trace library first: python -m einsummable_b200.build --trace")
    _lib.LIB_PATH = TRACE_LIB
    from . import einsummable_t, kernel_manager_t, scalarop_t as S
    which = argv[0] if argv else "gemm"
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
