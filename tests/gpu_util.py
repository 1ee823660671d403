"""Helpers for the GPU parity tests: numpy <-> device buffers through torch
(torch is plumbing here: device memory and streams only)."""
import numpy as np
import torch

import einsummable_b200 as es

NP = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "c64": np.complex64}
TORCH = {"f16": torch.float16, "f32": torch.float32, "f64": torch.float64, "c64": torch.complex64}


def to_dev(x, device="cuda:0"):
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def to_host(t):
    return t.cpu().numpy()


def run_einsummable(km, e, inputs, device="cuda:0", misalign=0):
    """build + launch through the C ABI; returns the flat output as numpy.
    misalign: byte offset added to every tensor's address (to force the scalar twin)."""
    ws_size = km.build(e)
    assert ws_size is not None, "build returned nullopt for " + repr(e)
    out_dt = e.out_dtype()

    def alloc(n, dt):
        if not misalign:
            return torch.empty(n, dtype=TORCH[dt], device=device), None
        item = np.dtype(NP[dt]).itemsize
        assert misalign % item == 0
        raw = torch.empty(n + misalign // item, dtype=TORCH[dt], device=device)
        return raw[misalign // item:], raw
    d_ins, keep = [], []
    for x in inputs:
        dt = {np.dtype(v): k for k, v in NP.items()}[x.dtype]
        t, raw = alloc(x.size, dt)
        t.copy_(torch.from_numpy(np.ascontiguousarray(x).reshape(-1)))
        d_ins.append(t)
        keep.append(raw)
    d_out, raw_out = alloc(e.out_nelem(), out_dt)
    d_out.zero_()
    ws = torch.empty(max(ws_size, 16), dtype=torch.uint8, device=device) if ws_size else None
    km(e, None, d_out, d_ins, None if ws is None else (ws, ws_size))
    torch.cuda.synchronize()
    return to_host(d_out)


def tolerance(dtype):
    """Relative tolerances stated for the path: f16 1e-2, f32 1e-5 (f32-accumulated
    sums), f64 1e-12."""
    return {"f16": 1e-2, "f32": 1e-5, "f64": 1e-12, "c64": 1e-5}[dtype]


def assert_close(got, want, dtype, what="", normwise=False):
    """Elementwise: |got-want| <= rtol*|want| (with a floor of 1% of the largest
    value).  normwise=True, for aggregated results, bounds the error by rtol times
    the largest value instead: a sum with cancellation has no meaningful
    per-element relative error, and the interpreter fixtures themselves
    accumulate f16 sums in f16 (src/einsummable/dbuffer.cc:346-350)."""
    wide = np.complex128 if dtype == "c64" else np.float64
    g, w = got.astype(wide), want.astype(wide)
    fin = np.isfinite(w)
    assert np.array_equal(np.isfinite(g), fin), what + ": non-finite mismatch"
    assert np.array_equal(g[~fin], w[~fin], equal_nan=True), what + ": inf/nan mismatch"
    rtol = tolerance(dtype)
    scale = float(np.abs(w[fin]).max()) if fin.any() else 1.0
    err = np.abs(g[fin] - w[fin])
    if normwise:
        bound = np.full(err.shape, rtol * max(scale, 1e-30))
    else:
        bound = rtol * np.maximum(np.abs(w[fin]), 1e-2 * max(scale, 1e-30))
    bad = err > bound
    assert not bad.any(), "%s: %d of %d beyond rtol %g (max err %g at scale %g)" % (
        what, int(bad.sum()), err.size, rtol, float(err.max()), scale)
