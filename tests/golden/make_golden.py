#!/usr/bin/env python3
"""Generates tests/golden/golden.json + golden.npz from the reference itself.

Runs in the build container only (needs the reference tree): it loads
oracle/_ref/libes_ref.so -- the reference's own interpreter compiled from its
sources by oracle/Makefile -- and records, for every case of cases.py, the
reference's outputs on seeded inputs.  The tests read only the two generated
files, so they run where the reference does not exist.

usage: python tests/golden/make_golden.py
"""
import ctypes
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
import cases  # noqa: E402

NP = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "c64": np.complex64}
CODE = {"f16": 0, "f32": 1, "f64": 2, "c64": 3}
CAST = {None: -1, "add": 0, "mul": 1, "min": 2, "max": 3}

L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libes_ref.so"))
L.ref_last_error.restype = ctypes.c_char_p


def ok(rc):
    if rc < 0:
        raise RuntimeError(L.ref_last_error().decode())
    return rc


def ref_text(fn, *args):
    buf = ctypes.create_string_buffer(1 << 16)
    ok(fn(*args, buf, 1 << 16))
    return buf.value.decode()


def parse_es(s, extents):
    lhs, out = s.split("->")
    letters = {}
    for ch in out + lhs.replace(",", ""):
        letters.setdefault(ch, len(letters))
    inns = [[letters[c] for c in t] for t in lhs.split(",")]
    shape = [0] * len(letters)
    for ch, m in letters.items():
        shape[m] = extents[ch]
    return shape, inns, len(out)


def rand(rng, n, dtype, rng_spec):
    if rng_spec == "ints":
        return rng.integers(0, 3, n).astype(NP[dtype])
    lo, hi = rng_spec
    if dtype == "c64":
        return (rng.uniform(lo, hi, n) + 1j * rng.uniform(lo, hi, n)).astype(np.complex64)
    return rng.uniform(lo, hi, n).astype(NP[dtype])


def hole_dtypes(text):
    import re
    d = {}
    for dt, k in re.findall(r"hole\|(f16|f32|f64|c64)@(\d+)", text):
        d[int(k)] = dt
    return d


def c_u64(xs):
    return (ctypes.c_uint64 * len(xs))(*xs)


def c_int(xs):
    return (ctypes.c_int * len(xs))(*xs)


def main():
    meta = {"einsummable": [], "merge": [], "touch": [], "fill": [], "scalarops": {}}
    arrays = {}

    # ---- scalarop builder strings (golden strings for the parser) ----
    for name in ["identity", "add", "mul", "div", "neg", "min", "max", "is_equal", "sub", "exp", "sigmoid",
                 "log", "sqrt", "inverse", "inverse_sqrt", "square", "relu", "silu", "silu_mul", "exp_sub",
                 "scale:0.25", "increment:1e-06", "power:3", "softmax_v3_sum:0.0883883",
                 "softmax_v3_norm:0.0883883"]:
        for dt in ["f16", "f32", "f64"]:
            text = ref_text(L.ref_scalarop_make, name.encode(), CODE[dt])
            info = ref_text(L.ref_scalarop_info, text.encode()).split("|")
            # info = text, cppstr, simplified, out dtype, num inputs (text holds '|' itself: rebuild)
            meta["scalarops"]["%s/%s" % (name, dt)] = text
    for name, dt in [("convert:f32", "f16"), ("convert:f16", "f32"), ("convert:f64", "f32"),
                     ("convert:f32", "f64"), ("conjugate", "c64"), ("project_real", "c64"),
                     ("project_imag", "c64"), ("complex", "c64"), ("mul", "c64"), ("add", "c64"),
                     ("identity", "c64")]:
        meta["scalarops"]["%s/%s" % (name, dt)] = ref_text(L.ref_scalarop_make, name.encode(), CODE[dt])

    # ---- einsummable cases through reference_einsummable_inplace ----
    for idx, (name, es, extents, join, castable, rng_spec) in enumerate(cases.EINSUMMABLE_CASES):
        rng = np.random.default_rng(1000 + idx)
        if isinstance(join, tuple):
            join_text = ref_text(L.ref_scalarop_make, join[1].encode(), CODE[join[2]])
        else:
            join_text = join
        shape, inns, out_rank = parse_es(es, extents)
        hd = hole_dtypes(join_text)
        ins = []
        for k, modes in enumerate(inns):
            n = int(np.prod([shape[m] for m in modes]))
            ins.append(rand(rng, n, hd[k], rng_spec))
        if name == "mm_f64_golden_shape":
            # the reference's own known-answer test (tests/reference.h:4-46)
            ins = [np.arange(8, 20, dtype=np.float64), np.arange(100, 120, dtype=np.float64)]
        info = ref_text(L.ref_scalarop_info, join_text.encode())
        out_dt = info.split("|")[-2]
        n_out = int(np.prod(shape[:out_rank]))
        out = np.zeros(n_out, dtype=NP[out_dt])
        flat_modes = [m for t in inns for m in t]
        ptrs = (ctypes.c_void_p * len(ins))(*[x.ctypes.data for x in ins])
        ok(L.ref_einsummable(len(shape), c_u64(shape), len(inns), c_int([len(t) for t in inns]),
                             c_int(flat_modes), out_rank, join_text.encode(), CAST[castable],
                             ctypes.c_void_p(out.ctypes.data), ptrs))
        merged = ref_text(L.ref_merge, len(shape), c_u64(shape), len(inns), c_int([len(t) for t in inns]),
                          c_int(flat_modes), out_rank, join_text.encode(), CAST[castable])
        meta["einsummable"].append(dict(name=name, join_shape=shape, inns=inns, out_rank=out_rank,
                                        join=join_text, castable=castable, out_dtype=out_dt,
                                        merged=merged))
        for k, x in enumerate(ins):
            arrays["es/%s/in%d" % (name, k)] = x
        arrays["es/%s/out" % name] = out

    # ---- merge_adjacent_dims / str / predicates ----
    for shape, inns, out_rank in cases.MERGE_CASES:
        n = len(inns)
        if n == 1:
            join = "hole|f32@0"
        elif n == 2:
            join = "*[hole|f32@0,hole|f32@1]"
        cast = 0 if out_rank < len(shape) else -1
        flat = [m for t in inns for m in t]
        merged = ref_text(L.ref_merge, len(shape), c_u64(shape), n, c_int([len(t) for t in inns]),
                          c_int(flat), out_rank, join.encode(), cast)
        meta["merge"].append(dict(join_shape=shape, inns=inns, out_rank=out_rank, join=join,
                                  castable=None if cast < 0 else "add", merged=merged))

    # ---- touches: random rank 1..4, dims 10..30 as exps/cpuexec_touch.cc:19-139 ----
    rng = np.random.default_rng(7)
    tid = 0
    fixed = [[(4, 3, 1, 0, 2), (6, 5, 2, 1, 3)], [(4, 4, 0, 0, 4), (6, 6, 0, 0, 6)],
             [(10, 10, 3, 3, 2), (20, 20, 0, 0, 20)]]
    for dtype in cases.TOUCH_DTYPES:
        for castable in cases.TOUCH_CASTABLES:
            if dtype == "c64" and castable in ("min", "max"):
                continue
            sels = list(fixed) if (dtype == "f16") else []
            for rank in range(1, 5):
                sel = []
                for _ in range(rank):
                    lo, hi = {1: (10, 31), 2: (10, 31), 3: (5, 11), 4: (3, 8)}[rank]
                    d_inn = int(rng.integers(lo, hi))
                    d_out = int(rng.integers(lo, hi))
                    size = int(rng.integers(1, min(d_inn, d_out) + 1))
                    sel.append((d_inn, d_out, int(rng.integers(0, d_inn - size + 1)),
                                int(rng.integers(0, d_out - size + 1)), size))
                sels.append(sel)
            for sel in sels:
                n_inn = int(np.prod([s[0] for s in sel]))
                n_out = int(np.prod([s[1] for s in sel]))
                if sel == fixed[0]:
                    inn, out0 = np.arange(24).astype(NP[dtype]), np.zeros(15, dtype=NP[dtype])
                else:
                    inn = rand(rng, n_inn, dtype, (0.5, 2.0) if castable == "mul" else (-3, 3))
                    out0 = rand(rng, n_out, dtype, (0.5, 2.0) if castable == "mul" else (-3, 3))
                d5 = c_u64([v for s in sel for v in s])
                o1, o2 = out0.copy(), out0.copy()
                ok(L.ref_touch(len(sel), d5, CAST[castable], CODE[dtype], ctypes.c_void_p(o1.ctypes.data),
                               ctypes.c_void_p(inn.ctypes.data)))
                ok(L.ref_execute_touch(len(sel), d5, CAST[castable], CODE[dtype],
                                       ctypes.c_void_p(o2.ctypes.data), ctypes.c_void_p(inn.ctypes.data)))
                # the interpreter and the CPU engine's executor must agree bit for bit
                assert o1.tobytes() == o2.tobytes(), (sel, castable, dtype)
                simp = (ctypes.c_uint64 * (5 * len(sel)))()
                r = ok(L.ref_touch_simplify(len(sel), d5, simp))
                name = "t%03d" % tid
                tid += 1
                meta["touch"].append(dict(name=name, selection=[list(s) for s in sel], castable=castable,
                                          dtype=dtype,
                                          simplified=[list(simp[5 * i:5 * i + 5]) for i in range(r)]))
                arrays["touch/%s/inn" % name] = inn
                arrays["touch/%s/out0" % name] = out0
                arrays["touch/%s/out" % name] = o1

    # ---- fills ----
    def sval(v):
        if v == float("inf"):
            return "INF"
        if v == float("-inf"):
            return "NINF"
        if isinstance(v, complex):
            return "(%g,%g)" % (v.real, v.imag)
        return "%g" % v
    for i, (dtype, lower, upper, nrow, ncol, start) in enumerate(cases.FILL_CASES):
        out = np.zeros(nrow * ncol, dtype=NP[dtype])
        ok(L.ref_fill_lowertri(CODE[dtype], sval(lower).encode(), sval(upper).encode(),
                               ctypes.c_uint64(nrow), ctypes.c_uint64(ncol), ctypes.c_int64(start),
                               ctypes.c_void_p(out.ctypes.data)))
        arrays["fill/%d" % i] = out
        meta["fill"].append(dict(dtype=dtype, lower=sval(lower), upper=sval(upper), nrow=nrow, ncol=ncol,
                                 start=start))

    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **arrays)
    print("wrote %d einsummable, %d merge, %d touch, %d fill cases" %
          (len(meta["einsummable"]), len(meta["merge"]), len(meta["touch"]), len(meta["fill"])))


if __name__ == "__main__":
    main()
