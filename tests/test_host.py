"""Host-side logic of the library, without a GPU: the C ABI loads and exports
every declared symbol, descriptors are validated, merge_adjacent_dims / touch
simplify match the reference fixtures, and every generated kernel compiles for
sm_100a."""
import ctypes
import os
import re

import pytest

import einsummable_b200 as es
from einsummable_b200 import _lib, einsummable_t, scalarop_t, touch_t
from conftest import ROOT, golden

G = golden()


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "es_b200.h")).read()
    declared = set(re.findall(r"\b(es_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), "missing symbol " + name
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    assert b"sm_100a" in _lib.load().es_b200_version()


def test_no_gpu_means_loud_failure_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(es.es_error) as ei:
        es.kernel_manager_t(0)
    assert ei.value.status == _lib.ES_CUDA_ERROR


@pytest.mark.parametrize("case", G.meta["merge"] + G.meta["einsummable"],
                         ids=lambda c: c.get("name", str(c["join_shape"])))
def test_native_merge_matches_reference(case):
    e = einsummable_t(case["join_shape"], case["inns"], case["out_rank"], case["join"], case["castable"])
    s, shape, orank, inns = case["merged"].split("|")[:4]
    m = e.merge_adjacent_dims()
    assert m.str() == s
    assert ",".join(map(str, m.join_shape)) == shape
    assert str(m.out_rank) == orank
    assert ";".join(",".join(map(str, t)) for t in m.inns) == inns
    assert e.str() == case["merged"].split("|")[4]


@pytest.mark.parametrize("case", G.meta["touch"], ids=lambda c: c["name"])
def test_native_touch_simplify_matches_reference(case):
    t = touch_t(case["selection"], case["castable"], case["dtype"]).simplify()
    assert [list(s.astuple()) for s in t.selection] == case["simplified"]


@pytest.mark.parametrize("case", G.meta["einsummable"], ids=lambda c: c["name"])
def test_generated_kernel_compiles(case):
    e = einsummable_t(case["join_shape"], case["inns"], case["out_rank"], case["join"], case["castable"])
    kind = e.kernel_kind()
    assert kind
    log = e.compile_check()  # raises es_error(ES_COMPILE_ERROR) with the NVRTC log on failure
    assert "error" not in log.lower()
    assert "spill stores" not in log or " 0 bytes spill stores" in log


def test_python_builders_match_reference_strings():
    S = scalarop_t
    gold = G.meta["scalarops"]
    for dt in ("f16", "f32", "f64"):
        assert S.make_identity(dt).text == gold["identity/" + dt]
        assert S.make_add(dt).text == gold["add/" + dt]
        assert S.make_mul(dt).text == gold["mul/" + dt]
        assert S.make_sub(dt).text == gold["sub/" + dt]
        assert S.make_div(dt).text == gold["div/" + dt]
        assert S.make_neg(dt).text == gold["neg/" + dt]
        assert S.make_max(dt).text == gold["max/" + dt]
        assert S.make_min(dt).text == gold["min/" + dt]
        assert S.make_exp(dt).text == gold["exp/" + dt]
        assert S.make_log(dt).text == gold["log/" + dt]
        assert S.make_silu(dt).text == gold["silu/" + dt]
        assert S.make_sigmoid(dt).text == gold["sigmoid/" + dt]
        assert S.make_relu(dt).text == gold["relu/" + dt]
        assert S.make_square(dt).text == gold["square/" + dt]
        assert S.make_sqrt(dt).text == gold["sqrt/" + dt]
        assert S.make_inverse_sqrt(dt).text == gold["inverse_sqrt/" + dt]
        assert S.make_is_equal(dt).text == gold["is_equal/" + dt]
        assert S.make_scale(0.25, dt).text == gold["scale:0.25/" + dt]
        assert S.combine(S.make_mul(dt), [S.make_silu(dt), S.make_identity(dt)]).text == gold["silu_mul/" + dt]
        assert S.combine(S.make_exp(dt), [S.make_sub(dt)]).text == gold["exp_sub/" + dt]
    assert S.make_convert_dtype("f16", "f32").text == gold["convert:f32/f16"]
    assert S.make_conjugate().text == gold["conjugate/c64"]
    assert S.make_silu("f16").out_dtype() == "f16"
    assert S.make_convert_dtype("f16", "f32").out_dtype() == "f32"


def _describe_status(e):
    buf = ctypes.create_string_buffer(1 << 16)
    return _lib.load().es_b200_describe(ctypes.byref(e.to_desc()), 1, buf, 1 << 16)


def test_bad_descriptors_are_rejected_with_codes():
    lib = _lib.load()
    mul = scalarop_t.make_mul("f32")
    good = einsummable_t([4, 5, 6], [[0, 2], [2, 1]], 2, mul, "add")
    assert _describe_status(good) == _lib.ES_OK

    d = good.to_desc(); d.join_shape[1] = 0   # zero extent (src/einsummable/einsummable.cc:79-83)
    buf = ctypes.create_string_buffer(256)
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR
    assert b"zero" in lib.es_b200_last_error()

    d = good.to_desc(); d.castable = -1       # aggregation without castable (:39-41)
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR

    d = good.to_desc(); d.inn_modes[0][1] = 7  # mode out of range
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR

    d = good.to_desc(); d.n_inn = 1            # join has 2 holes, 1 input (:43-49)
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR

    d = good.to_desc(); d.join = b"*[hole|f32@0,hole|f16@1]"   # type failure
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR

    d = good.to_desc(); d.join = b"*[hole|f32@0,variable{lr|f32}]"  # unresolved variable
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR

    d = good.to_desc(); d.join = b"bogus[hole|f32@0]"
    assert lib.es_b200_describe(ctypes.byref(d), 1, buf, 256) == _lib.ES_BAD_DESCRIPTOR

    assert lib.es_b200_describe(None, 1, buf, 256) == _lib.ES_BAD_ARGUMENT
    # null handle on a launch entry point: error code, no crash
    assert lib.es_b200_launch_touch(None, None, 1, -1, 0, None, None, None) == _lib.ES_BAD_ARGUMENT
    assert lib.es_b200_fill_constant(None, 0, None, 4, None, None) == _lib.ES_BAD_ARGUMENT


def test_kernel_kinds_of_the_llama_layer():
    S = scalarop_t
    kinds = {
        "ew_vec": einsummable_t([8388608], [[0], [0]], 1, S.make_add("f16")),
        "red_row": einsummable_t([65536, 512], [[0, 1]], 1, S.make_identity("f32"), "max"),
        "ew_transpose": einsummable_t([64, 64], [[1, 0]], 2, S.make_identity("f32")),
        "red_col": einsummable_t([4096, 2048], [[1, 0]], 1, S.make_identity("f32"), "add"),
        "red_split": einsummable_t([4, 1 << 22], [[0, 1]], 1, S.make_identity("f32"), "add"),
    }
    for kind, e in kinds.items():
        assert e.kernel_kind().startswith(kind), (kind, e.kernel_kind())
    # ab,a->ab and ab,b->ab and the rope pattern all vectorise
    assert einsummable_t([2048, 4096], [[0, 1], [0]], 2, S.make_mul("f32")).kernel_kind() == "ew_vec"
    assert einsummable_t([2048, 4096], [[0, 1], [1]], 2, S.make_mul("f16")).kernel_kind() == "ew_vec"
    assert einsummable_t([4, 512, 32, 64], [[0, 1, 2, 3], [1, 3]], 4, S.make_mul("c64")).kernel_kind() == "ew_vec"
    assert einsummable_t([32, 512, 32, 128], [[0, 2, 1, 3]], 4, S.make_identity("f16")).kernel_kind() == "ew_vec"


@pytest.mark.parametrize("spec,extents,expect", [
    # every row pair is a 256-row item: 128 items for 148 SMs beat two waves of 128-row tiles
    ("ij,kj->ik", dict(i=2048, j=4096, k=4096), "items256=128,items128=0"),
    # two full waves of 256-row items, the rest as 128-row items (FFN shape)
    ("ij,kj->ik", dict(i=2048, j=4096, k=11008), "items256=296,items128=96"),
    # odd number of 128-row tiles: the last row is scheduled alone
    ("ij,kj->ik", dict(i=2176, j=1024, k=2816), "items256=88,items128=11"),
    # too few tiles to gain from larger items: one wave of 128-row tiles
    ("ij,kj->ik", dict(i=512, j=1024, k=768), None),
    # two k-blocks per tile (attention scores): epilogue-bound, 128-row tiles
    ("acbe,adbe->abcd", dict(a=4, b=32, c=512, d=512, e=128), None),
    # f32 (3xTF32) keeps 128 x 128 tiles
    ("ij,jk->ik", dict(i=2048, j=2048, k=2048), None),
])
def test_contraction_schedule_choice(spec, extents, expect):
    """The split into 256-row and 128-row work items is made at build time from the shape alone
    (host code: no GPU needed)."""
    dtype = "f32" if spec == "ij,jk->ik" else "f16"
    e = einsummable_t.from_str(spec, extents, scalarop_t.make_mul(dtype), "add")
    assert e._describe(1).startswith("contraction_tc")
    info = e._describe(4)
    assert "bm=128" in info and "stages=" in info
    if expect is None:
        assert "items256" not in info, info
    else:
        assert expect in info, info


def test_multiply_high_division_is_exact_below_2_31():
    """The tile decode of the contraction kernel and the index decode of the touch kernel divide by
    fixed divisors with q = umulhi(n, m) >> s, l = ceil(log2 d), m = ceil(2^(31+l) / d), s = l - 1
    (csrc/contraction.cu make_fd, csrc/kernels.cu make_fastdiv).  The claim: exact for every
    numerator below 2^31.  Checked here on the arithmetic itself, at the edges and at random."""
    import random

    def make(d):
        if d <= 1:
            return None
        l = (d - 1).bit_length()
        m = ((1 << (31 + l)) + d - 1) // d
        assert m < (1 << 32)
        return m, l - 1

    def div(n, d, f):
        return n if f is None else ((n * f[0]) >> 32) >> f[1]

    rng = random.Random(5)
    divisors = [1, 2, 3, 5, 7, 43, 148, 250, 344, 1000, 11008, 32000, (1 << 16) - 1, (1 << 16) + 1, (1 << 30) - 1,
                (1 << 30) + 1, (1 << 31) - 1] + [rng.randrange(1, 1 << 31) for _ in range(300)]
    for d in divisors:
        f = make(d)
        edge = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, (1 << 31) - 1, ((1 << 31) - 1) // d * d, ((1 << 31) - 1) // d * d - 1]
        for n in edge + [rng.randrange(0, 1 << 31) for _ in range(200)]:
            if 0 <= n < (1 << 31):
                assert div(n, d, f) == n // d, (n, d)


def test_generated_kernels_are_cached_on_disk(tmp_path):
    """build() compiles through a cache directory: the second process (here: the second call with a
    fresh library state is not needed -- the file is what matters) finds the cubin instead of running NVRTC."""
    import subprocess
    import sys
    import time
    code = (
        "import sys, time, ctypes; sys.path.insert(0, %r)\n"
        "from einsummable_b200 import _lib\n"
        "from einsummable_b200.einsummable import einsummable_t\n"
        "from einsummable_b200.scalarop import scalarop_t as S\n"
        "lib = _lib.load()\n"
        "e = einsummable_t([1234, 512], [[0, 1], [0, 1]], 2, S.combine(S.make_mul('f16'), [S.make_silu('f16'), S.make_identity('f16')]))\n"
        "buf = ctypes.create_string_buffer(256)\n"
        "t0 = time.time(); _lib.check(lib.es_b200_describe(ctypes.byref(e.to_desc()), 5, buf, 256)); print(buf.value.decode(), time.time() - t0)\n"
    ) % (ROOT,)
    env = dict(os.environ, ES_B200_CACHE_DIR=str(tmp_path / "kernels"))
    first = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert first.returncode == 0, first.stderr[-1000:]
    files = os.listdir(tmp_path / "kernels")
    assert len(files) == 1 and files[0].endswith(".cubin")
    size = os.path.getsize(tmp_path / "kernels" / files[0])
    assert first.stdout.split()[1] == "bytes=%d" % size
    stamp = os.path.getmtime(tmp_path / "kernels" / files[0])
    second = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert second.returncode == 0 and second.stdout.split()[1] == "bytes=%d" % size
    assert os.path.getmtime(tmp_path / "kernels" / files[0]) == stamp          # read, not rewritten
    assert float(second.stdout.split()[2]) < float(first.stdout.split()[2])    # a file read beats a compilation
    off = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                         env=dict(env, ES_B200_CACHE_DIR="0"), timeout=120)
    assert off.returncode == 0 and len(os.listdir(tmp_path / "kernels")) == 1
