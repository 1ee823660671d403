"""The oracle (oracle/es_oracle.py) against the reference's golden vectors and
against fixtures produced by the reference's own interpreter (tests/golden)."""
import numpy as np
import pytest

import es_oracle as O
from conftest import golden, ulp_distance

G = golden()
TRANSCENDENTAL = ("exp", "log", "power{-0.5}", "power{0.5}", "power{3}", "power{-2}")


def test_reference_matmul_known_answer():
    # tests/reference.h:4-46 -- the reference's own hard-coded vector
    lhs = np.arange(8, 20, dtype=np.float64)
    rhs = np.arange(100, 120, dtype=np.float64)
    want = [4110.0, 4148.0, 4186.0, 4224.0, 4262.0, 5830.0, 5884.0, 5938.0, 5992.0, 6046.0,
            7550.0, 7620.0, 7690.0, 7760.0, 7830.0]
    for mode in ("interp", "executor"):
        got = O.reference_einsummable([3, 5, 4], [[0, 2], [2, 1]], 2, "*[hole|f64@0,hole|f64@1]",
                                      "add", [lhs, rhs], mode)
        assert got.tolist() == want


def test_touch_known_answer():
    # produced by the reference's execute_touch / reference_touch on iota input
    sel = [(4, 3, 1, 0, 2), (6, 5, 2, 1, 3)]
    inn = np.arange(24, dtype=np.float16)
    out = np.zeros(15, dtype=np.float16)
    O.reference_touch(sel, None, out, inn)
    assert out.tolist() == [0, 8, 9, 10, 0, 0, 14, 15, 16, 0, 0, 0, 0, 0, 0]
    O.reference_touch(sel, "add", out, inn)
    assert out.tolist() == [0, 16, 18, 20, 0, 0, 28, 30, 32, 0, 0, 0, 0, 0, 0]
    assert O.touch_simplify([(4, 4, 0, 0, 4), (6, 6, 0, 0, 6)]) == [(24, 24, 0, 0, 24)]


@pytest.mark.parametrize("case", G.meta["einsummable"], ids=lambda c: c["name"])
def test_einsummable_interp_matches_reference(case):
    got = O.reference_einsummable(case["join_shape"], case["inns"], case["out_rank"], case["join"],
                                  case["castable"], G.es_inputs(case), "interp")
    want = G.es_output(case)
    assert got.dtype == want.dtype and got.shape == want.shape
    if any(t in case["join"] for t in TRANSCENDENTAL) or case["out_dtype"] == "c64":
        # libm / half.hpp transcendental and complex-multiply rounding may differ in the last place
        # (half.hpp's pow/exp are not correctly rounded; a 1-ulp difference in an inner
        # node of an f16 tree grows through the following products)
        tol = 4
        if case["castable"] is not None:
            np.testing.assert_allclose(got.astype(np.complex128 if got.dtype == np.complex64 else np.float64),
                                       want.astype(np.complex128 if got.dtype == np.complex64 else np.float64),
                                       rtol=2e-3 if case["out_dtype"] == "f16" else 1e-5)
        else:
            assert ulp_distance(got, want) <= tol, case["name"]
    else:
        assert got.tobytes() == want.tobytes(), case["name"]


@pytest.mark.parametrize("case", G.meta["einsummable"], ids=lambda c: c["name"])
def test_einsummable_executor_mode_close_to_reference(case):
    """The executor-convention oracle (f32 math for f16, wide accumulation) must
    stay within the stated tolerances of the interpreter on these small cases."""
    got = O.reference_einsummable(case["join_shape"], case["inns"], case["out_rank"], case["join"],
                                  case["castable"], G.es_inputs(case), "executor")
    want = G.es_output(case)
    wide = np.complex128 if want.dtype == np.complex64 else np.float64
    rtol = {"f16": 1e-2, "f32": 1e-5, "f64": 1e-12, "c64": 1e-5}[case["out_dtype"]]
    scale = max(1.0, float(np.abs(want.astype(wide)).max()))
    np.testing.assert_allclose(got.astype(wide), want.astype(wide), rtol=rtol, atol=rtol * scale)


@pytest.mark.parametrize("case", G.meta["merge"] + G.meta["einsummable"],
                         ids=lambda c: c.get("name", str(c["join_shape"])))
def test_merge_adjacent_dims(case):
    shape, inns, out_rank = O.merge_adjacent_dims(case["join_shape"], case["inns"], case["out_rank"])
    s, sh, orank, ins = case["merged"].split("|")[:4]
    assert O.einsummable_str(inns, out_rank) == s
    assert ",".join(map(str, shape)) == sh
    assert str(out_rank) == orank
    assert ";".join(",".join(map(str, t)) for t in inns) == ins
    # un-merged str
    assert O.einsummable_str(case["inns"], case["out_rank"]) == case["merged"].split("|")[4]


@pytest.mark.parametrize("case", G.meta["touch"], ids=lambda c: c["name"])
def test_touch_bit_exact(case):
    out = G.arrays["touch/%s/out0" % case["name"]].copy()
    O.reference_touch([tuple(s) for s in case["selection"]], case["castable"], out,
                      G.arrays["touch/%s/inn" % case["name"]])
    assert out.tobytes() == G.arrays["touch/%s/out" % case["name"]].tobytes()
    assert [list(s) for s in O.touch_simplify([tuple(s) for s in case["selection"]])] == case["simplified"]


@pytest.mark.parametrize("i", range(len(G.meta["fill"])))
def test_fill_lowertri(i):
    c = G.meta["fill"][i]
    conv = {"INF": float("inf"), "NINF": float("-inf")}

    def val(s):
        if s in conv:
            return conv[s]
        if s.startswith("("):
            a, b = s.strip("()").split(",")
            return complex(float(a), float(b))
        return float(s)
    got = O.reference_fill_lowertri(val(c["lower"]), val(c["upper"]), c["nrow"], c["ncol"], c["start"],
                                    c["dtype"])
    assert got.tobytes() == G.arrays["fill/%d" % i].tobytes()


def test_scalarop_parse_roundtrip_types():
    for key, text in G.meta["scalarops"].items():
        node = O.parse_scalarop(text)
        assert node.dtype in ("f16", "f32", "f64", "c64"), key
