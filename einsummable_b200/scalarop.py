"""Host-side mirror of the reference's scalarop_t builders.

A scalarop here is just the reference's text form (operator<<,
src/einsummable/scalarop.cc:2878-3011) plus the dtypes of its holes; the
builders below write the same trees the reference's make_* functions produce
after simplification (src/einsummable/scalarop.cc:2204-2527).  Evaluation
happens on the GPU only; there is no CPU evaluator in this package.
"""
import re

DTYPES = ("f16", "f32", "f64", "c64")
DTYPE_CODE = {d: i for i, d in enumerate(DTYPES)}
DTYPE_SIZE = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}
_default_dtype = "f32"


def default_dtype():
    return _default_dtype


def set_default_dtype(d):
    """set_default_dtype (src/einsummable/scalarop.h:282-286)"""
    global _default_dtype
    assert d in DTYPES
    _default_dtype = d


def _d(d):
    return default_dtype() if d is None else d


def _fmt(v):
    if isinstance(v, str):
        return v
    if v != v:
        return "NAN"
    if v == float("inf"):
        return "INF"
    if v == float("-inf"):
        return "NINF"
    return "%g" % v


class scalarop_t:
    """Text form + hole dtypes of a join op."""

    _hole = re.compile(r"hole\|(f16|f32|f64|c64)@(\d+)")

    def __init__(self, text):
        self.text = text
        self.hole_dtypes = {}
        for d, k in self._hole.findall(text):
            k = int(k)
            if self.hole_dtypes.setdefault(k, d) != d:
                raise ValueError("hole %d used with two dtypes" % k)

    def __str__(self):
        return self.text

    def __repr__(self):
        return "scalarop_t(%r)" % self.text

    def __eq__(self, other):
        return isinstance(other, scalarop_t) and other.text == self.text

    def __hash__(self):
        return hash(self.text)

    def num_inputs(self):
        return max(self.hole_dtypes) + 1 if self.hole_dtypes else 0

    def inn_dtype(self, k):
        return self.hole_dtypes[k]

    def out_dtype(self):
        """Dtype of the root node, by the reference's typing rules."""
        return _out_dtype(self.text)

    # ---- builders (names follow the reference) ----
    @staticmethod
    def from_string(s):
        return scalarop_t(s)

    @staticmethod
    def make_identity(d=None):
        return scalarop_t("hole|%s@0" % _d(d))

    @staticmethod
    def make_arg(arg, d=None):
        return scalarop_t("hole|%s@%d" % (_d(d), arg))

    @staticmethod
    def make_constant(value, d=None):
        return scalarop_t("constant{%s|%s}" % (_d(d), _fmt(value)))

    @staticmethod
    def make_add(d=None):
        return scalarop_t("+[hole|{0}@0,hole|{0}@1]".format(_d(d)))

    @staticmethod
    def make_mul(d=None):
        return scalarop_t("*[hole|{0}@0,hole|{0}@1]".format(_d(d)))

    @staticmethod
    def make_sub(d=None):
        return scalarop_t("+[hole|{0}@0,*[constant{{{0}|-1}},hole|{0}@1]]".format(_d(d)))

    @staticmethod
    def make_div(d=None):
        return scalarop_t("*[hole|{0}@0,power{{-1}}[hole|{0}@1]]".format(_d(d)))

    @staticmethod
    def make_neg(d=None):
        return scalarop_t("*[constant{{{0}|-1}},hole|{0}@0]".format(_d(d)))

    @staticmethod
    def make_max(d=None):
        return scalarop_t("ite_>[hole|{0}@0,hole|{0}@1,hole|{0}@0,hole|{0}@1]".format(_d(d)))

    @staticmethod
    def make_min(d=None):
        return scalarop_t("ite_<[hole|{0}@0,hole|{0}@1,hole|{0}@0,hole|{0}@1]".format(_d(d)))

    @staticmethod
    def make_is_equal(d=None):
        return scalarop_t(
            "ite_==[hole|{0}@0,hole|{0}@1,constant{{{0}|1}},constant{{{0}|0}}]".format(_d(d)))

    @staticmethod
    def make_scale(value, d=None):
        return scalarop_t("*[constant{{{0}|{1}}},hole|{0}@0]".format(_d(d), _fmt(value)))

    @staticmethod
    def make_increment(value, d=None):
        return scalarop_t("+[constant{{{0}|{1}}},hole|{0}@0]".format(_d(d), _fmt(value)))

    @staticmethod
    def make_exp(d=None):
        return scalarop_t("exp[hole|%s@0]" % _d(d))

    @staticmethod
    def make_log(d=None):
        return scalarop_t("log[hole|%s@0]" % _d(d))

    @staticmethod
    def make_power(p, d=None):
        return scalarop_t("power{%s}[hole|%s@0]" % (_fmt(p), _d(d)))

    @staticmethod
    def make_square(d=None):
        return scalarop_t.make_power(2, d)

    @staticmethod
    def make_sqrt(d=None):
        return scalarop_t.make_power(0.5, d)

    @staticmethod
    def make_inverse(d=None):
        return scalarop_t.make_power(-1, d)

    @staticmethod
    def make_inverse_sqrt(d=None):
        return scalarop_t.make_power(-0.5, d)

    @staticmethod
    def make_sigmoid(d=None):
        return scalarop_t(
            "power{{-1}}[+[constant{{{0}|1}},exp[*[constant{{{0}|-1}},hole|{0}@0]]]]".format(_d(d)))

    @staticmethod
    def make_silu(d=None):
        return scalarop_t(
            "*[hole|{0}@0,power{{-1}}[+[constant{{{0}|1}},exp[*[constant{{{0}|-1}},hole|{0}@0]]]]]"
            .format(_d(d)))

    @staticmethod
    def make_relu(d=None):
        return scalarop_t(
            "ite_>=[constant{{{0}|0}},hole|{0}@0,constant{{{0}|0}},hole|{0}@0]".format(_d(d)))

    @staticmethod
    def make_convert_dtype(src, dst):
        return scalarop_t("to_%s[hole|%s@0]" % (dst, src))

    @staticmethod
    def make_conjugate(d="c64"):
        return scalarop_t("conj[hole|%s@0]" % d)

    @staticmethod
    def make_from_castable(castable, d=None):
        return {"add": scalarop_t.make_add, "mul": scalarop_t.make_mul,
                "min": scalarop_t.make_min, "max": scalarop_t.make_max}[castable](d)

    @staticmethod
    def combine(op, ops):
        """scalarop_t::combine: op's hole k is replaced by ops[k], whose own
        holes are renumbered after those of ops[0..k-1]
        (Example in src/einsummable/scalarop.h: op = *, ops = (x0+x1, x0+x1)
        gives (x0+x1)*(x2+x3))."""
        shifted, base = [], 0
        for o in ops:
            n = o.num_inputs()
            shifted.append(scalarop_t._hole.sub(
                lambda m, b=base: "hole|%s@%d" % (m.group(1), int(m.group(2)) + b), o.text))
            base += n
        text = scalarop_t._hole.sub(lambda m: "\0%d\0" % int(m.group(2)), op.text)
        for k, s in enumerate(shifted):
            text = text.replace("\0%d\0" % k, s)
        return scalarop_t(text)


def _out_dtype(text):
    """Root dtype by the rules of op_t::type_of (src/einsummable/scalarop.cc:762-905)."""
    pos = [0]

    def node():
        s = text[pos[0]:]
        m = re.match(r"constant\{(f16|f32|f64|c64)\|[^}]*\}", s)
        if m:
            pos[0] += m.end()
            return m.group(1)
        m = re.match(r"hole\|(f16|f32|f64|c64)@\d+", s)
        if m:
            pos[0] += m.end()
            return m.group(1)
        m = re.match(r"variable\{\w+\|(f16|f32|f64|c64)\}", s)
        if m:
            pos[0] += m.end()
            return m.group(1)
        m = re.match(r"(\+|\*|exp|log|power\{[^}]*\}|ite_(?:<=|>=|==|<|>)|to_(f16|f32|f64|c64)|conj|real|imag|complex)\[", s)
        if not m:
            raise ValueError("cannot parse scalarop at %r" % s[:20])
        op = m.group(1)
        pos[0] += m.end()
        kids = [node()]
        while text[pos[0]] == ",":
            pos[0] += 1
            kids.append(node())
        assert text[pos[0]] == "]"
        pos[0] += 1
        if op.startswith("to_"):
            return m.group(2)
        if op.startswith("ite_"):
            return kids[2]
        if op in ("real", "imag"):
            return "f32"
        if op == "complex":
            return "c64"
        return kids[0]
    return node()
