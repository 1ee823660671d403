"""Host-side mirrors of einsummable_t, touch_t and fill_t.

Field names and argument meaning follow the reference
(src/einsummable/einsummable.h:8-31, src/einsummable/touch.h:8-31,
src/einsummable/fill.h:11-83) so that tests read like the reference's own.
"""
import ctypes

from . import _lib
from .scalarop import DTYPE_CODE, DTYPE_SIZE, scalarop_t, default_dtype

CASTABLE_CODE = {None: -1, "add": 0, "mul": 1, "min": 2, "max": 3, "+": 0, "x": 1, "v": 2, "^": 3}


class einsummable_t:
    def __init__(self, join_shape, inns, out_rank, join, castable=None):
        self.join_shape = [int(x) for x in join_shape]
        self.inns = [list(map(int, t)) for t in inns]
        self.out_rank = int(out_rank)
        self.join = join if isinstance(join, scalarop_t) else scalarop_t(join)
        self.castable = castable
        if self.has_aggregation() and castable is None:
            raise ValueError("Must have castable when aggregating.")
        if self.join.num_inputs() != len(self.inns):
            raise ValueError("einsummable inns size not same as scalarop join")

    # ---- constructors named as in the reference ----
    @staticmethod
    def parse_str(s):
        """'ij,jk->ik' -> (inns, out_rank); output modes are numbered first."""
        lhs, out = s.replace(" ", "").split("->")
        letters = {}
        for ch in out:
            letters.setdefault(ch, len(letters))
        terms = lhs.split(",")
        for t in terms:
            for ch in t:
                letters.setdefault(ch, len(letters))
        return [[letters[ch] for ch in t] for t in terms], len(out)

    @staticmethod
    def from_str(s, shape_of, join, castable=None):
        """shape_of: dict letter -> extent."""
        inns, out_rank = einsummable_t.parse_str(s)
        lhs, out = s.replace(" ", "").split("->")
        order = {}
        for ch in out + lhs.replace(",", ""):
            order.setdefault(ch, len(order))
        join_shape = [0] * len(order)
        for ch, m in order.items():
            join_shape[m] = shape_of[ch]
        return einsummable_t(join_shape, inns, out_rank, join, castable)

    @staticmethod
    def from_matmul(di, dj, dk, dtype=None):
        """ij,jk->ik (einsummable_t::from_matmul)"""
        d = dtype or default_dtype()
        return einsummable_t([di, dk, dj], [[0, 2], [2, 1]], 2, scalarop_t.make_mul(d), "add")

    @staticmethod
    def from_matmul_st(di, dj, dk, dtype=None):
        """ij,kj->ik"""
        d = dtype or default_dtype()
        return einsummable_t([di, dk, dj], [[0, 2], [1, 2]], 2, scalarop_t.make_mul(d), "add")

    @staticmethod
    def from_matmul_ts(di, dj, dk, dtype=None):
        """ji,jk->ik"""
        d = dtype or default_dtype()
        return einsummable_t([di, dk, dj], [[2, 0], [2, 1]], 2, scalarop_t.make_mul(d), "add")

    @staticmethod
    def from_matmul_tt(di, dj, dk, dtype=None):
        """ji,kj->ik"""
        d = dtype or default_dtype()
        return einsummable_t([di, dk, dj], [[2, 0], [1, 2]], 2, scalarop_t.make_mul(d), "add")

    @staticmethod
    def aggregate(inn_shape, inn, out_rank, dtype=None, castable="add"):
        d = dtype or default_dtype()
        join_shape = [0] * len(inn_shape)
        for pos, m in enumerate(inn):
            join_shape[m] = inn_shape[pos]
        return einsummable_t(join_shape, [list(inn)], out_rank, scalarop_t.make_identity(d), castable)

    # ---- queries ----
    def has_aggregation(self):
        return self.out_rank < len(self.join_shape)

    def out_dtype(self):
        return self.join.out_dtype()

    def inn_dtype(self, k):
        return self.join.inn_dtype(k)

    def out_shape(self):
        return self.join_shape[:self.out_rank]

    def inn_shape(self, k):
        return [self.join_shape[m] for m in self.inns[k]]

    def inn_shapes(self):
        return [self.inn_shape(k) for k in range(len(self.inns))]

    def out_nelem(self):
        n = 1
        for x in self.out_shape():
            n *= x
        return n

    def str(self):
        terms = ["".join(chr(ord("a") + m) for m in t) for t in self.inns]
        return ",".join(terms) + "->" + "".join(chr(ord("a") + m) for m in range(self.out_rank))

    def __repr__(self):
        return "einsummable_t(%s %s %s %s)" % (self.str(), self.join_shape, self.join, self.castable)

    def to_desc(self):
        d = _lib.es_einsummable_desc_t()
        if len(self.join_shape) > _lib.ES_MAX_RANK or len(self.inns) > _lib.ES_MAX_INNS:
            raise ValueError("einsummable exceeds ES_MAX_RANK / ES_MAX_INNS")
        d.join_rank = len(self.join_shape)
        for i, s in enumerate(self.join_shape):
            d.join_shape[i] = s
        d.n_inn = len(self.inns)
        for k, t in enumerate(self.inns):
            d.inn_rank[k] = len(t)
            for j, m in enumerate(t):
                d.inn_modes[k][j] = m
        d.out_rank = self.out_rank
        d.castable = CASTABLE_CODE[self.castable]
        self._join_bytes = self.join.text.encode()  # keep alive
        d.join = self._join_bytes
        return d

    def _describe(self, what):
        lib = _lib.load()
        size = 1 << 16
        while True:
            buf = ctypes.create_string_buffer(size)
            st = lib.es_b200_describe(ctypes.byref(self.to_desc()), what, buf, size)
            if st == _lib.ES_BAD_ARGUMENT and b"too small" in lib.es_b200_last_error() and size < (1 << 24):
                size *= 4
                continue
            _lib.check(st)
            return buf.value.decode()

    def merge_adjacent_dims(self):
        """einsummable_t::merge_adjacent_dims, computed by the native library."""
        _, shape, out_rank, inns = self._describe(0).split("|")
        return einsummable_t([int(x) for x in shape.split(",")],
                             [[int(m) for m in t.split(",")] for t in inns.split(";")],
                             int(out_rank), self.join, self.castable)

    def kernel_kind(self):
        return self._describe(1)

    def kernel_source(self):
        return self._describe(2)

    def compile_check(self):
        """Generates and compiles the kernel for sm_100a (no GPU needed)."""
        return self._describe(3)


class touchdim_t:
    def __init__(self, d_inn, d_out, offset_inn, offset_out, size):
        self.d_inn, self.d_out = int(d_inn), int(d_out)
        self.offset_inn, self.offset_out, self.size = int(offset_inn), int(offset_out), int(size)

    def astuple(self):
        return (self.d_inn, self.d_out, self.offset_inn, self.offset_out, self.size)

    def __repr__(self):
        return "touchdim_t(d_inn=%d, d_out=%d, offset_inn=%d, offset_out=%d, size=%d)" % self.astuple()

    def __eq__(self, o):
        return self.astuple() == o.astuple()


class touch_t:
    def __init__(self, selection, castable, dtype):
        self.selection = [s if isinstance(s, touchdim_t) else touchdim_t(*s) for s in selection]
        self.castable = castable
        self.dtype = dtype

    def c_dims(self):
        arr = (_lib.es_touchdim_t * len(self.selection))()
        for i, s in enumerate(self.selection):
            arr[i] = _lib.es_touchdim_t(*s.astuple())
        return arr

    def simplify(self):
        """touch_t::simplify (src/einsummable/touch.cc:3-28), native."""
        lib = _lib.load()
        n = len(self.selection)
        out = (_lib.es_touchdim_t * n)()
        r = ctypes.c_int(0)
        _lib.check(lib.es_b200_touch_simplify(self.c_dims(), n, out, ctypes.byref(r)))
        sel = [touchdim_t(o.d_inn, o.d_out, o.offset_inn, o.offset_out, o.size) for o in out[:r.value]]
        return touch_t(sel, self.castable, self.dtype)

    def inn_nelem(self):
        n = 1
        for s in self.selection:
            n *= s.d_inn
        return n

    def out_nelem(self):
        n = 1
        for s in self.selection:
            n *= s.d_out
        return n


class fill_t:
    """fill_t::constant_t / fill_t::lowertri_t (src/einsummable/fill.h:11-33)."""

    class constant_t:
        def __init__(self, value, shape, dtype):
            self.value, self.shape, self.dtype = value, list(shape), dtype

    class lowertri_t:
        def __init__(self, lower, upper, nrow, ncol, start, dtype):
            self.lower, self.upper = lower, upper
            self.nrow, self.ncol, self.start, self.dtype = int(nrow), int(ncol), int(start), dtype
