"""kernel_manager_t: the reference's kernel-manager surface over the C ABI.

Same members and argument meaning as kernel_manager_t in
src/engine/gpu/gpu_kernel_manager.h:274-321: build() an einsummable into a
reusable kernel and get its workspace size (None = unsupported, the reference's
nullopt), then launch it -- or a touch, or a fill -- on a CUDA stream with
device pointers owned by the caller.  Pointers may be given as integers or as
torch CUDA tensors; streams as integers (cudaStream_t), torch streams or None
(the legacy default stream).
"""
import ctypes
import struct

import numpy as np

from . import _lib
from .einsummable import CASTABLE_CODE, einsummable_t, fill_t, touch_t
from .scalarop import DTYPE_CODE


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    raise TypeError("expected a device pointer (int) or a torch tensor")


def _stream(s):
    if s is None:
        return None
    if isinstance(s, int):
        return s or None
    if hasattr(s, "cuda_stream"):
        return s.cuda_stream or None
    raise TypeError("expected a cudaStream_t (int), a torch stream or None")


def scalar_bytes(value, dtype):
    """The 8 raw bytes of a scalar_t's payload (src/einsummable/scalarop.h:24-80)."""
    if dtype == "f16":
        b = np.float16(value).tobytes()
    elif dtype == "f32":
        b = np.float32(value).tobytes()
    elif dtype == "f64":
        b = np.float64(value).tobytes()
    elif dtype == "c64":
        b = np.complex64(value).tobytes()
    else:
        raise ValueError("unknown dtype %r" % (dtype,))
    return b + bytes(8 - len(b))


class kernel_manager_t:
    def __init__(self, device=0):
        self._lib = _lib.load()
        self.device = device
        h = ctypes.c_void_p()
        _lib.check(self._lib.es_b200_create(device, ctypes.byref(h)))
        self._h = h
        self._ids = {}

    def close(self):
        if getattr(self, "_h", None):
            self._lib.es_b200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_f32_policy(self, policy):
        """'3xtf32' (default) or 'tf32' for f32 contractions on the tensor cores."""
        code = {"3xtf32": 0, "tf32": 1}[policy]
        _lib.check(self._lib.es_b200_set_f32_policy(self._h, code))
        self._ids.clear()

    @staticmethod
    def _key(e):
        return (tuple(e.join_shape), tuple(map(tuple, e.inns)), e.out_rank, e.join.text, e.castable)

    def build(self, e):
        """Returns the workspace size in bytes, or None when unsupported."""
        ws, kid = ctypes.c_uint64(0), ctypes.c_uint64(0)
        st = self._lib.es_b200_build_einsummable(self._h, ctypes.byref(e.to_desc()),
                                                 ctypes.byref(ws), ctypes.byref(kid))
        if st == _lib.ES_NOT_SUPPORTED:
            return None
        _lib.check(st)
        self._ids[self._key(e)] = (kid.value, ws.value)
        return ws.value

    def workspace_size(self, e):
        return self._built(e)[1]

    def kernel_info(self, e):
        buf = ctypes.create_string_buffer(4096)
        _lib.check(self._lib.es_b200_kernel_info(self._h, self._built(e)[0], buf, 4096))
        return buf.value.decode()

    def _built(self, e):
        try:
            return self._ids[self._key(e)]
        except KeyError:
            # kernel_manager_t::operator() throws when build was not called
            # (src/engine/gpu/gpu_kernel_manager.cc:1257-1261)
            raise _lib.es_error(_lib.ES_NOT_BUILT, "get_built_kernel_info: this einsummable was not built")

    def __call__(self, op, stream, out, inns, workspace=None):
        if isinstance(op, touch_t):
            return self._touch(op, stream, out, inns)
        if not isinstance(op, einsummable_t):
            raise TypeError("expected an einsummable_t or a touch_t")
        kid, _ = self._built(op)
        inns = list(inns)
        arr = (ctypes.c_void_p * max(len(inns), 1))(*[_ptr(x) for x in inns])
        ws_ptr, ws_size = (None, 0) if workspace is None else (_ptr(workspace[0]), int(workspace[1]))
        _lib.check(self._lib.es_b200_launch_einsummable(
            self._h, kid, _stream(stream), _ptr(out), arr, len(inns), ws_ptr, ws_size))

    def _touch(self, t, stream, out, inn):
        _lib.check(self._lib.es_b200_launch_touch(
            self._h, t.c_dims(), len(t.selection), CASTABLE_CODE[t.castable], DTYPE_CODE[t.dtype],
            _stream(stream), _ptr(out), _ptr(inn)))

    def _touch_items(self, touches, outs, inns):
        n = len(touches)
        items = (_lib.es_touch_item_t * n)()
        for i, t in enumerate(touches):
            if t.dtype != touches[0].dtype:
                raise ValueError("touch_batch: mixed dtypes")
            for j, s in enumerate(t.selection):
                items[i].dims[j] = _lib.es_touchdim_t(*s.astuple())
            items[i].rank = len(t.selection)
            items[i].castable = CASTABLE_CODE[t.castable]
            items[i].out = _ptr(outs[i])
            items[i].inn = _ptr(inns[i])
        return items

    def touch_batch(self, touches, stream, outs, inns, items_dev):
        """Launches many touches of one dtype at once; items_dev is a device
        buffer of at least len(touches) * sizeof(es_touch_item_t) bytes."""
        items = self._touch_items(touches, outs, inns)
        _lib.check(self._lib.es_b200_launch_touch_batch(
            self._h, items, len(touches), DTYPE_CODE[touches[0].dtype], _stream(stream), _ptr(items_dev)))

    def prepare_touch_batch(self, touches, stream, outs, inns, items_dev):
        """Validates and lowers the touches once and stages them in items_dev;
        the result can be launched repeatedly with launch_prepared_touch_batch."""
        items = self._touch_items(touches, outs, inns)
        prepared = _lib.es_touch_batch_t()
        _lib.check(self._lib.es_b200_prepare_touch_batch(
            self._h, items, len(touches), DTYPE_CODE[touches[0].dtype], _stream(stream), _ptr(items_dev),
            ctypes.byref(prepared)))
        return prepared

    def launch_prepared_touch_batch(self, prepared, stream):
        _lib.check(self._lib.es_b200_launch_prepared_touch_batch(self._h, ctypes.byref(prepared), _stream(stream)))

    def constant_fill(self, c, stream, out):
        n = 1
        for s in c.shape:
            n *= s
        v = scalar_bytes(c.value, c.dtype)
        _lib.check(self._lib.es_b200_fill_constant(
            self._h, DTYPE_CODE[c.dtype], v, n, _stream(stream), _ptr(out)))

    def lowerTri_fill(self, l, stream, out):
        _lib.check(self._lib.es_b200_fill_lowertri(
            self._h, DTYPE_CODE[l.dtype], scalar_bytes(l.lower, l.dtype),
            scalar_bytes(l.upper, l.dtype), l.nrow, l.ncol, l.start, _stream(stream), _ptr(out)))

    def move(self, src_device, src, dst, nbytes, stream):
        """gpu_copy_t::launch: copy nbytes from src on src_device into dst on this manager's device."""
        _lib.check(self._lib.es_b200_move(
            self._h, src_device, _ptr(src), self.device, _ptr(dst), int(nbytes), _stream(stream)))

    def flag_signal(self, flag, stream, limit_ms=0):
        """Stream-ordered: wait until the (peer-visible) flag is 0, then set it to 1."""
        _lib.check(self._lib.es_b200_flag_signal(self._h, _ptr(flag), int(limit_ms), _stream(stream)))

    def flag_wait(self, flag, stream, limit_ms=0):
        """Stream-ordered: wait until the local flag is 1, then reset it to 0."""
        _lib.check(self._lib.es_b200_flag_wait(self._h, _ptr(flag), int(limit_ms), _stream(stream)))

    def pull(self, src, dst, nbytes, stream):
        """SM copy from a peer-mapped source into local memory."""
        _lib.check(self._lib.es_b200_pull(self._h, _ptr(src), _ptr(dst), int(nbytes), _stream(stream)))

    def attention(self, desc, stream, out, q, k, v, mask):
        """The fused attention chain (scores, mask, softmax, values) as one launch; `desc` is an
        attention_t (einsummable_b200.attention)."""
        c = desc.c_struct()
        _lib.check(self._lib.es_b200_launch_attention(
            self._h, ctypes.byref(c), _stream(stream), _ptr(out), _ptr(q), _ptr(k), _ptr(v),
            _ptr(mask) if mask is not None else None))

    def rowsum_f32_noalloc(self, stream, out, inn, rows, cols):
        """out[a] = sum_b inn[a,b] for f32 without any device allocation: the
        scratch of the two-pass reduction is a fixed array inside the library
        (rows <= 65536).  Meant for callers that cannot call cudaMalloc -- all
        device memory already belongs to the memgraph buffer, or the event loop
        cannot take cudaMalloc's device synchronisation.  Calls on one device
        share that array, so launches that may overlap on the GPU race; make the
        first call on a device before starting a stream capture."""
        _lib.check(self._lib.es_b200_rowsum_f32_noalloc(
            self._h, _ptr(inn), _ptr(out), int(rows), int(cols), _stream(stream)))

    def device_status(self):
        """Synchronises and returns the tensor-core kernels' error word (0 = fine)."""
        w = ctypes.c_uint(0)
        _lib.check(self._lib.es_b200_device_status(self._h, ctypes.byref(w)))
        return w.value

    def debug_trace(self, n=8000):
        """Clock samples of the last tensor-core contraction launch (trace builds only, see
        einsummable_b200/trace.py); raises with ES_NOT_SUPPORTED on the product library."""
        buf = (ctypes.c_ulonglong * n)()
        got = ctypes.c_int(0)
        _lib.check(self._lib.es_b200_debug_trace(self._h, buf, n, ctypes.byref(got)))
        return list(buf[:got.value])

    def counters(self):
        arr = (ctypes.c_uint64 * 4)()
        _lib.check(self._lib.es_b200_query_counters(self._h, arr))
        return dict(zip(("einsummable", "touch", "fill", "move"), arr))
