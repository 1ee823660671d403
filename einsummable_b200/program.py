"""program_t: ctypes wrapper of the library's program executor (es_b200_program_*).

A program is the static schedule of one GPU's share of a memgraph: every op names the
earlier ops it depends on, the library assigns the ops to lanes (CUDA streams) joined by
events and launches the whole schedule without returning to the host, or replays it as
one CUDA graph.  It stands where the reference has make_gpu_exec_graph and
exec_state_t::event_loop (src/engine/gpu/exec_graph.cc:37-256,
src/engine/exec_state.cc:110-219).
"""
import ctypes
import json

from . import _lib
from .einsummable import CASTABLE_CODE
from .kernel_manager import _ptr, _stream, scalar_bytes
from .scalarop import DTYPE_CODE


def _deps(deps):
    deps = sorted(set(int(d) for d in deps))
    arr = (ctypes.c_int * max(len(deps), 1))(*deps)
    return arr, len(deps)


class program_t:
    def __init__(self, km=None):
        """km: the kernel_manager_t of the device, or None for a schedule that is only
        inspected (describe) and never launched."""
        self._lib = _lib.load()
        self.km = km
        p = ctypes.c_void_p()
        _lib.check(self._lib.es_b200_program_create(km._h if km is not None else None, ctypes.byref(p)))
        self._p = p
        self.n_ops = 0
        self.workspace_bytes = None
        self._keep = []

    def close(self):
        if getattr(self, "_p", None):
            self._lib.es_b200_program_destroy(self._p)
            self._p = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _added(self, idx):
        self.n_ops += 1
        return idx.value

    def add_einsummable(self, kernel_id, out, inns, deps=()):
        arr = (ctypes.c_void_p * max(len(inns), 1))(*[_ptr(x) for x in inns])
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_einsummable(
            self._p, int(kernel_id), _ptr(out), arr, len(inns), d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_touch(self, t, castable, out, inn, deps=(), done_flag=None):
        """done_flag given: `inn` is peer-mapped memory (a move consumed in place); the last CTA
        raises the flag in the source rank's memory once the input has been read."""
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        if done_flag is not None:
            _lib.check(self._lib.es_b200_program_add_remote_touch(
                self._p, t.c_dims(), len(t.selection), CASTABLE_CODE[castable], DTYPE_CODE[t.dtype],
                _ptr(out), _ptr(inn), int(done_flag), d, nd, ctypes.byref(idx)))
            return self._added(idx)
        _lib.check(self._lib.es_b200_program_add_touch(
            self._p, t.c_dims(), len(t.selection), CASTABLE_CODE[castable], DTYPE_CODE[t.dtype],
            _ptr(out), _ptr(inn), d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_touch_batch(self, touches, castables, outs, inns, deps=()):
        n = len(touches)
        items = (_lib.es_touch_item_t * n)()
        for i, t in enumerate(touches):
            if t.dtype != touches[0].dtype:
                raise ValueError("touch batch: mixed dtypes")
            for j, s in enumerate(t.selection):
                items[i].dims[j] = _lib.es_touchdim_t(*s.astuple())
            items[i].rank = len(t.selection)
            items[i].castable = CASTABLE_CODE[castables[i]]
            items[i].out = _ptr(outs[i])
            items[i].inn = _ptr(inns[i])
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_touch_batch(
            self._p, items, n, DTYPE_CODE[touches[0].dtype], d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_fill_constant(self, c, out, deps=()):
        n = 1
        for s in c.shape:
            n *= s
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_fill_constant(
            self._p, DTYPE_CODE[c.dtype], scalar_bytes(c.value, c.dtype), n, _ptr(out), d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_fill_lowertri(self, l, out, deps=()):
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_fill_lowertri(
            self._p, DTYPE_CODE[l.dtype], scalar_bytes(l.lower, l.dtype), scalar_bytes(l.upper, l.dtype),
            l.nrow, l.ncol, l.start, _ptr(out), d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_attention(self, desc, out, q, k, v, mask, deps=()):
        """The fused attention chain as one op (desc: attention_t)."""
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        c = desc.c_struct()
        _lib.check(self._lib.es_b200_program_add_attention(
            self._p, ctypes.byref(c), _ptr(out), _ptr(q), _ptr(k), _ptr(v),
            _ptr(mask) if mask is not None else None, d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_copy(self, src, dst, nbytes, deps=()):
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_copy(self._p, _ptr(src), _ptr(dst), int(nbytes), d, nd,
                                                      ctypes.byref(idx)))
        return self._added(idx)

    def add_evict(self, dev_src, host_dst, nbytes, deps=()):
        """evict_t: device memory -> the storage id's (pinned) host block."""
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_evict(self._p, _ptr(dev_src), _ptr(host_dst), int(nbytes), d, nd,
                                                       ctypes.byref(idx)))
        return self._added(idx)

    def add_load(self, host_src, dev_dst, nbytes, deps=()):
        """load_t: the storage id's host block -> device memory."""
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_load(self._p, _ptr(host_src), _ptr(dev_dst), int(nbytes), d, nd,
                                                      ctypes.byref(idx)))
        return self._added(idx)

    def _flag_op(self, fn, flags, deps):
        arr = (ctypes.c_void_p * len(flags))(*[int(f) for f in flags])
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(fn(self._p, arr, len(flags), d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def add_signal(self, flags, deps=()):
        """Raises the flags (peer memory) to this run's number once `deps` have finished."""
        return self._flag_op(self._lib.es_b200_program_add_signal, flags, deps)

    def add_wait(self, flags, deps=()):
        """Waits (bounded) until every local flag has reached this run's number."""
        return self._flag_op(self._lib.es_b200_program_add_wait, flags, deps)

    def add_pull(self, items, deps=()):
        """items: (src, dst, nbytes, ready_flag or None, done_flag) per move; one launch for all."""
        arr = (_lib.es_pull_item_t * len(items))()
        for i, (src, dst, nbytes, ready, done) in enumerate(items):
            arr[i] = _lib.es_pull_item_t(int(src), int(dst), int(nbytes), int(ready) if ready else None, int(done))
        d, nd = _deps(deps)
        idx = ctypes.c_int(-1)
        _lib.check(self._lib.es_b200_program_add_pull(self._p, arr, len(items), d, nd, ctypes.byref(idx)))
        return self._added(idx)

    def finalize(self, max_lanes=0):
        ws = ctypes.c_uint64(0)
        _lib.check(self._lib.es_b200_program_finalize(self._p, int(max_lanes), ctypes.byref(ws)))
        self.workspace_bytes = ws.value
        return ws.value

    def set_workspace(self, workspace, nbytes):
        self._keep.append(workspace)
        _lib.check(self._lib.es_b200_program_set_workspace(self._p, _ptr(workspace), int(nbytes)))

    def set_exchange_lanes(self, lanes):
        """Before finalize: the number of lanes the pull / wait ops share (1..4, default 1)."""
        _lib.check(self._lib.es_b200_program_set_exchange_lanes(self._p, int(lanes)))

    def set_wait_limit(self, limit_ms):
        _lib.check(self._lib.es_b200_program_set_wait_limit(self._p, int(limit_ms)))

    def launch(self, stream=None):
        _lib.check(self._lib.es_b200_program_launch(self._p, _stream(stream)))

    def launch_timed(self, stream=None):
        """One run with an event pair around every op; returns milliseconds per op."""
        ms = (ctypes.c_float * max(self.n_ops, 1))()
        _lib.check(self._lib.es_b200_program_launch_timed(self._p, _stream(stream), ms, self.n_ops))
        return list(ms[:self.n_ops])

    def instantiate(self):
        _lib.check(self._lib.es_b200_program_instantiate(self._p))

    def replay(self, stream=None):
        _lib.check(self._lib.es_b200_program_replay(self._p, _stream(stream)))

    def replay_timed(self, stream=None):
        """One replay with the GPU's nanosecond timer read before and after every op: returns
        ([(start_ns, end_ns) per op], (run_begin_ns, run_end_ns))."""
        n = 2 * self.n_ops + 2
        ns = (ctypes.c_ulonglong * n)()
        _lib.check(self._lib.es_b200_program_replay_timed(self._p, _stream(stream), ns, n))
        return [(ns[2 * i], ns[2 * i + 1]) for i in range(self.n_ops)], (ns[n - 2], ns[n - 1])

    def reset_epoch(self):
        _lib.check(self._lib.es_b200_program_reset_epoch(self._p))

    def describe(self):
        need = ctypes.c_int(0)
        _lib.check(self._lib.es_b200_program_describe(self._p, None, 0, ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        _lib.check(self._lib.es_b200_program_describe(self._p, buf, need.value, None))
        return json.loads(buf.value.decode())
