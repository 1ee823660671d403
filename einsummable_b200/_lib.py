"""ctypes binding of libes_b200.so (the C ABI declared in include/es_b200.h)."""
import ctypes
import os

ES_MAX_RANK = 12
ES_MAX_INNS = 8

ES_OK, ES_NOT_SUPPORTED, ES_BAD_DESCRIPTOR, ES_WORKSPACE_TOO_SMALL = 0, 1, 2, 3
ES_CUDA_ERROR, ES_NOT_BUILT, ES_BAD_ARGUMENT, ES_COMPILE_ERROR = 4, 5, 6, 7

STATUS_NAMES = {
    0: "ES_OK", 1: "ES_NOT_SUPPORTED", 2: "ES_BAD_DESCRIPTOR", 3: "ES_WORKSPACE_TOO_SMALL",
    4: "ES_CUDA_ERROR", 5: "ES_NOT_BUILT", 6: "ES_BAD_ARGUMENT", 7: "ES_COMPILE_ERROR",
}


class es_einsummable_desc_t(ctypes.Structure):
    _fields_ = [
        ("join_rank", ctypes.c_int32),
        ("join_shape", ctypes.c_uint64 * ES_MAX_RANK),
        ("n_inn", ctypes.c_int32),
        ("inn_rank", ctypes.c_int32 * ES_MAX_INNS),
        ("inn_modes", (ctypes.c_int32 * ES_MAX_RANK) * ES_MAX_INNS),
        ("out_rank", ctypes.c_int32),
        ("castable", ctypes.c_int32),
        ("join", ctypes.c_char_p),
    ]


class es_touchdim_t(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in ("d_inn", "d_out", "offset_inn", "offset_out", "size")]


class es_touch_item_t(ctypes.Structure):
    _fields_ = [
        ("dims", es_touchdim_t * 4),
        ("rank", ctypes.c_int32),
        ("castable", ctypes.c_int32),
        ("out", ctypes.c_void_p),
        ("inn", ctypes.c_void_p),
    ]


class es_touch_batch_t(ctypes.Structure):
    _fields_ = [("n", ctypes.c_int32), ("dtype", ctypes.c_int32), ("width", ctypes.c_int32),
                ("pad", ctypes.c_int32), ("max_slots", ctypes.c_uint64), ("items_dev", ctypes.c_void_p)]


class es_pull_item_t(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("bytes", ctypes.c_uint64),
                ("ready_flag", ctypes.c_void_p), ("done_flag", ctypes.c_void_p)]


class es_attention_t(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_uint32), ("heads", ctypes.c_uint32), ("rows", ctypes.c_uint32),
                ("keys", ctypes.c_uint32), ("head_dim", ctypes.c_uint32), ("skip_known", ctypes.c_int32),
                ("skip_from", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3),
                ("v_stride", ctypes.c_int64 * 3), ("out_stride", ctypes.c_int64 * 3),
                ("mask_stride", ctypes.c_int64)]


LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libes_b200.so")

# every symbol include/es_b200.h declares: name -> (restype, argtypes)
_vp, _u64, _i, _cp = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_char_p
_desc_p = ctypes.POINTER(es_einsummable_desc_t)
_td_p = ctypes.POINTER(es_touchdim_t)
_ip = ctypes.POINTER(ctypes.c_int)
SYMBOLS = {
    "es_b200_create": (_i, [_i, ctypes.POINTER(_vp)]),
    "es_b200_destroy": (_i, [_vp]),
    "es_b200_set_f32_policy": (_i, [_vp, _i]),
    "es_b200_build_einsummable": (_i, [_vp, _desc_p, ctypes.POINTER(_u64), ctypes.POINTER(_u64)]),
    "es_b200_workspace_size": (_i, [_vp, _u64, ctypes.POINTER(_u64)]),
    "es_b200_launch_einsummable": (_i, [_vp, _u64, _vp, _vp, ctypes.POINTER(_vp), _i, _vp, _u64]),
    "es_b200_launch_touch": (_i, [_vp, _td_p, _i, _i, _i, _vp, _vp, _vp]),
    "es_b200_launch_touch_batch": (_i, [_vp, ctypes.POINTER(es_touch_item_t), _i, _i, _vp, _vp]),
    "es_b200_prepare_touch_batch": (_i, [_vp, ctypes.POINTER(es_touch_item_t), _i, _i, _vp, _vp,
                                         ctypes.POINTER(es_touch_batch_t)]),
    "es_b200_launch_prepared_touch_batch": (_i, [_vp, ctypes.POINTER(es_touch_batch_t), _vp]),
    "es_b200_debug_trace": (_i, [_vp, ctypes.POINTER(ctypes.c_ulonglong), _i, ctypes.POINTER(_i)]),
    "es_b200_fill_constant": (_i, [_vp, _i, _vp, _u64, _vp, _vp]),
    "es_b200_fill_lowertri": (_i, [_vp, _i, _vp, _vp, _u64, _u64, ctypes.c_int64, _vp, _vp]),
    "es_b200_move": (_i, [_vp, _i, _vp, _i, _vp, _u64, _vp]),
    "es_b200_flag_signal": (_i, [_vp, _vp, ctypes.c_uint32, _vp]),
    "es_b200_flag_wait": (_i, [_vp, _vp, ctypes.c_uint32, _vp]),
    "es_b200_pull": (_i, [_vp, _vp, _vp, _u64, _vp]),
    "es_b200_launch_attention": (_i, [_vp, ctypes.POINTER(es_attention_t), _vp, _vp, _vp, _vp, _vp, _vp]),
    "es_b200_kernel_info": (_i, [_vp, _u64, _cp, _i]),
    "es_b200_describe": (_i, [_desc_p, _i, _cp, _i]),
    "es_b200_touch_simplify": (_i, [_td_p, _i, _td_p, ctypes.POINTER(_i)]),
    "es_b200_rowsum_f32_noalloc": (_i, [_vp, _vp, _vp, _u64, _u64, _vp]),
    "es_b200_device_status": (_i, [_vp, ctypes.POINTER(ctypes.c_uint)]),
    "es_b200_query_counters": (_i, [_vp, ctypes.POINTER(_u64)]),
    "es_b200_query_work": (_i, [_vp, ctypes.POINTER(_u64), ctypes.POINTER(_u64)]),
    "es_b200_program_create": (_i, [_vp, ctypes.POINTER(_vp)]),
    "es_b200_program_destroy": (_i, [_vp]),
    "es_b200_program_add_einsummable": (_i, [_vp, _u64, _vp, ctypes.POINTER(_vp), _i, _ip, _i, _ip]),
    "es_b200_program_add_touch": (_i, [_vp, _td_p, _i, _i, _i, _vp, _vp, _ip, _i, _ip]),
    "es_b200_program_add_remote_touch": (_i, [_vp, _td_p, _i, _i, _i, _vp, _vp, _vp, _ip, _i, _ip]),
    "es_b200_program_add_touch_batch": (_i, [_vp, ctypes.POINTER(es_touch_item_t), _i, _i, _ip, _i, _ip]),
    "es_b200_program_add_fill_constant": (_i, [_vp, _i, _vp, _u64, _vp, _ip, _i, _ip]),
    "es_b200_program_add_fill_lowertri": (_i, [_vp, _i, _vp, _vp, _u64, _u64, ctypes.c_int64, _vp, _ip, _i, _ip]),
    "es_b200_program_add_copy": (_i, [_vp, _vp, _vp, _u64, _ip, _i, _ip]),
    "es_b200_program_add_evict": (_i, [_vp, _vp, _vp, _u64, _ip, _i, _ip]),
    "es_b200_program_add_load": (_i, [_vp, _vp, _vp, _u64, _ip, _i, _ip]),
    "es_b200_storage_create": (_i, [_u64, _i, ctypes.POINTER(_vp)]),
    "es_b200_storage_destroy": (_i, [_vp]),
    "es_b200_storage_write": (_i, [_vp, _i, _vp, _u64]),
    "es_b200_storage_read": (_i, [_vp, _i, _vp, _u64]),
    "es_b200_storage_remove": (_i, [_vp, _i]),
    "es_b200_storage_reference": (_i, [_vp, _i, ctypes.POINTER(_vp), ctypes.POINTER(_u64)]),
    "es_b200_evict": (_i, [_vp, _vp, _i, _vp, _u64, _vp]),
    "es_b200_load": (_i, [_vp, _vp, _i, _vp, _u64, _vp]),
    "es_b200_program_add_signal": (_i, [_vp, ctypes.POINTER(_vp), _i, _ip, _i, _ip]),
    "es_b200_program_add_attention": (_i, [_vp, ctypes.POINTER(es_attention_t), _vp, _vp, _vp, _vp, _vp, _ip, _i, _ip]),
    "es_b200_program_add_pull": (_i, [_vp, ctypes.POINTER(es_pull_item_t), _i, _ip, _i, _ip]),
    "es_b200_program_add_wait": (_i, [_vp, ctypes.POINTER(_vp), _i, _ip, _i, _ip]),
    "es_b200_program_finalize": (_i, [_vp, _i, ctypes.POINTER(_u64)]),
    "es_b200_program_set_workspace": (_i, [_vp, _vp, _u64]),
    "es_b200_program_set_wait_limit": (_i, [_vp, ctypes.c_uint32]),
    "es_b200_program_set_exchange_lanes": (_i, [_vp, _i]),
    "es_b200_program_launch": (_i, [_vp, _vp]),
    "es_b200_program_launch_timed": (_i, [_vp, _vp, ctypes.POINTER(ctypes.c_float), _i]),
    "es_b200_program_instantiate": (_i, [_vp]),
    "es_b200_program_replay": (_i, [_vp, _vp]),
    "es_b200_program_replay_timed": (_i, [_vp, _vp, ctypes.POINTER(ctypes.c_ulonglong), _i]),
    "es_b200_program_reset_epoch": (_i, [_vp]),
    "es_b200_program_describe": (_i, [_vp, _cp, _i, _ip]),
    "es_b200_wire_to_json": (_i, [_cp, _vp, _u64, _vp, _u64, ctypes.POINTER(_u64)]),
    "es_b200_wire_from_json": (_i, [_cp, _cp, _vp, _u64, ctypes.POINTER(_u64)]),
    "es_b200_weight_file_list": (_i, [_cp, _vp, _u64, ctypes.POINTER(_u64), _i, ctypes.POINTER(_i)]),
    "es_b200_weight_file_read": (_i, [_cp, _cp, _vp, _u64, ctypes.POINTER(_u64)]),
    "es_b200_weight_file_append": (_i, [_cp, _cp, _vp, _u64]),
    "es_b200_last_error": (_cp, []),
    "es_b200_version": (_cp, []),
}

_lib = None


def load():
    """Loads the library; there is no fallback when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libes_b200.so is not built (%s); run `python -m einsummable_b200.build`" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class es_error(RuntimeError):
    def __init__(self, status, msg):
        RuntimeError.__init__(self, "%s: %s" % (STATUS_NAMES.get(status, status), msg))
        self.status = status


def check(status):
    if status != ES_OK:
        raise es_error(status, load().es_b200_last_error().decode(errors="replace"))
