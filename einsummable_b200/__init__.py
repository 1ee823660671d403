"""B200-native kernel layer for einsummable's memgraph apply nodes.

The product is the C ABI in include/es_b200.h (libes_b200.so: hand-written and
generated sm_100a kernels).  This package is the thin host-side mirror of the
reference's kernel-manager interface on top of it.
"""
from . import _lib
from ._lib import es_error
from .einsummable import einsummable_t, fill_t, touch_t, touchdim_t
from .kernel_manager import kernel_manager_t, scalar_bytes
from .scalarop import DTYPE_CODE, DTYPE_SIZE, scalarop_t, default_dtype, set_default_dtype

__all__ = [
    "einsummable_t", "touch_t", "touchdim_t", "fill_t", "scalarop_t", "kernel_manager_t",
    "es_error", "default_dtype", "set_default_dtype", "scalar_bytes", "DTYPE_CODE", "DTYPE_SIZE",
]
