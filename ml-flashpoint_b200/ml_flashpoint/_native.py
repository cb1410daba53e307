"""ctypes binding of ``libmlf_b200.so``, the C ABI declared in ``include/mlf_b200.h``.

There is exactly one data path and it is native: if the library is missing, loading fails with
an error that says how to build it. Nothing here falls back to a Python or CPU implementation.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_uint8, c_uint32, c_uint64, c_void_p

MLF_OK = 0
MLF_ERR_INVALID = -1
MLF_ERR_IO = -2
MLF_ERR_CUDA = -3
MLF_ERR_BOUNDS = -4
MLF_ERR_CLOSED = -5
MLF_ERR_EXISTS = -6
MLF_ERR_TIMEOUT = -7
MLF_ERR_TOO_LARGE = -8
MLF_ERR_READONLY = -9

MLF_MAX_DIMS = 8
MLF_PACK = 0
MLF_UNPACK = 1
MLF_COPY_D2H = 0
MLF_COPY_H2D = 1
MLF_COPY_D2D = 2
MLF_IPC_HANDLE_BYTES = 64
MLF_NOALLOC_MAX_DESCS = 1024

LIB_NAME = "libmlf_b200.so"
# MLF_B200_LIB selects another build of the same library (tuning variants); default is the in-tree one
LIB_PATH = os.environ.get("MLF_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


class NativeError(RuntimeError):
    """A C-ABI call returned a negative status. ``code`` holds the ``MLF_ERR_*`` value."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class CopyDesc(ctypes.Structure):
    """Mirror of ``mlf_copy_desc``."""

    _fields_ = [
        ("tensor_ptr", c_uint64),
        ("image_off", c_uint64),
        ("elem_size", c_uint32),
        ("ndim", c_uint32),
        ("shape", c_int64 * MLF_MAX_DIMS),
        ("tensor_stride", c_int64 * MLF_MAX_DIMS),
        ("image_stride", c_int64 * MLF_MAX_DIMS),
    ]


_SIGNATURES = {
    # name: (restype, argtypes)
    "mlf_last_error": (c_char_p, []),
    "mlf_version": (c_char_p, []),
    "mlf_launch_count": (c_uint64, []),
    "mlf_selftest_wait_timeout": (c_int32, [c_uint64, c_void_p]),
    "mlf_buf_create": (c_int32, [c_char_p, c_uint64, c_int32, POINTER(c_void_p)]),
    "mlf_buf_open_ro": (c_int32, [c_char_p, POINTER(c_void_p)]),
    "mlf_buf_resize": (c_int32, [c_void_p, c_uint64]),
    "mlf_buf_close": (c_int32, [c_void_p, c_int64]),
    "mlf_buf_destroy": (None, [c_void_p]),
    "mlf_buf_id": (c_char_p, [c_void_p]),
    "mlf_buf_capacity": (c_uint64, [c_void_p]),
    "mlf_buf_host_ptr": (c_void_p, [c_void_p]),
    "mlf_buf_is_closed": (c_int32, [c_void_p]),
    "mlf_buf_is_readonly": (c_int32, [c_void_p]),
    "mlf_buf_register": (c_int32, [c_void_p]),
    "mlf_buf_unregister": (c_int32, [c_void_p]),
    "mlf_buf_is_registered": (c_int32, [c_void_p]),
    "mlf_buf_read_to_device": (c_int32, [c_void_p, c_uint64, c_void_p, c_uint64, c_int32]),
    "mlf_buf_read_to_device_hybrid": (c_int32, [c_void_p, c_uint64, c_void_p, c_uint64, c_int32, c_int32]),
    "mlf_last_lock_lane_bytes": (c_uint64, []),
    "mlf_buf_dev_ptr": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "mlf_plan_create": (c_int32, [POINTER(CopyDesc), c_uint64, c_int32, POINTER(c_void_p)]),
    "mlf_plan_destroy": (None, [c_void_p]),
    "mlf_plan_image_extent": (c_uint64, [c_void_p]),
    "mlf_plan_payload_bytes": (c_uint64, [c_void_p]),
    "mlf_plan_num_tiles": (c_uint64, [c_void_p]),
    "mlf_plan_launch": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p, c_int32]),
    "mlf_plan_status": (c_int32, [c_void_p]),
    "mlf_pack_noalloc": (c_int32, [POINTER(CopyDesc), c_uint64, c_void_p, c_uint64, c_void_p]),
    "mlf_memcpy_async": (c_int32, [c_void_p, c_void_p, c_uint64, c_int32, c_void_p]),
    "mlf_bounce_copy": (c_int32, [c_void_p, c_void_p, c_uint64, c_int32, c_int32]),
    "mlf_copy_kernel_launch": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p, c_int32]),
    "mlf_dev_alloc": (c_int32, [c_uint64, POINTER(c_void_p)]),
    "mlf_dev_free": (c_int32, [c_void_p]),
    "mlf_host_alloc": (c_int32, [c_uint64, POINTER(c_void_p)]),
    "mlf_host_free": (c_int32, [c_void_p]),
    "mlf_ipc_export": (c_int32, [c_void_p, POINTER(c_uint8)]),
    "mlf_ipc_open": (c_int32, [POINTER(c_uint8), POINTER(c_void_p)]),
    "mlf_ipc_close": (c_int32, [c_void_p]),
    "mlf_enable_peer_access": (c_int32, [c_int32]),
    "mlf_set_device": (c_int32, [c_int32]),
    "mlf_get_device": (c_int32, [POINTER(c_int32)]),
    "mlf_device_sm_count": (c_int32, [POINTER(c_int32)]),
    "mlf_stream_create": (c_int32, [POINTER(c_void_p)]),
    "mlf_stream_destroy": (c_int32, [c_void_p]),
    "mlf_stream_sync": (c_int32, [c_void_p]),
    "mlf_stream_wait_event": (c_int32, [c_void_p, c_void_p]),
    "mlf_event_create": (c_int32, [POINTER(c_void_p)]),
    "mlf_event_destroy": (c_int32, [c_void_p]),
    "mlf_event_record": (c_int32, [c_void_p, c_void_p]),
    "mlf_event_sync": (c_int32, [c_void_p]),
    "mlf_event_query": (c_int32, [c_void_p]),
    "mlf_event_elapsed_ms": (c_int32, [c_void_p, c_void_p, POINTER(c_float)]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None
_lib_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """The loaded library. Raises ``ImportError`` with build instructions if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_NAME} is missing at {LIB_PATH}. Build it with "
                    "`python ml-flashpoint_b200/build_native.py`; this package has no other data path."
                )
            loaded = ctypes.CDLL(LIB_PATH)
            for name, (restype, argtypes) in _SIGNATURES.items():
                fn = getattr(loaded, name)
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = loaded
    return _lib


def last_error() -> str:
    return lib().mlf_last_error().decode("utf-8", "replace")


def check(rc: int) -> int:
    """Raises ``NativeError`` for a negative status; passes non-negative values through."""
    if rc < 0:
        raise NativeError(rc, last_error() or f"native call failed with status {rc}")
    return rc
