"""``BufferObject``: a checkpoint object as a shared file mapping that CUDA can address.

Same surface as the reference's compiled class of this name and module path
(checkpoint_object_manager/buffer_object/bindings.cpp:27-100): two constructor forms, ``close``,
``resize``, ``get_id``, ``get_capacity``, ``get_data_ptr``, ``closed``, ``is_readonly`` and a 1-D
``uint8`` buffer protocol that honours read-only mappings. The implementation lives behind the
``mlf_buf_*`` entry points of ``libmlf_b200.so``; this class only binds them.

Beyond the reference: ``register_cuda`` page-locks the mapping and maps it into the CUDA address
space so kernels and copy engines can write checkpoint bytes into it, and ``get_device_ptr``
returns the device-visible address. The native layer drops and re-establishes the registration
around every ``resize`` and drops it on ``close``.
"""

from __future__ import annotations

import ctypes
from typing import Optional

from ml_flashpoint import _native


class BufferObject:
    def __init__(self, object_id: str, capacity: Optional[int] = None, overwrite: bool = False):
        self._handle = ctypes.c_void_p()
        lib = _native.lib()
        path = str(object_id).encode()
        if capacity is None:
            rc = lib.mlf_buf_open_ro(path, ctypes.byref(self._handle))
        else:
            if capacity < 0:
                raise RuntimeError(f"a buffer needs a capacity greater than 0: {object_id}")
            rc = lib.mlf_buf_create(path, int(capacity), 1 if overwrite else 0, ctypes.byref(self._handle))
        if rc < 0:
            self._handle = ctypes.c_void_p()
            raise RuntimeError(_native.last_error())

    # ------------------------------------------------------------------ reference surface
    def close(self, truncate_size: Optional[int] = None) -> None:
        """Unmaps and closes the file, truncating it first if ``truncate_size`` is given. Never raises."""
        if self._handle:
            _native.lib().mlf_buf_close(self._handle, -1 if truncate_size is None else int(truncate_size))

    def get_id(self) -> str:
        return _native.lib().mlf_buf_id(self._handle).decode()

    def get_capacity(self) -> int:
        return int(_native.lib().mlf_buf_capacity(self._handle))

    def resize(self, new_capacity: int) -> None:
        rc = _native.lib().mlf_buf_resize(self._handle, int(new_capacity))
        if rc < 0:
            raise RuntimeError(_native.last_error())

    def get_data_ptr(self) -> int:
        if self.closed:
            raise RuntimeError("Buffer is closed: cannot access data pointer.")
        return int(_native.lib().mlf_buf_host_ptr(self._handle) or 0)

    @property
    def closed(self) -> bool:
        return (not self._handle) or bool(_native.lib().mlf_buf_is_closed(self._handle))

    @property
    def is_readonly(self) -> bool:
        return bool(_native.lib().mlf_buf_is_readonly(self._handle))

    def __buffer__(self, flags: int) -> memoryview:
        if self.closed:
            message = "Cannot create buffer view on a closed BufferObject"
            raise BufferError(message) from RuntimeError(message)
        raw = (ctypes.c_ubyte * self.get_capacity()).from_address(self.get_data_ptr())
        view = memoryview(raw).cast("B")
        return view.toreadonly() if self.is_readonly else view

    # ------------------------------------------------------------------ CUDA registration
    def register_cuda(self) -> None:
        """Page-locks the mapping and maps it for the current CUDA device (idempotent)."""
        _native.check(_native.lib().mlf_buf_register(self._handle))

    def unregister_cuda(self) -> None:
        _native.check(_native.lib().mlf_buf_unregister(self._handle))

    @property
    def is_cuda_registered(self) -> bool:
        return bool(self._handle) and bool(_native.lib().mlf_buf_is_registered(self._handle))

    def get_device_ptr(self) -> int:
        """Device-visible address of byte 0; the mapping must be registered."""
        out = ctypes.c_void_p()
        _native.check(_native.lib().mlf_buf_dev_ptr(self._handle, ctypes.byref(out)))
        return int(out.value or 0)

    def read_to_device(self, offset: int, device_ptr: int, nbytes: int, threads: int = 0, lock_run_mib: int = 0) -> int:
        """Blocking copy of object bytes ``[offset, offset + nbytes)`` into device memory through the
        page-locked bounce ring, reading the file descriptor rather than the mapping. With
        ``lock_run_mib`` > 0 a lock lane works beside the ring's threads: it page-locks that many MiB
        of the file at a time and lets a copy engine read them in place. Returns the bytes the lane
        moved (0 without one)."""
        _native.check(
            _native.lib().mlf_buf_read_to_device_hybrid(
                self._handle, int(offset), ctypes.c_void_p(device_ptr), int(nbytes), int(threads), int(lock_run_mib)
            )
        )
        return int(_native.lib().mlf_last_lock_lane_bytes()) if lock_run_mib > 0 else 0

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                _native.lib().mlf_buf_destroy(handle)
            except Exception:
                pass
