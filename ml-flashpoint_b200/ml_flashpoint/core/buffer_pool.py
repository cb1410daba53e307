"""Pool of persistent, pre-sized buffer files reused from checkpoint to checkpoint.

Same contract as the reference's core/buffer_pool.py:35-342: ``num_buffers`` files
``buffer_<rank>_<idx>.dist`` are created up front; ``acquire`` hands one out and plants a symlink
at the object's path; a buffer becomes free again once that symlink no longer resolves (the
checkpoint was deleted); clients never really close a pooled buffer, closing only trims it to the
written size. New here: with ``register_cuda`` the pool page-locks each file when it is created
(the expensive part of a GPU save, paid once, off the save path), and trimming keeps the
registration alive through the native resize.
"""

import logging
import os
import threading
from dataclasses import dataclass
from typing import Dict, List, Optional

from ml_flashpoint.checkpoint_object_manager.buffer_io import BufferIO
from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE
from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)

PADDING_SIZE = 1024 * 1024
RESIZE_FACTOR = 1.1


class PooledBufferIO:
    """Client-side handle of a pooled ``BufferIO``: forwards everything, but never closes it."""

    def __init__(self, buffer_io: BufferIO):
        self._buffer_io = buffer_io
        self._closed = False

    def __getattr__(self, name):
        if self._closed:
            _LOGGER.warning("PooledBufferIO: Accessing closed buffer")
        return getattr(self._buffer_io, name)

    @log_execution_time(logger=_LOGGER, name="close", level=logging.INFO)
    def close(self, truncate: bool = True):
        """Releases the handle. The file stays open for reuse; it is trimmed to the written size."""
        if self._closed:
            return
        self._closed = True
        inner = self._buffer_io
        if not truncate or inner.is_readonly:
            return
        try:
            wanted = METADATA_SIZE + inner._metadata.len_written_data
            if wanted != len(inner._mv):
                _LOGGER.debug("PooledBufferIO: Truncating reusable buffer from %d to %d bytes", len(inner._mv), wanted)
                inner.resize(wanted)
        except Exception:
            _LOGGER.warning("PooledBufferIO: Failed to truncate buffer during close.", exc_info=True)

    @property
    def closed(self) -> bool:
        return self._closed or self._buffer_io.closed

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()

    def _auto_resize(self, required_bytes: int):
        """Grows the file so that ``required_bytes`` more fit at the cursor: 10 % or 1 MiB headroom."""
        now = self._buffer_io.buffer_obj.get_capacity()
        need = METADATA_SIZE + self._buffer_io.tell() + required_bytes
        grown = int(max(now * RESIZE_FACTOR, need + PADDING_SIZE))
        _LOGGER.debug("PooledBufferIO: Auto-resizing from %d to %d bytes (required: %d)", now, grown, need)
        self._buffer_io.resize(grown)

    def _ensure_room(self, nbytes: int) -> None:
        if METADATA_SIZE + self._buffer_io.tell() + nbytes > self._buffer_io.buffer_obj.get_capacity():
            self._auto_resize(nbytes)

    def write(self, data: bytes) -> int:
        self._ensure_room(len(data))
        return self._buffer_io.write(data)

    def next_buffer_slice(self, size: int) -> memoryview:
        self._ensure_room(size)
        return self._buffer_io.next_buffer_slice(size)

    def ensure_total_size(self, total_bytes: int) -> None:
        """Sizes the file to exactly ``total_bytes`` if it differs (one remap instead of grow + trim)."""
        if self._buffer_io.buffer_obj.get_capacity() != total_bytes:
            self._buffer_io.resize(total_bytes)


@dataclass
class BufferPoolConfig:
    pool_dir_path: str
    rank: int
    num_buffers: int
    buffer_size: int
    register_cuda: bool = False

    def __post_init__(self):
        if not self.pool_dir_path:
            raise ValueError("pool_dir_path must be provided in BufferPoolConfig")
        for field in ("rank", "num_buffers", "buffer_size"):
            value = getattr(self, field)
            if not isinstance(value, int) or value < 0:
                raise ValueError(f"{field} must be a non-negative integer in BufferPoolConfig")


class BufferPool:
    def __init__(
        self,
        pool_dir_path: str,
        rank: int = 0,
        num_buffers: int = 3,
        buffer_size: int = 0,
        register_cuda: bool = False,
    ):
        if num_buffers <= 0:
            raise ValueError(f"Number of buffers must be positive. Got {num_buffers}.")
        if buffer_size <= 0:
            raise ValueError(f"Buffer size must be positive. Got {buffer_size}.")
        if not pool_dir_path:
            raise ValueError("Pool directory path must be provided.")
        self.pool_dir = pool_dir_path
        self.rank = rank
        self.num_buffers = num_buffers
        self.buffer_size = buffer_size
        self.register_cuda = register_cuda
        self.free_buffers: List[BufferIO] = []
        # pool file path -> (its BufferIO, the symlink that keeps it in use)
        self.active_buffers: Dict[str, tuple[BufferIO, str]] = {}
        self._lock = threading.Lock()
        try:
            os.makedirs(self.pool_dir, exist_ok=True)
            self._preallocate_buffers()
        except OSError:
            _LOGGER.exception("Failed to create/populate BufferPool.")
            raise

    @log_execution_time(logger=_LOGGER, name="acquire", level=logging.INFO)
    def acquire(self, associated_symlink: Optional[str] = None) -> PooledBufferIO:
        """Hands out a free buffer, linked from ``associated_symlink``; ``RuntimeError`` if none is free."""
        with self._lock:
            self._gc()
            if not self.free_buffers:
                raise RuntimeError(f"BufferPool exhausted. All {self.num_buffers} buffers are in use.")
            candidate = self.free_buffers.pop()
            try:
                return PooledBufferIO(self._reuse_buffer(candidate, associated_symlink))
            except Exception:
                _LOGGER.exception("Failed to reuse buffer for '%s'. Releasing buffer.", associated_symlink)
                self.active_buffers.pop(candidate.buffer_obj.get_id(), None)
                self.free_buffers.append(candidate)
                raise

    def relink(self, buffer_io, old_symlink: str, new_symlink: str) -> None:
        """Renames the link that keeps ``buffer_io`` in use and records the new name, atomically with
        respect to garbage collection (objects received from a peer are written under a temporary
        name and renamed when complete)."""
        inner = getattr(buffer_io, "_buffer_io", buffer_io)
        path = inner.buffer_obj.get_id()
        with self._lock:
            os.rename(old_symlink, new_symlink)
            if path in self.active_buffers:
                self.active_buffers[path] = (inner, new_symlink)

    def _gc(self) -> None:
        """Frees every active buffer whose symlink is gone or dangling."""
        # exists(), not lexists(): a link whose target vanished counts as gone too
        dead = [path for path, (_, link) in self.active_buffers.items() if link and not os.path.exists(link)]
        for path in dead:
            _LOGGER.debug("Garbage collecting buffer %s", path)
            buf, _ = self.active_buffers.pop(path)
            self.free_buffers.append(buf)

    def teardown(self) -> None:
        """Closes every buffer. The files stay on disk."""
        with self._lock:
            for buf in self.free_buffers + [b for b, _ in self.active_buffers.values()]:
                try:
                    buf.close(truncate=True)
                except Exception:
                    _LOGGER.warning("PooledBufferIO: Failed to close buffer during teardown.", exc_info=True)
            self.free_buffers.clear()
            self.active_buffers.clear()

    @log_execution_time(logger=_LOGGER, name="_reuse_buffer", level=logging.INFO)
    def _reuse_buffer(self, buffer_io: BufferIO, symlink: Optional[str]) -> BufferIO:
        buffer_io.seek(0)
        buffer_io._metadata.len_written_data = 0
        path = buffer_io.buffer_obj.get_id()
        self.active_buffers[path] = (buffer_io, symlink)
        if symlink:
            os.symlink(path, symlink)
        return buffer_io

    def _preallocate_buffers(self) -> None:
        for idx in range(self.num_buffers):
            path = os.path.join(self.pool_dir, f"buffer_{self.rank}_{idx}.dist")
            try:
                _LOGGER.debug("Pre-allocating buffer: %s with size %d", path, self.buffer_size)
                obj = BufferObject(path, self.buffer_size, overwrite=True)
                if self.register_cuda:
                    obj.register_cuda()
                self.free_buffers.append(BufferIO(obj))
            except Exception:
                _LOGGER.exception("Failed to pre-allocate buffer %s", path)
                raise
