"""``BufferIO``: a file-like cursor over one checkpoint object.

Call-compatible with the reference's class (checkpoint_object_manager/buffer_io.py:26-530): the
first ``METADATA_SIZE`` bytes of the underlying ``BufferObject`` hold the metadata block, every
position is relative to the byte after it, ``len_written_data`` is a high-water mark, and ``close``
truncates the file to what was written. Added for the GPU path: ``host_address`` /
``device_address`` expose where a stream position lives so that kernels and copy engines can be
pointed at the mapping.
"""

import io
from typing import Optional, Union

from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject
from ml_flashpoint.core.mlf_logging import get_logger

from .buffer_metadata import METADATA_SIZE, BufferMetadataType

_LOGGER = get_logger(__name__)

_READ_OPS = frozenset({"read", "readinto", "seek"})
_WRITE_OPS = _READ_OPS | {"write"}


class BufferIO:
    def __init__(self, buffer_obj: BufferObject):
        if buffer_obj.closed:
            raise ValueError("Cannot initialize BufferIO with a closed BufferObject.")
        self.buffer_obj = buffer_obj
        self._pos: int = 0
        self._mv: Optional[memoryview] = None
        self._metadata: Optional[BufferMetadataType] = None
        self._map_views(first_time=True)

    def _map_views(self, first_time: bool) -> None:
        """(Re)creates the memoryview of the mapping and the metadata struct over its head."""
        try:
            self._mv = memoryview(self.buffer_obj)
        except TypeError:
            raise ValueError("Underlying BufferObject does not support the buffer protocol.")
        except Exception:
            if first_time:
                raise
            raise ValueError("Failed to recreate memoryview after resize.")
        if len(self._mv) < METADATA_SIZE:
            raise ValueError(f"Buffer size must be at least {METADATA_SIZE} bytes.")
        head = self._mv[:METADATA_SIZE]
        try:
            if self.buffer_obj.is_readonly:
                # a read-only mapping cannot back a live ctypes struct: work on a snapshot
                self._metadata = BufferMetadataType.from_buffer_copy(head)
            else:
                self._metadata = BufferMetadataType.from_buffer(head)
        except Exception as e:
            raise IOError(f"Could not initialize metadata from buffer: {e}") from e

    # ------------------------------------------------------------------ state checks
    def _check_validity(self, operation: str = None):
        if self.closed:
            raise ValueError("I/O operation on a closed BufferIO object")
        if operation is None:
            return
        if self.buffer_obj.is_readonly:
            if operation not in _READ_OPS:
                raise TypeError(f"Operation '{operation}' is not supported in read-only mode.")
        elif operation not in _WRITE_OPS:
            raise TypeError(f"Operation '{operation}' is not supported in read-write mode.")

    def _update_written_data_length(self, new_length: int):
        if new_length > self._metadata.len_written_data:
            self._metadata.len_written_data = new_length

    @property
    def closed(self) -> bool:
        return self.buffer_obj is None or self.buffer_obj.closed

    @property
    def is_readonly(self) -> bool:
        self._check_validity()
        return self.buffer_obj.is_readonly

    # ------------------------------------------------------------------ writing
    def write(self, data: bytes) -> int:
        """Copies ``data`` to the cursor; ``ValueError`` if it would pass the end of the mapping."""
        self._check_validity("write")
        n = len(data)
        if n == 0:
            return 0
        begin = METADATA_SIZE + self._pos
        if begin + n > len(self._mv):
            raise ValueError(
                "Write operation exceeds buffer capacity. "
                f"Attempted to write {n} bytes at position {self._pos} "
                f"which would exceed the total capacity of {len(self._mv)}."
            )
        self._mv[begin : begin + n] = data
        self._pos += n
        self._update_written_data_length(self._pos)
        return n

    def next_buffer_slice(self, size: int) -> memoryview:
        """Claims the next ``size`` bytes: returns a writable view of them and moves the cursor past."""
        self._check_validity("write")
        if size < 0:
            raise ValueError(f"Size must be non-negative, got {size}")
        begin = METADATA_SIZE + self._pos
        if begin + size > len(self._mv):
            raise ValueError(
                f"Requested slice (size={size}) exceeds buffer capacity "
                f"(pos={self._pos}, cap={len(self._mv) - METADATA_SIZE})"
            )
        claimed = self._mv[begin : begin + size]
        self._pos += size
        self._update_written_data_length(self._pos)
        return claimed

    def set_format_signature(self, signature: bytes) -> None:
        self._check_validity("write")
        if len(signature) > 8:
            raise ValueError(f"Format signature must be at most 8 bytes, got {len(signature)}")
        self._metadata.format_signature = signature

    # ------------------------------------------------------------------ reading
    def _readable(self, wanted: int) -> int:
        left = self._metadata.len_written_data - self._pos
        if left <= 0:
            return 0
        return left if wanted < 0 else min(wanted, left)

    def read(self, size: int = -1) -> bytes:
        """Up to ``size`` bytes from the cursor (all written data if negative); ``b""`` at the end."""
        self._check_validity("read")
        n = self._readable(size)
        if n <= 0:
            return b""
        begin = METADATA_SIZE + self._pos
        out = self._mv[begin : begin + n].tobytes()
        self._pos += n
        return out

    def readinto(self, b: Union[bytearray, memoryview]) -> int:
        self._check_validity("readinto")
        if not isinstance(b, (bytearray, memoryview)) or (isinstance(b, memoryview) and b.readonly):
            raise TypeError(f"readinto() argument must be a writable bytes-like object, not {type(b).__name__}")
        if len(b) == 0:
            return 0
        n = self._readable(len(b))
        if n <= 0:
            return 0
        begin = METADATA_SIZE + self._pos
        try:
            b[:n] = self._mv[begin : begin + n]
        except Exception as e:
            raise OSError(f"Failed to read data into buffer from slice [{begin}:{begin + n}]") from e
        self._pos += n
        return n

    def seek(self, offset: int, whence: int = io.SEEK_SET) -> int:
        self._check_validity("seek")
        if whence == io.SEEK_SET:
            target = offset
        elif whence == io.SEEK_CUR:
            target = self._pos + offset
        elif whence == io.SEEK_END:
            target = self._metadata.len_written_data + offset
        else:
            raise ValueError(f"invalid whence value ({whence})")
        if target < 0:
            raise ValueError(f"Negative seek position is not allowed ({target})")
        self._pos = target
        return target

    def tell(self) -> int:
        self._check_validity()
        return self._pos

    def flush(self):
        """No-op: the mapping is shared with the page cache, there is nothing to push."""
        self._check_validity()

    @property
    def format_signature(self) -> bytes:
        self._check_validity()
        return self._metadata.format_signature

    # ------------------------------------------------------------------ lifecycle
    def close(self, truncate: bool = True) -> None:
        """Closes the underlying object; a writable one is first cut to metadata + written bytes."""
        if self.closed:
            return
        try:
            if truncate and not self.buffer_obj.is_readonly:
                self.buffer_obj.close(truncate_size=METADATA_SIZE + self._metadata.len_written_data)
            else:
                self.buffer_obj.close()
        finally:
            if self._mv is not None:
                self._metadata = None
                try:
                    self._mv.release()
                except BufferError:
                    pass  # a caller still holds a slice; the mapping itself is already gone
                self._mv = None
            self.buffer_obj = None
            self._pos = -1

    def resize(self, new_size: int) -> None:
        """Changes the size of the mapping (metadata block included). The address may change."""
        self._check_validity("write")
        if new_size < METADATA_SIZE:
            raise ValueError(f"New size must be at least {METADATA_SIZE} bytes, got {new_size}.")
        _LOGGER.info("Resizing BufferIO from %d to %d bytes.", len(self._mv), new_size)
        self._metadata = None
        try:
            self._mv.release()
        except BufferError:
            pass
        self._mv = None
        self.buffer_obj.resize(new_size)
        self._map_views(first_time=False)

    def __enter__(self):
        self._check_validity()
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()

    # ------------------------------------------------------------------ addresses for the GPU path
    def host_address(self, pos: int = 0) -> int:
        """Host address of stream position ``pos`` (byte ``METADATA_SIZE + pos`` of the mapping)."""
        self._check_validity()
        return self.buffer_obj.get_data_ptr() + METADATA_SIZE + pos

    def device_address(self, pos: int = 0) -> int:
        """Device-visible address of stream position ``pos``; registers the mapping on first use."""
        self._check_validity()
        if not self.buffer_obj.is_cuda_registered:
            self.buffer_obj.register_cuda()
        return self.buffer_obj.get_device_ptr() + METADATA_SIZE + pos

    @property
    def capacity(self) -> int:
        """Bytes of the mapping, metadata block included."""
        self._check_validity()
        return len(self._mv)
