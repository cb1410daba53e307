"""``CheckpointObjectManager``: where checkpoint objects are created, opened and deleted.

Call-compatible with the reference (checkpoint_object_manager/checkpoint_object_manager.py:30-284):
write buffers come from the per-process ``BufferPool`` when one is configured and has a free
buffer, otherwise a standalone file is created at the object's path; reads are read-only mappings;
one pool per process is shared through a class-level registry.
"""

import os
import shutil
import threading
from typing import ClassVar, Optional

from ml_flashpoint.checkpoint_object_manager.buffer_io import BufferIO
from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE
from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject
from ml_flashpoint.core.buffer_pool import BufferPool, BufferPoolConfig
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.mlf_logging import get_logger

_LOGGER = get_logger(__name__)


class CheckpointObjectManager:
    _worker_pool: ClassVar[Optional[BufferPool]] = None
    _worker_pool_lock: ClassVar[threading.Lock] = threading.Lock()

    def __init__(self, pool_config: Optional[BufferPoolConfig] = None):
        self._pool_config = pool_config

    def _get_or_create_buffer_pool(self) -> Optional[BufferPool]:
        cls = CheckpointObjectManager
        if cls._worker_pool:
            return cls._worker_pool
        if not self._pool_config:
            return None
        with cls._worker_pool_lock:
            if cls._worker_pool is None:
                cfg = self._pool_config
                try:
                    _LOGGER.info("Initializing BufferPool with config: %s", cfg)
                    extra = {"register_cuda": True} if getattr(cfg, "register_cuda", False) else {}
                    cls._worker_pool = BufferPool(
                        pool_dir_path=cfg.pool_dir_path,
                        num_buffers=cfg.num_buffers,
                        rank=cfg.rank,
                        buffer_size=cfg.buffer_size,
                        **extra,
                    )
                except Exception:
                    _LOGGER.exception("Failed to initialize BufferPool")
        return cls._worker_pool

    def teardown_pool(self):
        cls = CheckpointObjectManager
        with cls._worker_pool_lock:
            pool, cls._worker_pool = cls._worker_pool, None
        if pool:
            try:
                pool.teardown()
            except Exception as e:
                _LOGGER.debug("Failed to teardown BufferPool: %s", e)

    def acquire_buffer(self, object_id: CheckpointObjectId, buffer_size: int, overwrite: bool = True) -> "BufferIO":
        """A writable buffer for ``object_id``: pooled if possible, else a new file of ``buffer_size`` + metadata.

        A pooled buffer may be smaller than asked; it grows on demand while being written.
        """
        if buffer_size <= 0:
            raise ValueError("Buffer size must be a positive integer.")
        total = buffer_size + METADATA_SIZE
        path = str(object_id)
        try:
            os.makedirs(os.path.dirname(path), exist_ok=True)
            if os.path.exists(path):
                if not overwrite:
                    raise FileExistsError(f"File {object_id} already exists and overwrite=False")
                self.delete_object(object_id)
            pool = self._get_or_create_buffer_pool()
            if pool:
                return pool.acquire(associated_symlink=path)
        except RuntimeError:
            _LOGGER.debug("BufferPool exhausted. Falling back to standalone buffer creation.")
        try:
            return BufferIO(BufferObject(path, total, overwrite))
        except Exception as e:
            _LOGGER.exception("Failed to create buffer for object_id='%s'", object_id)
            raise RuntimeError(f"Failed to create buffer for '{object_id}'") from e

    def get_buffer(self, object_id: CheckpointObjectId) -> Optional["BufferIO"]:
        """Read-only view of an existing object, or None if it cannot be opened."""
        try:
            return BufferIO(BufferObject(str(object_id)))
        except (OSError, ValueError, RuntimeError):
            _LOGGER.exception("Could not open buffer '%s'. Returning None.", object_id)
            return None

    def close_buffer(self, buffer_io: BufferIO, skip_close_if_symlink: bool = False, truncate: bool = True) -> None:
        if not isinstance(buffer_io, BufferIO) or buffer_io.closed:
            _LOGGER.warning("Attempted to close an invalid or already-closed buffer. Ignoring.")
            return
        object_id = buffer_io.buffer_obj.get_id()
        # objects that are symlinks point into the pool, whose buffers outlive their clients
        if skip_close_if_symlink and os.path.islink(object_id):
            _LOGGER.debug("Buffer for object_id='%s' is a symlink. Ignoring.", object_id)
            return
        try:
            buffer_io.close(truncate=truncate)
        except Exception:
            _LOGGER.exception("An error occurred while closing buffer for object_id='%s'.", object_id)
            raise

    def delete_container(self, container_id: CheckpointContainerId) -> None:
        """Removes a container directory and everything in it; a missing directory is not an error."""
        path = str(container_id)

        def _ignore_missing(func, failed_path, exc_info):
            if not isinstance(exc_info[1], FileNotFoundError):
                raise exc_info[1]

        try:
            if os.path.isdir(path):
                shutil.rmtree(path, onerror=_ignore_missing)
            else:
                _LOGGER.warning("Container '%s' is not a directory or does not exist. Nothing to delete from disk.", path)
        except OSError:
            _LOGGER.exception("Error deleting container directory '%s'", path)
            raise

    def delete_object(self, object_id: CheckpointObjectId) -> None:
        """Removes an object file or the symlink standing for it."""
        path = str(object_id)
        try:
            if os.path.lexists(path):
                os.remove(path)
            else:
                _LOGGER.warning("Object '%s' does not exist. Nothing to delete.", path)
        except OSError:
            _LOGGER.exception("Error deleting object '%s'", path)
            raise
