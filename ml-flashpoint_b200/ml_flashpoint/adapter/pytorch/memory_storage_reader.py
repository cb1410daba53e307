"""PyTorch DCP ``StorageReader`` over memory-backed checkpoint objects.

Same surface as the reference's adapter/pytorch/memory_storage_reader.py:46-160. Read items are
grouped per object; each object is handed to ``MLFlashpointCheckpointLoader.read_data``, which
restores all of its tensors with one scatter-unpack kernel launch.
"""

import logging
import os
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, List, Union

import torch
from torch.distributed.checkpoint import StorageReader
from torch.distributed.checkpoint import metadata as torchdistmeta
from torch.distributed.checkpoint.filesystem import FileSystem, _StorageInfo
from torch.distributed.checkpoint.planner import LoadPlan, LoadPlanner, ReadItem
from torch.futures import Future

from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.checkpoint_loader import MLFlashpointCheckpointLoader
from ml_flashpoint.core.hfid import generate_hfid
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


class MemoryStorageReader(StorageReader):
    _path: str
    _checkpoint_container_id: CheckpointContainerId
    _load_id: str
    _checkpoint_loader: MLFlashpointCheckpointLoader
    _storage_data: dict[torchdistmeta.MetadataIndex, _StorageInfo] | None

    def __init__(self, path: Union[str, os.PathLike], checkpoint_loader: MLFlashpointCheckpointLoader):
        super().__init__()
        self.reset(path)
        self._checkpoint_loader = checkpoint_loader
        self._storage_data = None

    def reset(self, checkpoint_id: Union[str, os.PathLike, None] = None) -> None:
        self._path = checkpoint_id
        self._checkpoint_container_id = CheckpointContainerId(str(checkpoint_id))
        self._load_id = generate_hfid("memreaderload")

    @log_execution_time(logger=_LOGGER, name="read_metadata", level=logging.INFO)
    def read_metadata(self) -> torchdistmeta.Metadata:
        metadata = self._checkpoint_loader.read_metadata(self._checkpoint_container_id)
        if self._load_id:
            metadata.storage_meta.load_id = self._load_id
        return metadata

    def set_up_storage_reader(self, metadata: torchdistmeta.Metadata, is_coordinator: bool) -> None:
        self._storage_data = metadata.storage_data
        if self._storage_data is None:
            raise ValueError("metadata.storage_data cannot be None.")

    def prepare_local_plan(self, plan: LoadPlan) -> LoadPlan:
        return plan

    def prepare_global_plan(self, plans: list[LoadPlan]) -> list[LoadPlan]:
        return plans

    @log_execution_time(logger=_LOGGER, name="read_data", level=logging.INFO)
    def read_data(self, plan: LoadPlan, planner: LoadPlanner) -> Future[None]:
        by_object: Dict[str, List[ReadItem]] = {}
        for item in plan.items:
            by_object.setdefault(self._storage_data[item.storage_index].relative_path, []).append(item)

        if by_object:
            t0 = time.perf_counter()
            with ThreadPoolExecutor() as pool:
                tasks = [
                    pool.submit(
                        self._checkpoint_loader.read_data,
                        CheckpointObjectId(str(Path(self._path) / relative_path)),
                        items,
                        planner,
                        self._storage_data,
                    )
                    for relative_path, items in by_object.items()
                ]
                for task in tasks:
                    task.result()  # re-raises what the reader thread raised
            elapsed = time.perf_counter() - t0
            if elapsed > 0:
                nbytes = sum(self._storage_data[i.storage_index].length for i in plan.items)
                # log post-processing parses this line
                _LOGGER.info(
                    "Read %d bytes in %.4f s (%.2f GB/s) from %d files", nbytes, elapsed, nbytes / 1e9 / elapsed, len(by_object)
                )
        else:
            _LOGGER.info("Rank %d: No files to read for plan in '%s'", torch.distributed.get_rank(), self._path)
        done: Future = Future()
        done.set_result(None)
        return done

    @classmethod
    def validate_checkpoint_id(cls, checkpoint_id: Union[str, os.PathLike]) -> bool:
        return FileSystem.validate_checkpoint_id(checkpoint_id)
