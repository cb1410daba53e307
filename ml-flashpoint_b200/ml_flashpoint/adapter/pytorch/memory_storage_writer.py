"""PyTorch DCP ``StorageWriter`` that saves into memory-backed checkpoint objects.

Same surface as the reference's adapter/pytorch/memory_storage_writer.py:53-401: usable directly with
``dcp.save`` (``write_data``), or in the split form ``prepare_write_data_buckets`` ->
``stage_write_data_buckets`` -> ``write_staged_data_buckets`` that Megatron-style async saving needs.
Per-checkpoint write results and completion events live in ``multiprocessing.Manager`` containers
so that a writer process can hand them back to the trainer.

Difference on the data path: staging does not copy tensors to the host. The gather-pack kernel
reads them from HBM when the bucket is written, so ``stage_write_data_buckets`` only makes sure the
producing stream has finished.
"""

import concurrent.futures
import dataclasses
import logging
import os
import time
from typing import Optional, Union

import torch
import torch.multiprocessing as torch_mp
from torch.distributed.checkpoint import Metadata, SavePlan, SavePlanner, StorageWriter, staging
from torch.distributed.checkpoint.filesystem import _StorageInfo
from torch.distributed.checkpoint.metadata import STATE_DICT_TYPE, MetadataIndex, StorageMeta
from torch.distributed.checkpoint.storage import WriteResult
from torch.futures import Future as TorchFuture

from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.checkpoint_saver import MLFlashpointCheckpointSaver, ObjectWriteBucket
from ml_flashpoint.core.hfid import generate_hfid
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


@dataclasses.dataclass
class _StorageDataContext:
    """Carried in ``SavePlan.storage_data``: the object-name prefix unique to one rank's plan."""

    prefix: str


class MemoryStorageWriter(StorageWriter, staging.BlockingAsyncStager):
    def __init__(
        self,
        checkpoint_saver: MLFlashpointCheckpointSaver,
        mp_manager_future: concurrent.futures.Future,
        thread_count: int = 1,
    ):
        """``mp_manager_future`` resolves to a ``torch.multiprocessing.Manager`` (create it with the
        spawn context so that it does not inherit CUDA state). ``thread_count`` < 1 is raised to 1."""
        super().__init__()
        self._current_checkpoint_id: CheckpointContainerId | None = None
        self._current_save_id: str | None = None
        self._checkpoint_saver: MLFlashpointCheckpointSaver = checkpoint_saver
        if thread_count < 1:
            _LOGGER.warning("thread_count must be >= 1, but was %d. Setting to 1.", thread_count)
            thread_count = 1
        self._thread_count = thread_count
        # only valid in the process that created the writer: managers cannot be pickled
        self._main_process_torchmp_manager_future = mp_manager_future
        self._write_events_per_checkpoint_id: Optional[dict[CheckpointContainerId, torch_mp.Event]] = None
        self._write_results_per_checkpoint_id: Optional[dict[CheckpointContainerId, list[WriteResult]]] = None

    def __getstate__(self):
        state = self.__dict__.copy()
        state.pop("_main_process_torchmp_manager_future", None)
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._main_process_torchmp_manager_future = None

    def _check_checkpoint_id(self) -> None:
        if self._current_checkpoint_id is None:
            raise ValueError("MemoryStorageWriter has not been reset. Call reset() before using this method.")

    @property
    def current_checkpoint_id(self) -> Optional[CheckpointContainerId]:
        return self._current_checkpoint_id

    @property
    def path(self) -> Optional[str]:
        return None if self._current_checkpoint_id is None else self._current_checkpoint_id.data

    @property
    def checkpoint_saver(self) -> MLFlashpointCheckpointSaver:
        return self._checkpoint_saver

    # ------------------------------------------------------------------ StorageWriter protocol
    def reset(self, checkpoint_id: Union[str, os.PathLike, None] = None) -> None:
        self._current_checkpoint_id = CheckpointContainerId(checkpoint_id)
        self._current_save_id = generate_hfid("memwritersave")
        if self._write_events_per_checkpoint_id is None and self._main_process_torchmp_manager_future is not None:
            manager = self._main_process_torchmp_manager_future.result()
            self._write_events_per_checkpoint_id = manager.dict()
            self._write_results_per_checkpoint_id = manager.dict()

    def storage_meta(self) -> Optional[StorageMeta]:
        self._check_checkpoint_id()
        return StorageMeta(checkpoint_id=self._current_checkpoint_id.data, save_id=self._current_save_id)

    def set_up_storage_writer(self, is_coordinator: bool) -> None:
        pass

    @log_execution_time(logger=_LOGGER, name="prepare_local_plan")
    def prepare_local_plan(self, plan: SavePlan) -> SavePlan:
        self._check_checkpoint_id()
        # idempotent: marks the checkpoint dirty and creates its directory if nobody did yet
        self._checkpoint_saver.initialize_checkpoint(self._current_checkpoint_id)
        return plan

    @log_execution_time(logger=_LOGGER, name="prepare_global_plan")
    def prepare_global_plan(self, plans: list[SavePlan]) -> list[SavePlan]:
        return [dataclasses.replace(p, storage_data=_StorageDataContext(f"__{i}_")) for i, p in enumerate(plans)]

    @log_execution_time(logger=_LOGGER, name="stage", level=logging.INFO)
    def stage(self, state_dict: STATE_DICT_TYPE) -> STATE_DICT_TYPE:
        """Snapshot for ``dcp.async_save``: every tensor is cloned where it lives.

        The reference offloads the state dict to (pinned) host memory here. With 180 GB of HBM a
        device-side clone is the cheaper snapshot: it runs at HBM speed, the trainer continues at
        once, and the background save packs from the clone straight into the object.
        """
        from torch.utils._pytree import tree_map_only

        snapshot = tree_map_only(torch.Tensor, lambda t: t.detach().clone(), state_dict)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        return snapshot

    # ------------------------------------------------------------------ split save path
    @log_execution_time(logger=_LOGGER, name="prepare_write_data_buckets")
    def prepare_write_data_buckets(
        self, checkpoint_id: CheckpointContainerId, plan: SavePlan, planner: SavePlanner
    ) -> list[ObjectWriteBucket]:
        if checkpoint_id not in self._write_events_per_checkpoint_id:
            self._write_events_per_checkpoint_id[checkpoint_id] = self._main_process_torchmp_manager_future.result().Event()
        return self.checkpoint_saver.prepare_write_data(
            checkpoint_id, plan.items, planner, plan.storage_data.prefix, bucket_count=self._thread_count
        )

    @staticmethod
    @log_execution_time(logger=_LOGGER, name="stage_write_data_buckets", level=logging.INFO)
    def stage_write_data_buckets(
        _: CheckpointContainerId, write_buckets: list[ObjectWriteBucket], non_blocking: bool = True
    ):
        """Returns fresh bucket objects whose tensors are final and still device-resident.

        The reference copies every tensor to pageable host memory here and synchronises
        (memory_storage_writer.py:211-233); that copy is what the pack kernel makes unnecessary.
        """
        staged = [dataclasses.replace(b, tensor_data=list(b.tensor_data)) for b in write_buckets]
        if torch.cuda.is_available() and any(t.is_cuda for b in staged for _, t in b.tensor_data):
            torch.cuda.current_stream().synchronize()
        return staged

    @log_execution_time(logger=_LOGGER, name="write_staged_write_buckets", level=logging.INFO)
    def write_staged_data_buckets(
        self,
        checkpoint_id: CheckpointContainerId,
        staged_write_buckets: list[ObjectWriteBucket],
        replicate_after_write: bool,
    ) -> TorchFuture[list[WriteResult]]:
        t0 = time.perf_counter()
        write_results = self._checkpoint_saver.write_data(
            checkpoint_id,
            write_buckets=staged_write_buckets,
            thread_count=self._thread_count,
            replicate_after_write=replicate_after_write,
        )
        elapsed = time.perf_counter() - t0
        if elapsed > 0:
            written = sum(r.size_in_bytes for r in write_results)
            # log post-processing parses this line
            _LOGGER.info(
                "Written %d bytes in %.4f s (%.2f GB/s) from %d buckets",
                written,
                elapsed,
                written / 1e9 / elapsed,
                len(staged_write_buckets),
            )
        self._write_results_per_checkpoint_id[checkpoint_id] = write_results
        self._write_events_per_checkpoint_id[checkpoint_id].set()
        done: TorchFuture = TorchFuture()
        done.set_result(write_results)
        return done

    def launch_staged_data_buckets(
        self,
        checkpoint_id: CheckpointContainerId,
        staged_write_buckets: list[ObjectWriteBucket],
        replicate_after_write: bool = False,
    ):
        """Overlapped form of ``write_staged_data_buckets``: queues the pack kernels and transfers and
        returns a ``PendingSave`` at once. Call ``complete_launched_buckets`` with it later to publish
        the results (this is what a training loop uses to hide the host transfer behind compute)."""
        return self._checkpoint_saver.write_data_async(checkpoint_id, staged_write_buckets, replicate_after_write)

    def complete_launched_buckets(self, checkpoint_id: CheckpointContainerId, pending) -> list[WriteResult]:
        """Waits for a ``PendingSave``, records its write results for ``get_write_results`` and signals
        completion, exactly as ``write_staged_data_buckets`` does for a blocking write."""
        write_results = pending.result()
        self._write_results_per_checkpoint_id[checkpoint_id] = write_results
        self._write_events_per_checkpoint_id[checkpoint_id].set()
        return write_results

    @log_execution_time(logger=_LOGGER, name="write_data", level=logging.INFO)
    def write_data(self, plan: SavePlan, planner: SavePlanner) -> TorchFuture[list[WriteResult]]:
        self._check_checkpoint_id()
        if not isinstance(plan.storage_data, _StorageDataContext) or not plan.storage_data.prefix:
            raise ValueError(
                "SavePlan.storage_data is not a valid _StorageDataContext or prefix is empty. "
                "This is likely because prepare_global_plan was not called on this SavePlan."
            )
        buckets = self.prepare_write_data_buckets(self.current_checkpoint_id, plan, planner)
        return self.write_staged_data_buckets(self.current_checkpoint_id, buckets, replicate_after_write=True)

    def replicate_written_objects(self, object_ids: set[CheckpointObjectId]) -> list[concurrent.futures.Future]:
        """Starts replication of already written objects; call before ``finalize_checkpoint``."""
        futures = []
        for object_id in object_ids:
            futures.extend(self._checkpoint_saver.async_replicate_object(object_id))
        return futures

    @log_execution_time(logger=_LOGGER, name="get_write_results")
    def get_write_results(
        self, checkpoint_id: CheckpointContainerId, wait_timeout_sec: float = 15.0
    ) -> list[WriteResult]:
        """Waits for the write of ``checkpoint_id`` to be signalled, then returns its results.

        ``KeyError`` if no write was ever prepared for it, ``RuntimeError`` on timeout.
        """
        if not self._write_events_per_checkpoint_id[checkpoint_id].wait(timeout=wait_timeout_sec):
            msg = (
                "Event was never set for checkpoint_id '%s', meaning we cannot confirm that the write "
                "has completed, and its results are available." % checkpoint_id
            )
            _LOGGER.error(msg)
            raise RuntimeError(msg)
        return self._write_results_per_checkpoint_id.get(checkpoint_id)

    @log_execution_time(logger=_LOGGER, name="finish")
    def finish(self, metadata: Metadata, results: list[list[WriteResult]]) -> None:
        self._check_checkpoint_id()
        self.finish_checkpoint(self.current_checkpoint_id, metadata, results)

    @log_execution_time(logger=_LOGGER, name="finish_checkpoint", level=logging.INFO)
    def finish_checkpoint(
        self, checkpoint_id: CheckpointContainerId, metadata: Metadata, results: list[list[WriteResult]]
    ) -> None:
        """``finish`` with an explicit checkpoint id, safe when saves of several steps overlap."""
        storage_data: dict[MetadataIndex, _StorageInfo] = {}
        for idx, per_rank in enumerate(results):
            if per_rank is None:
                msg = (
                    "finish: write results[%d] is None! This suggests an error in producing or gathering "
                    "the write_results list from that local rank (%d)." % (idx, idx)
                )
                _LOGGER.error(msg)
                raise RuntimeError(msg)
            for wr in per_rank:
                storage_data[wr.index] = wr.storage_data
        metadata.storage_data = storage_data
        metadata.storage_meta = self.storage_meta()
        self._checkpoint_saver.write_metadata(checkpoint_id, metadata)
        self._write_results_per_checkpoint_id.pop(checkpoint_id, None)

    @classmethod
    def validate_checkpoint_id(cls, checkpoint_id: Union[str, os.PathLike]) -> bool:
        try:
            CheckpointContainerId(checkpoint_id)
            return True
        except Exception as e:
            _LOGGER.warning("Unable to validate checkpoint_id: %s, %s", checkpoint_id, e)
            return False
