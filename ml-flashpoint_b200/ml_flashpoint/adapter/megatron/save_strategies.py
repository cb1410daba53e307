"""Megatron-LM async save strategy over the B200 data path.

Same class and constructor as the reference's adapter/megatron/save_strategies.py:76-261
(``MLFlashpointMegatronAsyncSaveStrategy(storage_writer, backend, version, use_cached_ckpt_structure)``,
``async_save`` returning an ``AsyncRequest`` whose finalize functions replicate, write the global
metadata and finalize the checkpoint).

The division of labour differs. The reference blocks the trainer while every tensor is copied to
host memory, then hands the host copies to Megatron's writer process, which performs the memcpy
into the object. Here the trainer process, which owns the CUDA context and the tensors, queues
the pack kernel and the host transfer on side streams during ``async_save`` and returns as soon as
the kernel has read the tensors (milliseconds); nothing heavy is left for the writer process, so
``async_fn`` only sets up logging there, and the first finalize function, back in the trainer
process, waits for the transfer and publishes the write results.
"""

import copy
import json
import logging
import os
from functools import partial
from pathlib import Path
from typing import Union

import torch
from megatron.core.dist_checkpointing.mapping import ShardedStateDict
from megatron.core.dist_checkpointing.strategies.async_utils import AsyncRequest
from megatron.core.dist_checkpointing.strategies.base import AsyncSaveShardedStrategy
from megatron.core.dist_checkpointing.strategies.torch import (
    MCoreSavePlanner,
    _replace_state_dict_keys_with_sharded_keys,
    mcore_to_pyt_state_dict,
)
from torch.distributed.checkpoint.metadata import Metadata
from torch.distributed.checkpoint.planner import SavePlan
from torch.distributed.checkpoint.utils import _DistWrapper

from ml_flashpoint.adapter.pytorch import custom_state_dict_saver as statedictsaver
from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter
from ml_flashpoint.core import mlf_logging, utils
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
from ml_flashpoint.core.checkpoint_saver import MLFlashpointCheckpointSaver
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


def _save_checkpoint(checkpoint_id: CheckpointContainerId, rank: int, step: int):
    """``async_fn`` of the ``AsyncRequest``; runs in Megatron's writer process.

    The bytes are already on their way from the trainer process (see the module docstring), so
    this only tags the writer process's log lines with the rank and step it is working for.
    """
    mlf_logging.setup_worker_logging(rank, step)
    _LOGGER.debug("save of '%s' is being completed by the trainer process's side streams", checkpoint_id)


def default_backend_format_name() -> str:
    return "ml_flashpoint"


def default_backend_format_version() -> int:
    return 1


class MLFlashpointMegatronAsyncSaveStrategy(AsyncSaveShardedStrategy):
    def __init__(
        self,
        storage_writer: MemoryStorageWriter,
        backend: str = default_backend_format_name(),
        version: int = default_backend_format_version(),
        use_cached_ckpt_structure: bool = False,
    ):
        """``use_cached_ckpt_structure`` reuses the save plan of the previous checkpoint once it has
        been seen unchanged twice, which skips the planning collectives (and lets the engine reuse
        its uploaded copy plan as well)."""
        super().__init__(backend=backend, version=version)
        self._storage_writer: MemoryStorageWriter = storage_writer
        self._checkpoint_saver: MLFlashpointCheckpointSaver = storage_writer.checkpoint_saver
        self._cached_central_plan: SavePlan | None = None
        self._cached_local_plan: SavePlan | None = None
        self._cached_global_metadata: Metadata | None = None
        self._validated_cache_reuse: bool = False
        self._use_cached_ckpt_structure: bool = use_cached_ckpt_structure

    @property
    def thread_count(self) -> int:
        return self._storage_writer._thread_count

    def can_handle_sharded_objects(self) -> bool:
        return True

    @log_execution_time(logger=_LOGGER, name="async_save", level=logging.INFO)
    def async_save(self, sharded_state_dict: ShardedStateDict, checkpoint_dir: Union[str, Path]) -> AsyncRequest:
        """Plans the save, queues the pack kernel and transfers, and returns an ``AsyncRequest``.

        On return the tensors of ``sharded_state_dict`` may be modified again. The caller must
        schedule the request as with any Megatron async strategy; its finalize functions must run in
        this process.
        """
        checkpoint_id = CheckpointContainerId(checkpoint_dir)
        self._checkpoint_saver.initialize_checkpoint(checkpoint_id)
        previous = self._storage_writer
        # a fresh writer per checkpoint: saves of consecutive steps may overlap
        self._storage_writer = MemoryStorageWriter(
            checkpoint_saver=self._checkpoint_saver,
            mp_manager_future=previous._main_process_torchmp_manager_future,
            thread_count=previous._thread_count,
        )
        self._storage_writer.reset(checkpoint_id.data)

        sharded_state_dict, _, _ = _replace_state_dict_keys_with_sharded_keys(
            sharded_state_dict=sharded_state_dict, keep_only_main_replica=True
        )
        pyt_state_dict = mcore_to_pyt_state_dict(sharded_state_dict)

        use_dist = not utils.get_env_val_bool("DISABLE_DIST", False)
        planner = MCoreSavePlanner(can_run_decentralized_global_plan=False)
        world = _DistWrapper(group=None, use_dist=use_dist, coordinator_rank=0)
        cached = None
        if self._use_cached_ckpt_structure:
            cached = (self._cached_central_plan, self._cached_local_plan, self._validated_cache_reuse)
        (
            write_buckets,
            global_metadata,
            self._cached_central_plan,
            self._cached_local_plan,
            self._validated_cache_reuse,
        ) = statedictsaver.generate_plan(
            checkpoint_id=checkpoint_id,
            state_dict=pyt_state_dict,
            storage_writer=self._storage_writer,
            planner=planner,
            world_dist_wrapper=world,
            cached_ckpt_structure=cached,
        )
        if global_metadata is None:  # planning was skipped: the structure is the cached one
            global_metadata = copy.deepcopy(self._cached_global_metadata)
        else:
            self._cached_global_metadata = copy.deepcopy(global_metadata)

        staged = self._storage_writer.stage_write_data_buckets(checkpoint_id, write_buckets, non_blocking=True)
        pending = self._storage_writer.launch_staged_data_buckets(checkpoint_id, staged, replicate_after_write=False)
        pending.wait_safe_to_mutate()

        # Megatron looks for this file to recognise a checkpoint directory
        with open(os.path.join(checkpoint_dir, "metadata.json"), "w") as f:
            json.dump({"sharded_backend": ""}, f)

        writer = self._storage_writer
        finalize_fns = [
            partial(writer.complete_launched_buckets, checkpoint_id, pending),
            partial(writer.replicate_written_objects, object_ids={b.object_id for b in staged}),
            partial(
                statedictsaver.finish_write,
                checkpoint_id=checkpoint_id,
                storage_writer=writer,
                global_metadata=global_metadata,
                world_dist_wrapper=world,
            ),
            partial(self._checkpoint_saver.finalize_checkpoint, checkpoint_id=checkpoint_id),
        ]
        rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else -1
        return AsyncRequest(
            async_fn=_save_checkpoint,
            async_fn_args=(),
            async_fn_kwargs={"checkpoint_id": checkpoint_id, "rank": rank, "step": mlf_logging.get_current_step()},
            finalize_fns=finalize_fns,
        )
