"""The three phases of a DCP save as separate calls: plan, write, finish.

Same functions as the reference's adapter/pytorch/custom_state_dict_saver.py:41-227 (which in turn
follows torch's ``state_dict_saver.save``): ``generate_plan`` runs local and global planning (with
optional reuse of a cached plan) and resolves the write buckets, ``write_data`` writes them,
``finish_write`` gathers every rank's write results and lets each node's first rank write the
global metadata.
"""

import logging

import torch.cuda
from torch import distributed as torchdist
from torch.distributed.checkpoint import state_dict_saver as torchdistsaver
from torch.distributed.checkpoint.logger import _dcp_method_logger
from torch.distributed.checkpoint.planner import SavePlan
from torch.distributed.checkpoint.storage import WriteResult
from torch.distributed.checkpoint.utils import _DistWrapper

from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter
from ml_flashpoint.core import utils
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
from ml_flashpoint.core.checkpoint_saver import ObjectWriteBucket
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


@log_execution_time(logger=_LOGGER, name="generate_plan", level=logging.INFO)
def generate_plan(
    checkpoint_id: CheckpointContainerId,
    state_dict: torchdistsaver.STATE_DICT_TYPE,
    storage_writer: MemoryStorageWriter,
    planner: torchdistsaver.SavePlanner,
    world_dist_wrapper: _DistWrapper,
    cached_ckpt_structure: tuple[SavePlan, SavePlan, bool] | None = None,
) -> tuple[list[ObjectWriteBucket], torchdistsaver.Metadata | None, SavePlan, SavePlan, bool]:
    """Plans a save without writing anything.

    ``cached_ckpt_structure`` is ``(central plan, local plan, validated)`` from an earlier call.
    Once ``validated`` is True the collectives are skipped and the cached plans are reused.
    Returns ``(write buckets, global metadata or None, central plan, local plan, validated)`` where
    ``validated`` says that this call's central plan equals the cached one, i.e. the checkpoint
    structure is stable and the next call may skip planning.
    """
    cached_central, cached_local, reuse = cached_ckpt_structure or (None, None, False)
    global_metadata: torchdistsaver.Metadata | None = None
    log_kwargs = {"checkpoint_id": storage_writer.current_checkpoint_id, "process_group": world_dist_wrapper.group}

    @_dcp_method_logger(**log_kwargs)
    def local_step() -> SavePlan:
        planner.set_up_planner(
            state_dict=state_dict,
            storage_meta=storage_writer.storage_meta(),
            is_coordinator=world_dist_wrapper.is_coordinator,
        )
        storage_writer.set_up_storage_writer(world_dist_wrapper.is_coordinator)
        plan = cached_local if (cached_local and reuse) else planner.create_local_plan()
        return storage_writer.prepare_local_plan(plan)

    @_dcp_method_logger(**log_kwargs)
    def global_step(all_local_plans: list[SavePlan]) -> list[SavePlan]:
        nonlocal global_metadata
        all_local_plans, global_metadata = planner.create_global_plan(all_local_plans)
        return storage_writer.prepare_global_plan(all_local_plans)

    if reuse and cached_central:
        local_plan = local_step()
        central_plan = cached_central
    else:
        with log_execution_time(logger=_LOGGER, name="generate_plan__reduce_scatter_plan"):
            local_plan = local_step()
            central_plan = world_dist_wrapper.reduce_scatter("plan", lambda: local_plan, global_step)
        with log_execution_time(logger=_LOGGER, name="generate_plan__broadcast_metadata"):
            global_metadata = world_dist_wrapper.broadcast_object(global_metadata)

    final_local_plan = planner.finish_plan(central_plan)
    buckets = storage_writer.prepare_write_data_buckets(checkpoint_id, final_local_plan, planner)
    return buckets, global_metadata, central_plan, local_plan, cached_central == central_plan


@log_execution_time(logger=_LOGGER, name="write_data", level=logging.INFO)
def write_data(
    checkpoint_id: CheckpointContainerId,
    storage_writer: MemoryStorageWriter,
    staged_write_buckets: list[ObjectWriteBucket],
    replicate_after_write: bool,
) -> list[WriteResult]:
    return storage_writer.write_staged_data_buckets(checkpoint_id, staged_write_buckets, replicate_after_write).wait()


@log_execution_time(logger=_LOGGER, name="finish_write", level=logging.INFO)
def finish_write(
    checkpoint_id: CheckpointContainerId,
    storage_writer: MemoryStorageWriter,
    global_metadata: torchdistsaver.Metadata,
    world_dist_wrapper: _DistWrapper,
) -> None:
    """Call only after the write of ``checkpoint_id`` is known to be complete on this rank."""
    gathered = world_dist_wrapper.gather_object(storage_writer.get_write_results(checkpoint_id))
    with log_execution_time(logger=_LOGGER, name="finish_write__broadcast_results"):
        gathered = world_dist_wrapper.broadcast_object(gathered)
    if torchdist.get_node_local_rank() == 0:
        storage_writer.finish_checkpoint(checkpoint_id=checkpoint_id, metadata=global_metadata, results=gathered)


def _get_local_rank_0_global_ranks() -> list[int]:
    """Global ranks that are local rank 0 on their node, assuming one process per GPU."""
    per_node = torch.cuda.device_count()
    return [i * per_node for i in range(utils.get_num_of_nodes())]
