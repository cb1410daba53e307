"""Megatron-LM load strategy over the B200 data path.

Same class as the reference's adapter/megatron/load_strategies.py:57-159: converts the MCore
sharded state dict to DCP form, runs ``dcp.load`` through ``MemoryStorageReader`` (one
scatter-unpack kernel per object), converts back; metadata queries read the pickled ``.metadata``.
"""

import io
import logging
from pathlib import Path
from typing import Union

import torch
from megatron.core.dist_checkpointing.mapping import ShardedObject, ShardedStateDict, ShardedTensor, StateDict
from megatron.core.dist_checkpointing.strategies.base import LoadShardedStrategy
from megatron.core.dist_checkpointing.strategies.torch import (
    MCoreLoadPlanner,
    _replace_sharded_keys_with_state_dict_keys,
    _replace_state_dict_keys_with_sharded_keys,
    _restore_dict_types,
    _unwrap_pyt_sharded_tensor,
    mcore_to_pyt_state_dict,
)
from torch.distributed import checkpoint as torch_dist_checkpoint
from torch.distributed._shard.sharded_tensor import ShardedTensor as TorchShardedTensor
from torch.distributed.checkpoint import BytesStorageMetadata, Metadata, TensorStorageMetadata

from ml_flashpoint.adapter.pytorch.memory_storage_reader import MemoryStorageReader
from ml_flashpoint.core.checkpoint_loader import CheckpointContainerId, MLFlashpointCheckpointLoader
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time
from ml_flashpoint.replication.replication_manager import ReplicationManager

_LOGGER = get_logger(__name__)


class MLFlashpointMegatronLoadStrategy(LoadShardedStrategy):
    def __init__(self, replication_manager: ReplicationManager, checkpoint_loader: MLFlashpointCheckpointLoader):
        super().__init__()
        self.checkpoint_loader = checkpoint_loader
        self._replication_manager = replication_manager

    def _metadata(self, checkpoint_dir: Union[str, Path]) -> Metadata:
        metadata = self.checkpoint_loader.read_metadata(CheckpointContainerId(checkpoint_dir))
        if metadata is None or not hasattr(metadata, "state_dict_metadata"):
            raise RuntimeError(f"Failed to load valid metadata from {checkpoint_dir}")
        return metadata

    @log_execution_time(logger=_LOGGER, name="load", level=logging.INFO)
    def load(self, sharded_state_dict: ShardedStateDict, checkpoint_dir: Union[str, Path]) -> StateDict:
        original = sharded_state_dict
        sharded_state_dict, flat_mapping, rename_mapping = _replace_state_dict_keys_with_sharded_keys(sharded_state_dict)
        pyt_state_dict = mcore_to_pyt_state_dict(sharded_state_dict, is_loading=True)
        torch_dist_checkpoint.load(
            state_dict=pyt_state_dict,
            storage_reader=MemoryStorageReader(path=checkpoint_dir, checkpoint_loader=self.checkpoint_loader),
            planner=MCoreLoadPlanner(),
        )
        loaded: dict[str, Union[TorchShardedTensor, list[io.BytesIO]]] = {
            key: _unwrap_pyt_sharded_tensor(value) for key, value in pyt_state_dict.items()
        }
        loaded = _replace_sharded_keys_with_state_dict_keys(loaded, flat_mapping, rename_mapping)
        _restore_dict_types(loaded, original)
        return loaded

    @log_execution_time(logger=_LOGGER, name="load_tensors_metadata", level=logging.INFO)
    def load_tensors_metadata(self, checkpoint_dir: Union[str, Path], metadata: Metadata = None) -> StateDict:
        """Data-less ``ShardedTensor`` for every tensor recorded in the checkpoint metadata."""
        if metadata is None:
            metadata = self._metadata(checkpoint_dir)
        out = {}
        for key, entry in metadata.state_dict_metadata.items():
            if isinstance(entry, TensorStorageMetadata):
                shape_only = torch.empty(entry.size, **entry.properties.__dict__, device="meta")
                out[key] = ShardedTensor.from_rank_offsets(key, shape_only).without_data()
        return out

    @log_execution_time(logger=_LOGGER, name="load_sharded_metadata", level=logging.INFO)
    def load_sharded_metadata(self, checkpoint_dir: Union[str, Path]) -> ShardedStateDict:
        """Tensors as in ``load_tensors_metadata`` plus an empty ``ShardedObject`` per byte item."""
        metadata = self._metadata(checkpoint_dir)
        out = {}
        for key, entry in metadata.state_dict_metadata.items():
            if isinstance(entry, BytesStorageMetadata):
                obj = ShardedObject.empty_from_unique_key(key)
                out[obj.unique_key] = obj
        out.update(self.load_tensors_metadata(checkpoint_dir, metadata))
        return out

    def check_backend_compatibility(self, loaded_backend):
        pass

    def check_version_compatibility(self, loaded_version):
        pass

    @property
    def can_handle_sharded_objects(self) -> bool:
        return True
