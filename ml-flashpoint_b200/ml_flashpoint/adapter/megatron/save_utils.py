"""Entry point for saving a Megatron checkpoint with node-local common state.

Same function as the reference's adapter/megatron/save_utils.py:29-79: like Megatron's
``dist_checkpointing.save`` it splits the checkpoint into sharded and common parts, but every
node's first rank writes ``common.pt`` (recovery reads it locally), and a failing save is logged
and swallowed so that training continues.
"""

import os
from pathlib import Path
from typing import Any, Optional, Union

import torch
from megatron.core.dist_checkpointing import state_dict_utils as mcore_state_dict_utils
from megatron.core.dist_checkpointing.strategies.async_utils import AsyncRequest
from megatron.core.dist_checkpointing.strategies.common import COMMON_STATE_FNAME

from ml_flashpoint.core.mlf_logging import get_logger

_LOGGER = get_logger(__name__)


def save_local_aware_megatron_checkpoint(
    checkpoint: dict[str, Any],
    checkpoint_dir: Union[str, Path],
    save_strategy,
    async_save: bool = True,
) -> Optional[AsyncRequest]:
    """Returns the strategy's ``AsyncRequest`` for an async save, otherwise (or on failure) None."""
    sharded_state_dict, common_state_dict = mcore_state_dict_utils.save_preprocess(checkpoint)
    if torch.distributed.get_node_local_rank() == 0:
        os.makedirs(checkpoint_dir, exist_ok=True)
        torch.save(common_state_dict, os.path.join(checkpoint_dir, COMMON_STATE_FNAME))
    try:
        if async_save:
            return save_strategy.async_save(sharded_state_dict=sharded_state_dict, checkpoint_dir=checkpoint_dir)
        save_strategy.save(sharded_state_dict=sharded_state_dict, checkpoint_dir=checkpoint_dir)
    except Exception:
        _LOGGER.exception("Failed to save ML Flashpoint checkpoint. Skipping saving and continuing.")
    return None
