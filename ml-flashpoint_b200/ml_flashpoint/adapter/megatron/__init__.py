"""Megatron-LM ``dist_checkpointing`` strategies backed by the B200 data path (needs megatron-core)."""

from ml_flashpoint.adapter.megatron.save_utils import (
    save_local_aware_megatron_checkpoint as save_local_aware_megatron_checkpoint,
)
