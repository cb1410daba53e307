"""Lightning callback that triggers an ML Flashpoint save every N steps.

Same surface as the reference's adapter/nemo/checkpoint_callback.py:44-200: the callback asks the
trainer to save ``<base>/step-<N>_ckpt`` with ``storage_options`` that mark the save as an ML
Flashpoint one; the checkpoint IO routes on the path prefix. At the end of training it drains
pending saves, shuts the replication manager down and (by default) removes the whole base container.
"""

import logging
from typing import Any, Optional, Union

import lightning.pytorch as pl
from lightning.pytorch import callbacks as pl_callbacks
from lightning.pytorch.utilities import types as pl_util_types
from nemo.utils.callbacks.dist_ckpt_io import AsyncFinalizableCheckpointIO

from ml_flashpoint.core import mlf_logging
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


class MLFlashpointMarker:
    """Type of the sentinel that marks a save as an ML Flashpoint save in ``storage_options``."""


ML_FLASHPOINT_TYPE = MLFlashpointMarker()
ML_FLASHPOINT_OPTS_KEY = "ML_FLASHPOINT_OPTS"


class MLFlashpointCheckpointCallback(pl_callbacks.Callback):
    def __init__(
        self,
        checkpoint_base_container: Union[str, CheckpointContainerId],
        every_n_steps: int,
        skip_every_n_steps: Optional[int] = None,
        enabled: bool = True,
        keep_mlf_checkpoint_on_train_end: bool = False,
    ):
        """``checkpoint_base_container`` must be unique per job run and equal to the one given to
        ``MLFlashpointAutoResume``. Steps divisible by ``skip_every_n_steps`` are left to the
        long-term checkpointing strategy."""
        self.base_container = CheckpointContainerId(checkpoint_base_container)
        self.every_n_steps = every_n_steps
        self.skip_every_n_steps = 0 if skip_every_n_steps is None else skip_every_n_steps
        self._enabled = enabled
        self._replication_manager = None
        self._keep_mlf_checkpoint_on_train_end = keep_mlf_checkpoint_on_train_end
        self._validate()

    @property
    def replication_manager(self):
        return self._replication_manager

    @replication_manager.setter
    def replication_manager(self, manager):
        # injected by the wrapper: users create the callback before the managers exist
        self._replication_manager = manager

    def _validate(self):
        if not isinstance(self.every_n_steps, int) or self.every_n_steps < 1:
            raise ValueError(f"every_n_steps must be a positive integer, got '{self.every_n_steps}' instead.")
        if not isinstance(self.skip_every_n_steps, int) or self.skip_every_n_steps < 0:
            raise ValueError(
                f"skip_every_n_steps must be a non-negative integer, got '{self.skip_every_n_steps}' instead."
            )

    def _format_checkpoint_version_container_id(self, step: int) -> CheckpointContainerId:
        return CheckpointContainerId.create_child(self.base_container, CheckpointContainerId.format_version_container(step))

    @log_execution_time(logger=_LOGGER, name="on_train_batch_end", level=logging.INFO)
    def on_train_batch_end(
        self,
        trainer: "pl.Trainer",
        pl_module: "pl.LightningModule",
        outputs: pl_util_types.STEP_OUTPUT,
        batch: Any,
        batch_idx: int,
    ) -> None:
        step = trainer.global_step
        mlf_logging.update_training_step(step)
        if not self._enabled:
            return
        if step % self.every_n_steps != 0:
            return
        if self.skip_every_n_steps > 0 and step % self.skip_every_n_steps == 0:
            _LOGGER.info("%s skipping save this step: '%d' (left to the long-term strategy)", type(self).__name__, step)
            return
        target = self._format_checkpoint_version_container_id(step)
        options = dict(ckpt_type=ML_FLASHPOINT_TYPE, step=step)
        _LOGGER.info("%s saving checkpoint path: '%s', ckpt_options: %s", type(self).__name__, target, options)
        trainer.save_checkpoint(target.data, storage_options={ML_FLASHPOINT_OPTS_KEY: options})

    @log_execution_time(logger=_LOGGER, name="on_train_end", level=logging.INFO)
    def on_train_end(self, trainer: "pl.Trainer", pl_module: "pl.LightningModule") -> None:
        checkpoint_io = trainer.strategy.checkpoint_io
        if isinstance(checkpoint_io, AsyncFinalizableCheckpointIO):
            checkpoint_io.maybe_finalize_save_checkpoint(blocking=True)
        trainer.strategy.barrier("mlf_cleanup_barrier")
        if self.replication_manager is not None:
            self.replication_manager.shutdown()
        if trainer.local_rank == 0:
            if self._keep_mlf_checkpoint_on_train_end:
                _LOGGER.info("Local rank 0: keeping ML Flashpoint checkpoints (keep_mlf_checkpoint_on_train_end).")
            else:
                trainer.strategy.checkpoint_io.remove_checkpoint(self.base_container.data)
