"""Lightning ``CheckpointIO`` that routes saves and loads between ML Flashpoint and a long-term strategy.

Same classes as the reference's adapter/nemo/checkpoint_io.py:64-477:

* ``MLFlashpointCheckpointIO`` decides by path prefix: anything under the ML Flashpoint base
  container is saved through the Megatron strategies of this package (pack kernel + transfer queued
  in the trainer process), everything else goes to the wrapped ``MegatronCheckpointIO``.
* ``MLFlashpointAsyncFinalizableCheckpointIO`` keeps a separate, persistent async-call queue for ML
  Flashpoint saves, so that their finalization (which frees the previous step's buffers) is not
  held up behind a slow long-term save.
"""

import logging
import os
import threading
from typing import Any, Optional, Union, cast

import torch
from lightning.fabric.utilities.types import _PATH
from megatron.core import dist_checkpointing as mcore_dist_checkpointing
from megatron.core.dist_checkpointing.strategies.async_utils import AsyncCallsQueue
from megatron.core.dist_checkpointing.strategies.async_utils import AsyncRequest as MegatronAsyncRequest
from megatron.core.dist_checkpointing.strategies.common import COMMON_STATE_FNAME, TorchCommonLoadStrategy
from nemo.lightning.io.pl import MegatronCheckpointIO, TrainerContext, _fix_tensors_device
from nemo.lightning.pytorch.trainer import Trainer
from nemo.utils.callbacks.dist_ckpt_io import AsyncCompatibleCheckpointIO, AsyncFinalizableCheckpointIO

from ml_flashpoint.adapter.megatron.load_strategies import MLFlashpointMegatronLoadStrategy
from ml_flashpoint.adapter.megatron.save_strategies import MLFlashpointMegatronAsyncSaveStrategy
from ml_flashpoint.adapter.megatron.save_utils import save_local_aware_megatron_checkpoint
from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


def _is_ml_flashpoint_checkpoint(flashpoint_base_dir: Union[str, CheckpointContainerId], path: _PATH) -> bool:
    """ML Flashpoint checkpoints are exactly the paths under the base container."""
    return str(path).startswith(str(flashpoint_base_dir))


class MLFlashpointCheckpointIO(AsyncCompatibleCheckpointIO):
    def __init__(
        self,
        flashpoint_base_path: Union[str, CheckpointContainerId],
        alt_checkpoint_io: MegatronCheckpointIO,
        chkpt_obj_manager: CheckpointObjectManager,
        save_strategy: MLFlashpointMegatronAsyncSaveStrategy,
        load_strategy: MLFlashpointMegatronLoadStrategy,
        trainer: Trainer,
        async_save: bool = True,
        always_save_context: bool = False,
    ):
        self.flashpoint_base_dir = CheckpointContainerId(flashpoint_base_path)
        self.fallback_checkpoint_io = alt_checkpoint_io
        self.chkpt_obj_manager = chkpt_obj_manager
        self.save_strategy = save_strategy
        self.load_strategy = load_strategy
        self.trainer = trainer
        self.async_save = async_save
        self.always_save_context = always_save_context

    def _mine(self, path: _PATH) -> bool:
        return _is_ml_flashpoint_checkpoint(self.flashpoint_base_dir, path)

    @log_execution_time(logger=_LOGGER, name="MLFlashpointCheckpointIO.save_checkpoint", level=logging.INFO)
    def save_checkpoint(
        self, checkpoint: dict[str, Any], path: _PATH, storage_options: Optional[Any] = None
    ) -> Optional[MegatronAsyncRequest]:
        """Returns the ``AsyncRequest`` of an async ML Flashpoint save, else what the fallback returns / None."""
        if not self._mine(path):
            return self.fallback_checkpoint_io.save_checkpoint(checkpoint, path, storage_options=storage_options)
        content_metadata = (storage_options or {}).get("content_metadata")
        if content_metadata is not None:
            # travels in common.pt: the stub metadata.json cannot carry it (see load_content_metadata)
            checkpoint["content_metadata"] = content_metadata
        request = save_local_aware_megatron_checkpoint(
            checkpoint=checkpoint, checkpoint_dir=path, save_strategy=self.save_strategy, async_save=self.async_save
        )
        if self.always_save_context:
            self._save_context(path)
        return request

    @log_execution_time(logger=_LOGGER, name="MLFlashpointCheckpointIO._save_context", level=logging.INFO)
    def _save_context(self, path: _PATH) -> Optional[threading.Thread]:
        """Dumps the trainer context on global rank 0 and hands the files to every other node's first rank."""
        context_path = os.path.join(path, "context")
        files: dict[str, bytes] = {}
        if torch.distributed.get_rank() == 0:
            try:
                TrainerContext.from_trainer(self.trainer).io_dump(context_path, yaml_attrs=["model"])
                for root, _, names in os.walk(context_path):
                    for name in names:
                        full = os.path.join(root, name)
                        with open(full, "rb") as f:
                            files[os.path.relpath(full, context_path)] = f.read()
            except Exception as e:
                _LOGGER.warning(f"Failed to dump/read context for broadcast: {e}")
        box = [files]
        torch.distributed.broadcast_object_list(box, src=0)
        files = box[0]
        if torch.distributed.get_node_local_rank() != 0 or torch.distributed.get_rank() == 0:
            return None

        def _write(target: str, data: dict):
            try:
                os.makedirs(target, exist_ok=True)
                for rel, content in data.items():
                    full = os.path.join(target, rel)
                    os.makedirs(os.path.dirname(full), exist_ok=True)
                    with open(full, "wb") as f:
                        f.write(content)
            except Exception as e:
                _LOGGER.warning(f"Failed to write propagated context: {e}")

        worker = threading.Thread(target=_write, args=(context_path, files))
        worker.start()
        return worker

    @log_execution_time(logger=_LOGGER, name="MLFlashpointCheckpointIO.load_checkpoint", level=logging.INFO)
    def load_checkpoint(
        self, path: _PATH, sharded_state_dict=None, map_location: Optional[Any] = None, **kwargs
    ) -> dict[str, Any]:
        """Extra keyword arguments NeMo passes are forwarded to the fallback and ignored here."""
        if not self._mine(path):
            return self.fallback_checkpoint_io.load_checkpoint(
                path, sharded_state_dict=sharded_state_dict, map_location=map_location, **kwargs
            )
        try:
            state_dict = mcore_dist_checkpointing.load(
                sharded_state_dict=sharded_state_dict,
                checkpoint_dir=str(path),
                sharded_strategy=self.load_strategy,
                common_strategy=TorchCommonLoadStrategy(),
            )
            if torch.cuda.is_initialized():
                _fix_tensors_device(state_dict)
            return state_dict
        except Exception:
            _LOGGER.exception(
                "Failed to load ML Flashpoint checkpoint. If this problem persists, "
                "consider disabling ML Flashpoint or "
                "deleting the Flashpoint base container across all training nodes. "
                "Re-raising the exception."
            )
            raise

    @log_execution_time(logger=_LOGGER, name="MLFlashpointCheckpointIO.remove_checkpoint", level=logging.INFO)
    def remove_checkpoint(self, path: _PATH) -> None:
        if self._mine(path):
            self.chkpt_obj_manager.delete_container(CheckpointContainerId(path))
        else:
            self.fallback_checkpoint_io.remove_checkpoint(path)

    @log_execution_time(logger=_LOGGER, name="MLFlashpointCheckpointIO.load_content_metadata", level=logging.INFO)
    def load_content_metadata(self, path: Optional[_PATH] = None, preloaded_state_dict: Optional[dict] = None) -> dict:
        """Content metadata of an ML Flashpoint checkpoint lives in ``common.pt``: its ``metadata.json``
        is only the stub Megatron's validation wants."""
        if not self._mine(path):
            return self.fallback_checkpoint_io.load_content_metadata(path, preloaded_state_dict)
        if preloaded_state_dict is not None:
            return preloaded_state_dict.get("content_metadata")
        common = os.path.join(path, COMMON_STATE_FNAME)
        if os.path.exists(common):
            state = torch.load(common, map_location="cpu", weights_only=False)
            if "content_metadata" in state:
                return state["content_metadata"]
        _LOGGER.warning("Checkpoint at %s exists but does not contain 'content_metadata'.", path)
        return None


class MLFlashpointAsyncFinalizableCheckpointIO(AsyncFinalizableCheckpointIO):
    """Use together with NeMo's ``AsyncFinalizerCallback``, which drives ``maybe_finalize_save_checkpoint``."""

    def __init__(self, checkpoint_io: AsyncCompatibleCheckpointIO):
        if not isinstance(checkpoint_io, AsyncCompatibleCheckpointIO) or not isinstance(checkpoint_io, MLFlashpointCheckpointIO):
            raise ValueError("Incompatible wrapped checkpoint_io type: %s", type(checkpoint_io))
        super().__init__(checkpoint_io)
        self._mlf_async_calls_queue = AsyncCallsQueue(persistent=True)
        self._alt_async_calls_queue = AsyncCallsQueue()

    @property
    def mlf_checkpoint_io(self) -> MLFlashpointCheckpointIO:
        return cast(MLFlashpointCheckpointIO, self.checkpoint_io)

    def _queue_for(self, path: _PATH):
        if _is_ml_flashpoint_checkpoint(self.mlf_checkpoint_io.flashpoint_base_dir, path):
            return "ml_flashpoint", self._mlf_async_calls_queue
        return "alternative", self._alt_async_calls_queue

    @log_execution_time(logger=_LOGGER, name="MLFlashpointAsyncFinalizableCheckpointIO.save_checkpoint", level=logging.INFO)
    def save_checkpoint(self, checkpoint: dict[str, Any], path: _PATH, storage_options: Optional[Any] = None) -> None:
        """Schedules the wrapped IO's ``AsyncRequest`` on the queue that matches the path. A
        ``finalize_fn`` in ``storage_options`` is consumed here and runs after the request's own."""
        extra_finalize = (storage_options or {}).pop("finalize_fn", None)
        request = self.checkpoint_io.save_checkpoint(checkpoint, path, storage_options)
        if extra_finalize is not None:
            request.add_finalize_fn(extra_finalize)
        kind, calls = self._queue_for(path)
        index = calls.schedule_async_request(request)
        _LOGGER.debug("Scheduled an async call #%d for path '%s' on '%s' queue", index, path, kind)

    @log_execution_time(
        logger=_LOGGER, name="MLFlashpointAsyncFinalizeCheckpointIO.maybe_finalize_save_checkpoint", level=logging.INFO
    )
    def maybe_finalize_save_checkpoint(self, blocking: bool = False) -> bool:
        """Finalizes every async save that has completed on all ranks (all of them if ``blocking``)."""
        queues = (self._mlf_async_calls_queue, self._alt_async_calls_queue)
        if all(q.get_num_unfinalized_calls() == 0 for q in queues):
            return False
        finalized = 0
        for q in queues:
            finalized += len(q.maybe_finalize_async_calls(blocking))
        return finalized > 0

    @log_execution_time(logger=_LOGGER, name="MLFlashpointAsyncFinalizeCheckpointIO.teardown")
    def teardown(self) -> None:
        super().teardown()
        pending = self._mlf_async_calls_queue.get_num_unfinalized_calls() + self._alt_async_calls_queue.get_num_unfinalized_calls()
        if pending > 0:
            _LOGGER.warning("Some async checkpoint saves might be not finalized properly.")
        # the buffer pool lives where buffers are acquired, which here is this (the trainer) process
        self.mlf_checkpoint_io.chkpt_obj_manager.teardown_pool()
        try:
            # a writer process that created a pool of its own drops it as well
            self._mlf_async_calls_queue.schedule_async_request(
                MegatronAsyncRequest(
                    async_fn=self.mlf_checkpoint_io.chkpt_obj_manager.teardown_pool, async_fn_args=(), finalize_fns=[]
                )
            )
        except Exception:
            pass
        if hasattr(self._mlf_async_calls_queue, "close"):
            self._mlf_async_calls_queue.close()
            caller = getattr(self._mlf_async_calls_queue, "persistent_caller", None)
            if caller and hasattr(caller, "close"):
                caller.close = lambda: None  # closing twice would raise inside Megatron
