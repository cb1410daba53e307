"""Lightning callback that logs ``event=<hook>`` for the training-loop hooks, for timeline analysis
of logs (reference: adapter/nemo/event_logging_callback.py:26-162)."""

import lightning.pytorch as pl
from lightning.pytorch import callbacks as pl_callbacks

from ml_flashpoint.core.mlf_logging import get_logger

_LOGGER = get_logger(__name__)

_HOOKS = (
    "on_train_start",
    "on_train_end",
    "on_train_batch_start",
    "on_train_batch_end",
    "on_validation_batch_start",
    "on_validation_batch_end",
    "on_test_epoch_start",
    "on_test_epoch_end",
    "on_test_batch_start",
    "on_test_batch_end",
    "load_state_dict",
    "on_save_checkpoint",
    "on_load_checkpoint",
    "on_before_backward",
    "on_after_backward",
    "on_before_optimizer_step",
    "on_before_zero_grad",
)


class EventLoggingCallback(pl_callbacks.Callback):
    def _log_event(self, hook_name: str) -> None:
        _LOGGER.info(f"event={hook_name}")


def _make_hook(name: str):
    def hook(self, *args, **kwargs) -> None:
        self._log_event(name)

    hook.__name__ = name
    hook.__doc__ = f"Logs ``event={name}``."
    return hook


for _name in _HOOKS:
    setattr(EventLoggingCallback, _name, _make_hook(_name))
del _name
