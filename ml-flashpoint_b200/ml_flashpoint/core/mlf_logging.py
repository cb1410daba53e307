"""Rank- and step-stamped logging (reference: core/mlf_logging.py:31-111).

Line prefix: ``[MLF <time> <LEVEL> Step=<step> Rank=<rank> <logger>:<line>]``. The step lives in
a process-shared integer so that worker processes forked from the trainer log the same step.
"""

import logging
import multiprocessing
import sys

import torch

from ml_flashpoint.core import utils

_MISSING_NONNEG_NUMERIC_VAL = -1
_TRAINING_STEP = multiprocessing.Value("i", _MISSING_NONNEG_NUMERIC_VAL)
_STATIC_RANK = _MISSING_NONNEG_NUMERIC_VAL

_FORMAT = "[MLF %(asctime)s %(levelname)s Step=%(curr_step)s Rank=%(rank)s %(name)s:%(lineno)d] %(message)s"


def update_training_step(new_val: int):
    with _TRAINING_STEP.get_lock():
        _TRAINING_STEP.value = new_val


def get_current_step() -> int:
    return _TRAINING_STEP.value


def setup_worker_logging(rank: int, step: int):
    """Pins the rank shown in this process's log lines (workers have no process group)."""
    global _STATIC_RANK
    _STATIC_RANK = rank
    update_training_step(step)


class TrainingContextFormatter(logging.Formatter):
    def format(self, record):
        if _STATIC_RANK != _MISSING_NONNEG_NUMERIC_VAL:
            record.rank = _STATIC_RANK
        elif torch.distributed.is_initialized():
            record.rank = torch.distributed.get_rank()
        else:
            record.rank = _MISSING_NONNEG_NUMERIC_VAL
        record.curr_step = _TRAINING_STEP.value
        return super().format(record)


def get_logger(name: str, stream=sys.stderr) -> logging.Logger:
    """Logger with the MLF prefix; level from ``MLFLASHPOINT_LOG_LEVEL`` (default DEBUG)."""
    logger = logging.getLogger(name)
    if not logger.handlers:
        handler = logging.StreamHandler(stream=stream)
        handler.setFormatter(TrainingContextFormatter(_FORMAT))
        logger.addHandler(handler)
        wanted = utils.get_env_val_str("LOG_LEVEL", "DEBUG").upper()
        logger.setLevel(logging._nameToLevel.get(wanted, logging.DEBUG))
    logger.propagate = False
    return logger
