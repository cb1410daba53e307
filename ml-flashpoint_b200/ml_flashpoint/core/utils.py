"""Environment flags, node counting and timing helpers (reference: core/utils.py:27-159)."""

import logging
import os
import time
from contextlib import contextmanager

import torch
import torch.distributed as dist

_ENV_PREFIX = "MLFLASHPOINT"


def get_env_var_prefix() -> str:
    return _ENV_PREFIX


def _env(name: str, default):
    return os.environ.get(f"{_ENV_PREFIX}_{name}", default)


def get_env_val_bool(env_var_name: str, default_val: bool) -> bool:
    """``MLFLASHPOINT_<name>`` read as "true"/"false" (any case); anything else is False."""
    return str(_env(env_var_name, default_val)).lower() == "true"


def get_env_val_str(env_var_name: str, default_val: str) -> str:
    return _env(env_var_name, default_val)


def get_env_val_int(env_var_name: str, default_val: int) -> int:
    raw = _env(env_var_name, default_val)
    if raw is None:
        return default_val
    try:
        return int(raw)
    except ValueError:
        return default_val


def get_accelerator_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def get_num_of_nodes() -> int:
    """Node count from ``NNODES``, then ``SLURM_NNODES``, then world size / GPUs per node."""
    for var in ("NNODES", "SLURM_NNODES"):
        if var in os.environ:
            return int(os.environ[var])
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    world = dist.get_world_size()
    per_node = get_accelerator_count()
    if per_node == 0:
        raise RuntimeError("torch.cuda.device_count() returned 0.")
    if world % per_node:
        raise RuntimeError(
            f"Inconsistent setup: world_size ({world}) is not evenly divisible by the GPU count per node ({per_node})."
        )
    return world // per_node


@contextmanager
def log_execution_time(logger: logging.Logger, name: str, level: int = logging.DEBUG):
    """Context manager / decorator logging ``"<name> took <seconds>s"`` (4 decimals).

    Log post-processing keys on this exact line shape.
    """
    t0 = time.perf_counter()
    try:
        yield
    finally:
        logger.log(level, "%s took %.4fs", name, time.perf_counter() - t0)
