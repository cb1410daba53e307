"""Minimal stand-ins for the megatron-core symbols the Megatron adapter imports.

megatron-core is not installed where these tests run (the reference's own tests mock it too).
The stand-ins implement the contract the adapter relies on, with identity conversions: an MCore
"sharded state dict" here is already a flat DCP state dict.
"""

import dataclasses
import sys
import types
from typing import Any, Optional, Tuple

import torch
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner


class AsyncRequest:
    def __init__(self, async_fn, async_fn_args, finalize_fns, async_fn_kwargs=None):
        self.async_fn = async_fn
        self.async_fn_args = async_fn_args
        self.async_fn_kwargs = async_fn_kwargs or {}
        self.finalize_fns = list(finalize_fns)
        self.is_frozen = False

    def add_finalize_fn(self, fn):
        self.finalize_fns.append(fn)

    def execute_sync(self):
        self.async_fn(*self.async_fn_args, **self.async_fn_kwargs)
        for fn in self.finalize_fns:
            fn()


class AsyncSaveShardedStrategy:
    def __init__(self, backend, version):
        self.backend, self.version = backend, version

    def save(self, sharded_state_dict, checkpoint_dir):
        self.async_save(sharded_state_dict, checkpoint_dir).execute_sync()


class LoadShardedStrategy:
    pass


class MCoreSavePlanner(DefaultSavePlanner):
    def __init__(self, can_run_decentralized_global_plan=True, **kw):
        super().__init__(**kw)


class MCoreLoadPlanner(DefaultLoadPlanner):
    pass


@dataclasses.dataclass
class ShardedTensor:
    """Field-compatible stand-in for megatron-core's sharded tensor record."""

    key: str
    data: Optional[torch.Tensor] = dataclasses.field(default=None, repr=False)
    dtype: Optional[torch.dtype] = None
    local_shape: Tuple[int, ...] = ()
    global_shape: Tuple[int, ...] = ()
    global_offset: Tuple[int, ...] = ()
    axis_fragmentations: Optional[Tuple[int, ...]] = None
    replica_id: Any = 0
    prepend_axis_num: int = 0
    allow_shape_mismatch: bool = False
    flattened_range: Optional[slice] = None

    @classmethod
    def from_rank_offsets(cls, key, data, *rank_offsets, replica_id=0, prepend_axis_num=0, flattened_range=None, **init_kwargs):
        shape = tuple(data.shape)
        global_shape, global_offset, fragmentations = list(shape), [0] * len(shape), [1] * len(shape)
        for axis, rank_offset, fragmentation in rank_offsets:
            global_shape[axis] = shape[axis] * fragmentation
            global_offset[axis] = shape[axis] * rank_offset
            fragmentations[axis] = fragmentation
        return cls(
            key, data, data.dtype, shape, tuple(global_shape), tuple(global_offset), tuple(fragmentations),
            replica_id, prepend_axis_num, flattened_range=flattened_range, **init_kwargs,
        )

    def without_data(self):
        return dataclasses.replace(self, data=None)


@dataclasses.dataclass
class ShardedObject:
    """Field-compatible stand-in for megatron-core's sharded non-tensor record."""

    key: str
    data: Any = None
    global_shape: Tuple[int, ...] = (1,)
    global_offset: Tuple[int, ...] = (0,)
    replica_id: Any = 0

    @property
    def unique_key(self):
        return f"{self.key}/shard_{'.'.join(map(str, self.global_offset))}_{'.'.join(map(str, self.global_shape))}"

    @classmethod
    def empty_from_unique_key(cls, unique_key, replica_id=0):
        key, sep, shard = unique_key.rpartition("/")
        if not sep or not shard.startswith("shard_"):
            raise ValueError(f"'{unique_key}' is not the unique key of a sharded object")
        offset, shape = shard[len("shard_"):].split("_")
        return cls(key, None, tuple(map(int, shape.split("."))), tuple(map(int, offset.split("."))), replica_id)

    def without_data(self):
        return dataclasses.replace(self, data=None)


class AsyncCallsQueue:
    """Runs the async part at once and keeps finalization for ``maybe_finalize_async_calls``."""

    def __init__(self, persistent=False):
        self.persistent = persistent
        self._waiting = []
        self._count = 0
        self.closed = False

    def schedule_async_request(self, request):
        request.async_fn(*request.async_fn_args, **request.async_fn_kwargs)
        self._count += 1
        self._waiting.append((self._count, request))
        return self._count

    def get_num_unfinalized_calls(self):
        return len(self._waiting)

    def maybe_finalize_async_calls(self, blocking=False):
        done = []
        for index, request in self._waiting:
            for fn in request.finalize_fns:
                fn()
            done.append(index)
        self._waiting = []
        return done

    def close(self):
        self.closed = True


class _Delegating:
    def __init__(self, inner):
        self.base_strategy = inner

    def __getattr__(self, name):
        return getattr(self.base_strategy, name)


def _dist_load(sharded_state_dict, checkpoint_dir, sharded_strategy, common_strategy):
    import os

    state = torch.load(os.path.join(checkpoint_dir, "common.pt"), weights_only=False)
    state.update(sharded_strategy.load(sharded_state_dict, checkpoint_dir))
    return state


def install_nemo():
    """Stand-ins for the lightning / nemo symbols the NeMo adapter imports."""
    import dataclasses
    from pathlib import Path
    from typing import Optional

    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    class Callback:
        pass

    class CheckpointIO:
        pass

    class AsyncCompatibleCheckpointIO(CheckpointIO):
        pass

    class AsyncFinalizableCheckpointIO(CheckpointIO):
        """Wrapper that forwards to the wrapped checkpoint IO, as NeMo's does."""

        def __init__(self, checkpoint_io):
            self.checkpoint_io = checkpoint_io

        def save_checkpoint(self, checkpoint, path, storage_options=None):
            return self.checkpoint_io.save_checkpoint(checkpoint, path, storage_options)

        def load_checkpoint(self, path, *args, **kwargs):
            return self.checkpoint_io.load_checkpoint(path, *args, **kwargs)

        def remove_checkpoint(self, path):
            return self.checkpoint_io.remove_checkpoint(path)

        def teardown(self):
            self.torn_down = True

    class MegatronCheckpointIO(AsyncCompatibleCheckpointIO):
        def __init__(self):
            self.calls = []

        def save_checkpoint(self, checkpoint, path, storage_options=None):
            self.calls.append(("save", str(path)))
            return AsyncRequest(lambda: None, (), [])

        def load_checkpoint(self, path, sharded_state_dict=None, map_location=None, **kwargs):
            self.calls.append(("load", str(path)))
            return {"from": "fallback"}

        def remove_checkpoint(self, path):
            self.calls.append(("remove", str(path)))

        def load_content_metadata(self, path=None, preloaded_state_dict=None):
            return {"from": "fallback"}

    class MegatronStrategy:
        def __init__(self, checkpoint_io):
            self.checkpoint_io = checkpoint_io
            self.barriers = []

        def barrier(self, name=None):
            self.barriers.append(name)

    class Trainer:
        # class-level names so that a mock built with this class as its spec has them
        strategy = None
        callbacks = ()
        global_rank = local_rank = node_rank = global_step = current_epoch = 0
        world_size = num_nodes = num_devices = 1
        model = lightning_module = optimizers = None

        def __init__(self, strategy, callbacks=(), global_rank=0, local_rank=0):
            self.strategy, self.callbacks = strategy, list(callbacks)
            self.global_rank, self.local_rank, self.global_step = global_rank, local_rank, 0
            self.saved = []

        def save_checkpoint(self, path, storage_options=None):
            self.saved.append((path, storage_options))

    @dataclasses.dataclass
    class RestoreConfig:
        path: str
        load_model_state: bool = True
        load_optim_state: bool = False
        load_artifacts: bool = True

    @dataclasses.dataclass(kw_only=True)
    class AutoResume:
        restore_config: Optional[RestoreConfig] = None
        resume_from_directory: Optional[str] = None
        resume_from_path: Optional[str] = None
        resume_if_exists: bool = False
        resume_past_end: bool = False
        resume_ignore_no_checkpoint: bool = False
        fallback_path: Optional[Path] = None

        def _find_trainer_ckpt_path(self):
            return self.fallback_path

    class TrainerContext:
        @classmethod
        def from_trainer(cls, trainer):
            return cls()

        def io_dump(self, path, yaml_attrs=None):
            import os

            os.makedirs(path, exist_ok=True)
            with open(os.path.join(path, "model.yaml"), "w") as f:
                f.write("model: stub\n")

    pl = module("lightning")
    plp = module("lightning.pytorch", Trainer=Trainer, LightningModule=object)
    cbs = module("lightning.pytorch.callbacks", Callback=Callback)
    plp.callbacks = cbs
    pl.pytorch = plp
    module("lightning.pytorch.utilities")
    module("lightning.pytorch.utilities.types", STEP_OUTPUT=object)
    module("lightning.fabric")
    module("lightning.fabric.utilities")
    module("lightning.fabric.utilities.types", _PATH=str)
    module("nemo")
    module("nemo.utils")
    module("nemo.utils.callbacks")
    module(
        "nemo.utils.callbacks.dist_ckpt_io",
        AsyncCompatibleCheckpointIO=AsyncCompatibleCheckpointIO, AsyncFinalizableCheckpointIO=AsyncFinalizableCheckpointIO,
    )
    io_mod = module("nemo.lightning.io", ConnectorMixin=object)
    nl = module("nemo.lightning", AutoResume=AutoResume, io=io_mod)
    sys.modules["nemo"].lightning = nl
    module("nemo.lightning.io.pl", MegatronCheckpointIO=MegatronCheckpointIO, TrainerContext=TrainerContext, _fix_tensors_device=lambda sd: None)
    module("nemo.lightning.pytorch")
    module("nemo.lightning.pytorch.trainer", Trainer=Trainer)
    strategies = module("nemo.lightning.pytorch.strategies", MegatronStrategy=MegatronStrategy, FSDPStrategy=type("FSDPStrategy", (), {}))
    strategies.__path__ = []  # a package: it has the submodule below
    strategies.utils = module("nemo.lightning.pytorch.strategies.utils", RestoreConfig=RestoreConfig)
    sys.modules["megatron.core.dist_checkpointing.strategies.async_utils"].AsyncCallsQueue = AsyncCallsQueue
    sys.modules["megatron.core.dist_checkpointing.strategies.common"].TorchCommonLoadStrategy = type("TorchCommonLoadStrategy", (), {})
    sys.modules["megatron.core.dist_checkpointing"].load = _dist_load
    sys.modules["megatron.core"].dist_checkpointing = sys.modules["megatron.core.dist_checkpointing"]
    module(
        "megatron.core.dist_checkpointing.strategies.fully_parallel",
        FullyParallelSaveStrategyWrapper=type("FullyParallelSaveStrategyWrapper", (_Delegating,), {}),
        FullyParallelLoadStrategyWrapper=type("FullyParallelLoadStrategyWrapper", (_Delegating,), {}),
    )


def install():
    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    module("megatron")
    module("megatron.core")
    module("megatron.core.dist_checkpointing")
    module(
        "megatron.core.dist_checkpointing.mapping",
        ShardedStateDict=dict, StateDict=dict, ShardedTensor=ShardedTensor, ShardedObject=ShardedObject,
    )
    module("megatron.core.dist_checkpointing.strategies")
    module("megatron.core.dist_checkpointing.strategies.async_utils", AsyncRequest=AsyncRequest)
    module(
        "megatron.core.dist_checkpointing.strategies.base",
        AsyncSaveShardedStrategy=AsyncSaveShardedStrategy, LoadShardedStrategy=LoadShardedStrategy,
    )
    module("megatron.core.dist_checkpointing.strategies.common", COMMON_STATE_FNAME="common.pt")
    module(
        "megatron.core.dist_checkpointing.strategies.torch",
        MCoreSavePlanner=MCoreSavePlanner,
        MCoreLoadPlanner=MCoreLoadPlanner,
        _replace_state_dict_keys_with_sharded_keys=lambda sharded_state_dict, keep_only_main_replica=False: (sharded_state_dict, {}, {}),
        _replace_sharded_keys_with_state_dict_keys=lambda sd, flat, rename: sd,
        _restore_dict_types=lambda sd, original: None,
        _unwrap_pyt_sharded_tensor=lambda v: v,
        mcore_to_pyt_state_dict=lambda sd, is_loading=False: sd,
    )
    sdu = module(
        "megatron.core.dist_checkpointing.state_dict_utils",
        save_preprocess=lambda ckpt: ({k: v for k, v in ckpt.items() if isinstance(v, torch.Tensor)},
                                      {k: v for k, v in ckpt.items() if not isinstance(v, torch.Tensor)}),
    )
    sys.modules["megatron.core.dist_checkpointing"].state_dict_utils = sdu
