"""Minimal stand-ins for the megatron-core symbols the Megatron adapter imports.

megatron-core is not installed where these tests run (the reference's own tests mock it too).
The stand-ins implement the contract the adapter relies on, with identity conversions: an MCore
"sharded state dict" here is already a flat DCP state dict.
"""

import sys
import types

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


class ShardedTensor:
    def __init__(self, key, data):
        self.key, self.data = key, data

    @classmethod
    def from_rank_offsets(cls, key, data, *offsets):
        return cls(key, data)

    def without_data(self):
        return ShardedTensor(self.key, None)


class ShardedObject:
    def __init__(self, key):
        self.unique_key = key

    @classmethod
    def empty_from_unique_key(cls, key):
        return cls(key)


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
        def __init__(self, checkpoint_io):
            self.checkpoint_io = checkpoint_io

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
        def __init__(self, strategy, callbacks=(), global_rank=0, local_rank=0):
            self.strategy, self.callbacks = strategy, list(callbacks)
            self.global_rank, self.local_rank, self.global_step = global_rank, local_rank, 0
            self.saved = []

        def save_checkpoint(self, path, storage_options=None):
            self.saved.append((path, storage_options))

    @dataclasses.dataclass(kw_only=True)
    class AutoResume:
        resume_if_exists: bool = False
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
    module("nemo.lightning.pytorch.strategies", MegatronStrategy=MegatronStrategy)
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
