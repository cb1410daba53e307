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
        self.finalize_fns = finalize_fns
        self.is_frozen = False

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
