"""Megatron-LM strategies against stand-in megatron modules (megatron-core is not installed here).

What is checked is this package's side of the contract: the ``AsyncRequest`` shape, that the
tensors are safe to mutate when ``async_save`` returns, that the finalize functions publish
results / metadata / finalization in order, plan caching, and a load through the load strategy.
"""

import concurrent.futures
import json
import os

import pytest
import torch
import torch.multiprocessing as torch_mp

import cases
import megatron_standins
from helpers import NumpyCopyEngine, make_loader, make_saver, tensor_bytes


@pytest.fixture
def strategies(monkeypatch, tmp_path):
    megatron_standins.install()
    monkeypatch.setenv("MLFLASHPOINT_DISABLE_DIST", "true")
    monkeypatch.setenv("NNODES", "1")
    monkeypatch.setattr(torch.distributed, "get_node_local_rank", lambda *a, **k: 0)
    from ml_flashpoint.adapter.megatron.load_strategies import MLFlashpointMegatronLoadStrategy
    from ml_flashpoint.adapter.megatron.save_strategies import MLFlashpointMegatronAsyncSaveStrategy
    from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter

    engine = NumpyCopyEngine()
    replicated = []

    class _Replication:  # single node: nothing to send, the buffer is closed at once (as upstream does)
        def async_replicate(self, buffer_io):
            replicated.append(buffer_io.buffer_obj.get_id())
            buffer_io.close()
            return []

    saver, com = make_saver(copy_engine=engine, replication_manager=_Replication())
    manager = torch_mp.Manager()
    fut = concurrent.futures.Future()
    fut.set_result(manager)
    writer = MemoryStorageWriter(saver, fut)
    save = MLFlashpointMegatronAsyncSaveStrategy(writer, use_cached_ckpt_structure=True)
    load = MLFlashpointMegatronLoadStrategy(None, make_loader(com, copy_engine=engine))
    yield save, load, saver
    manager.shutdown()


def test_async_save_request_and_load_round_trip(strategies, tmp_path):
    save, load, saver = strategies
    case = cases.CASES["gpt2_tiny"]()
    state = dict(case["tensors"])
    ckpt = str(tmp_path / "step-10_ckpt")
    request = save.async_save(state, ckpt)
    assert save.can_handle_sharded_objects() and save.thread_count == 1
    assert save.backend == "ml_flashpoint" and save.version == 1
    assert json.load(open(os.path.join(ckpt, "metadata.json"))) == {"sharded_backend": ""}
    assert os.path.exists(str(tmp_path / "step-10_ckpt__0__unfinished"))
    # nothing that crosses into the writer process may hold tensors
    assert set(request.async_fn_kwargs) == {"checkpoint_id", "rank", "step"}
    assert len(request.finalize_fns) == 4
    assert not os.path.exists(os.path.join(ckpt, ".metadata"))
    originals = {k: v.clone() for k, v in state.items()}
    for v in state.values():
        v.zero_()  # the trainer moves on as soon as async_save has returned
    request.async_fn(*request.async_fn_args, **request.async_fn_kwargs)
    for fn in request.finalize_fns:
        fn()
    assert os.path.exists(os.path.join(ckpt, ".metadata"))
    assert not os.path.exists(str(tmp_path / "step-10_ckpt__0__unfinished"))

    fresh = {k: torch.full_like(v, 7) for k, v in originals.items()}
    loaded = load.load(fresh, ckpt)
    for k, v in originals.items():
        assert tensor_bytes(loaded[k]) == tensor_bytes(v), k
    meta = load.load_tensors_metadata(ckpt)
    assert set(meta) == set(originals) and all(m.data is None for m in meta.values())
    assert set(load.load_sharded_metadata(ckpt)) == set(originals)
    assert load.can_handle_sharded_objects


def test_plan_is_reused_once_the_structure_has_repeated(strategies, tmp_path):
    save, _, _ = strategies
    state = dict(cases.CASES["two_buckets"]()["tensors"])
    seen = []
    for step in (1, 2, 3):
        save.async_save(state, str(tmp_path / f"step-{step}_ckpt")).execute_sync()
        seen.append(save._validated_cache_reuse)
    assert seen == [False, True, True]  # first save has nothing to compare with
    # older steps are removed by a detached `rm -rf`; give it a moment
    import time

    deadline = time.time() + 20
    while time.time() < deadline and os.path.exists(str(tmp_path / "step-1_ckpt")):
        time.sleep(0.05)
    assert not os.path.exists(str(tmp_path / "step-1_ckpt")) and os.path.exists(str(tmp_path / "step-3_ckpt"))


def test_save_utils_writes_common_state_and_swallows_failures(strategies, tmp_path):
    from ml_flashpoint.adapter.megatron import save_local_aware_megatron_checkpoint

    save, _, _ = strategies
    ckpt = str(tmp_path / "step-4_ckpt")
    checkpoint = {"w": torch.arange(6.0), "iteration": 4, "args": {"lr": 0.1}}
    request = save_local_aware_megatron_checkpoint(checkpoint, ckpt, save, async_save=True)
    assert request is not None
    assert torch.load(os.path.join(ckpt, "common.pt"), weights_only=False) == {"iteration": 4, "args": {"lr": 0.1}}
    request.execute_sync()

    class _Broken:
        def async_save(self, **kw):
            raise RuntimeError("no space left")

    assert save_local_aware_megatron_checkpoint(checkpoint, str(tmp_path / "step-5_ckpt"), _Broken()) is None
    assert save_local_aware_megatron_checkpoint(checkpoint, str(tmp_path / "step-6_ckpt"), save, async_save=False) is None
    assert os.path.exists(str(tmp_path / "step-6_ckpt" / ".metadata"))
