"""Megatron-LM and NeMo adapter flows with the CUDA engine and device tensors.

The adapters' host logic is tested on the CPU with the numpy engine double; here the same flows move
their bytes with the pack / unpack kernels: the trainer-process save (``async_save`` returns with
the sources safe to mutate), the finalize functions, the load strategies, and the checkpoint IO
routing. megatron-core / nemo / lightning are not installed: stand-in modules provide their names.
"""

import concurrent.futures
import os
import sys

import pytest
import torch
import torch.multiprocessing as torch_mp

import cases
import megatron_standins
import mlf_oracle as oracle
from helpers import case_to_device, make_loader, make_saver, tensor_bytes

pytestmark = pytest.mark.gpu


class _LocalReplication:
    """Single node: nothing to send, the buffer is closed at once (as the reference does)."""

    def async_replicate(self, buffer_io):
        buffer_io.close()
        return []

    def shutdown(self):
        pass


@pytest.fixture
def stack(monkeypatch, shm_path):
    megatron_standins.install()
    megatron_standins.install_nemo()
    monkeypatch.setenv("MLFLASHPOINT_DISABLE_DIST", "true")
    monkeypatch.setenv("NNODES", "1")
    monkeypatch.setattr(torch.distributed, "get_node_local_rank", lambda *a, **k: 0)
    monkeypatch.setattr(torch.distributed, "get_rank", lambda *a, **k: 0)
    monkeypatch.setattr(torch.distributed, "broadcast_object_list", lambda box, src=0: None)
    import importlib

    for name in [m for m in sys.modules if m.startswith("ml_flashpoint.adapter.nemo")]:
        del sys.modules[name]  # bind to this test's stand-in classes
    from ml_flashpoint.adapter.megatron.load_strategies import MLFlashpointMegatronLoadStrategy
    from ml_flashpoint.adapter.megatron.save_strategies import MLFlashpointMegatronAsyncSaveStrategy
    from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    CheckpointObjectManager._worker_pool = None
    engine = CudaCopyEngine(mode="staged")
    pool = BufferPoolConfig(str(shm_path / "pool"), 0, 2, 4 << 20, register_cuda=True)
    replication = _LocalReplication()
    saver, com = make_saver(copy_engine=engine, pool_config=pool, replication_manager=replication)
    manager = torch_mp.Manager()
    future = concurrent.futures.Future()
    future.set_result(manager)
    save = MLFlashpointMegatronAsyncSaveStrategy(MemoryStorageWriter(saver, future), use_cached_ckpt_structure=True)
    load = MLFlashpointMegatronLoadStrategy(replication, make_loader(com, copy_engine=engine))
    checkpoint_io = importlib.import_module("ml_flashpoint.adapter.nemo.checkpoint_io")
    yield {"save": save, "load": load, "com": com, "engine": engine, "io_module": checkpoint_io, "base": str(shm_path / "mlf")}
    manager.shutdown()
    com.teardown_pool()


def test_megatron_async_save_packs_in_the_trainer_process_and_loads_back(stack):
    save, load = stack["save"], stack["load"]
    for step in (10, 20):  # the second save finds the pool buffers already sized and page-locked
        state = dict(case_to_device(cases.CASES["views"](), "cuda")["tensors"])  # seeded: same values each time
        originals = {k: v.clone() for k, v in state.items()}
        ckpt = os.path.join(stack["base"], f"step-{step}_ckpt")
        request = save.async_save(state, ckpt)
        for v in state.values():
            (v._base if v._base is not None else v).zero_()  # the trainer moves on as soon as async_save has returned
        torch.cuda.synchronize()
        request.async_fn(*request.async_fn_args, **request.async_fn_kwargs)
        for fn in request.finalize_fns:
            fn()
        assert os.path.exists(os.path.join(ckpt, ".metadata"))
        objects = sorted(f for f in os.listdir(ckpt) if f.endswith(".distcp"))
        assert len(objects) == 1
        cpu_case = {"tensors": {k: v.cpu() for k, v in originals.items()}, "blobs": {}, "bucket_count": 1}
        ((_, want, _),) = oracle.save_case(cpu_case)
        with open(os.path.join(ckpt, objects[0]), "rb") as f:
            assert f.read() == want
        fresh = {k: torch.full_like(v, 7) for k, v in originals.items()}
        loaded = load.load(fresh, ckpt)
        for k, v in originals.items():
            assert loaded[k].is_cuda and tensor_bytes(loaded[k]) == tensor_bytes(v), k


def test_nemo_checkpoint_io_saves_and_loads_through_the_kernels(stack):
    fallback = sys.modules["nemo.lightning.io.pl"].MegatronCheckpointIO()
    strategy = sys.modules["nemo.lightning.pytorch.strategies"].MegatronStrategy(fallback)
    trainer = sys.modules["nemo.lightning.pytorch.trainer"].Trainer(strategy)
    io = stack["io_module"].MLFlashpointCheckpointIO(
        stack["base"], fallback, stack["com"], stack["save"], stack["load"], trainer, async_save=True
    )
    tensors = dict(case_to_device(cases.CASES["two_buckets"](), "cuda")["tensors"])
    checkpoint = dict(tensors)
    checkpoint["iteration"] = 30
    ckpt = os.path.join(stack["base"], "step-30_ckpt")
    request = io.save_checkpoint(checkpoint, ckpt, storage_options={"content_metadata": {"mcore": "0.13"}})
    assert request is not None and not fallback.calls
    request.execute_sync()
    assert os.path.exists(os.path.join(ckpt, ".metadata")) and os.path.exists(os.path.join(ckpt, "common.pt"))
    fresh = {k: torch.zeros_like(v) for k, v in tensors.items()}
    loaded = io.load_checkpoint(ckpt, sharded_state_dict=fresh)
    assert loaded["iteration"] == 30
    for k, v in tensors.items():
        assert loaded[k].is_cuda and tensor_bytes(loaded[k]) == tensor_bytes(v), k
    io.remove_checkpoint(ckpt)
    assert not os.path.exists(ckpt)
