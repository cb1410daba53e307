"""NeMo 2.0 / Lightning adapter against stand-in nemo, lightning and megatron modules.

None of those packages is installed where these tests run (the reference's own adapter tests mock
them as well), so what is pinned here is this package's side of the contract: when the callback
saves, how the checkpoint IO routes by path, that an ML Flashpoint save goes through the Megatron
strategies and loads back, queue separation of the async wrapper, the auto-resume lookup and the
trainer wrapping rules.
"""

import concurrent.futures
import json
import os
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as torch_mp

import cases
import megatron_standins
from helpers import NumpyCopyEngine, make_loader, make_saver, tensor_bytes


@pytest.fixture
def nemo(monkeypatch, tmp_path):
    megatron_standins.install()
    megatron_standins.install_nemo()
    monkeypatch.setenv("MLFLASHPOINT_DISABLE_DIST", "true")
    monkeypatch.setenv("NNODES", "1")
    monkeypatch.setattr(torch.distributed, "get_node_local_rank", lambda *a, **k: 0)
    monkeypatch.setattr(torch.distributed, "get_rank", lambda *a, **k: 0)
    monkeypatch.setattr(torch.distributed, "broadcast_object_list", lambda box, src=0: None)
    import importlib
    import sys

    for name in [m for m in sys.modules if m.startswith("ml_flashpoint.adapter.nemo")]:
        del sys.modules[name]  # bind to this test's stand-in classes
    mods = {n: importlib.import_module(f"ml_flashpoint.adapter.nemo.{n}") for n in
            ("checkpoint_callback", "checkpoint_io", "auto_resume", "nemo_checkpoint_loader", "wrapper_util", "event_logging_callback")}
    return mods


def _io_stack(nemo, tmp_path, always_save_context=False):
    from ml_flashpoint.adapter.megatron.load_strategies import MLFlashpointMegatronLoadStrategy
    from ml_flashpoint.adapter.megatron.save_strategies import MLFlashpointMegatronAsyncSaveStrategy
    from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter
    import sys

    engine = NumpyCopyEngine()

    class _Replication:
        def async_replicate(self, buffer_io):
            buffer_io.close()
            return []

        def shutdown(self):
            self.down = True

    replication = _Replication()
    saver, com = make_saver(copy_engine=engine, replication_manager=replication)
    manager = torch_mp.Manager()
    fut = concurrent.futures.Future()
    fut.set_result(manager)
    save = MLFlashpointMegatronAsyncSaveStrategy(MemoryStorageWriter(saver, fut))
    load = MLFlashpointMegatronLoadStrategy(replication, make_loader(com, copy_engine=engine))
    fallback = sys.modules["nemo.lightning.io.pl"].MegatronCheckpointIO()
    base = str(tmp_path / "mlf")
    trainer = sys.modules["nemo.lightning.pytorch.trainer"].Trainer(sys.modules["nemo.lightning.pytorch.strategies"].MegatronStrategy(fallback))
    io = nemo["checkpoint_io"].MLFlashpointCheckpointIO(base, fallback, com, save, load, trainer, async_save=True, always_save_context=always_save_context)
    return io, fallback, base, manager, replication, com, trainer


def test_callback_saves_on_schedule(nemo, tmp_path):
    cb_mod = nemo["checkpoint_callback"]
    with pytest.raises(ValueError):
        cb_mod.MLFlashpointCheckpointCallback(str(tmp_path), every_n_steps=0)
    with pytest.raises(ValueError):
        cb_mod.MLFlashpointCheckpointCallback(str(tmp_path), every_n_steps=5, skip_every_n_steps=-1)
    import sys

    trainer = sys.modules["nemo.lightning.pytorch.trainer"].Trainer(strategy=None)
    cb = cb_mod.MLFlashpointCheckpointCallback(str(tmp_path / "base"), every_n_steps=5, skip_every_n_steps=20)
    for step in range(1, 41):
        trainer.global_step = step
        cb.on_train_batch_end(trainer, None, None, None, step)
    assert [Path(p).name for p, _ in trainer.saved] == [f"step-{s}_ckpt" for s in (5, 10, 15, 25, 30, 35)]
    opts = trainer.saved[0][1][cb_mod.ML_FLASHPOINT_OPTS_KEY]
    assert opts["ckpt_type"] is cb_mod.ML_FLASHPOINT_TYPE and opts["step"] == 5
    off = cb_mod.MLFlashpointCheckpointCallback(str(tmp_path / "base"), every_n_steps=1, enabled=False)
    off.on_train_batch_end(trainer, None, None, None, 1)
    assert len(trainer.saved) == 6


def test_checkpoint_io_routes_saves_and_loads(nemo, tmp_path):
    io, fallback, base, manager, _, _, _ = _io_stack(nemo, tmp_path)
    try:
        elsewhere = str(tmp_path / "longterm" / "step-5")
        io.save_checkpoint({"w": torch.ones(2)}, elsewhere)
        assert io.load_checkpoint(elsewhere) == {"from": "fallback"}
        io.remove_checkpoint(elsewhere)
        assert [c[0] for c in fallback.calls] == ["save", "load", "remove"]
        assert io.load_content_metadata(elsewhere) == {"from": "fallback"}

        tensors = dict(cases.CASES["two_buckets"]()["tensors"])
        checkpoint = dict(tensors)
        checkpoint["iteration"] = 30
        ckpt = os.path.join(base, "step-30_ckpt")
        request = io.save_checkpoint(checkpoint, ckpt, storage_options={"content_metadata": {"mcore": "0.13"}})
        assert request is not None and len(fallback.calls) == 3
        request.execute_sync()
        assert os.path.exists(os.path.join(ckpt, ".metadata")) and os.path.exists(os.path.join(ckpt, "common.pt"))
        assert io.load_content_metadata(ckpt) == {"mcore": "0.13"}
        assert io.load_content_metadata(ckpt, preloaded_state_dict={"content_metadata": 1}) == 1
        fresh = {k: torch.zeros_like(v) for k, v in tensors.items()}
        loaded = io.load_checkpoint(ckpt, sharded_state_dict=fresh)
        assert loaded["iteration"] == 30
        for k, v in tensors.items():
            assert tensor_bytes(loaded[k]) == tensor_bytes(v)
        io.remove_checkpoint(ckpt)
        assert not os.path.exists(ckpt)
        with pytest.raises(Exception):
            io.load_checkpoint(ckpt, sharded_state_dict=fresh)  # errors surface to the trainer
    finally:
        manager.shutdown()


def test_context_is_saved_when_requested(nemo, tmp_path):
    io, _, base, manager, _, _, _ = _io_stack(nemo, tmp_path, always_save_context=True)
    try:
        ckpt = os.path.join(base, "step-1_ckpt")
        io.save_checkpoint({"w": torch.ones(3)}, ckpt).execute_sync()
        assert os.path.exists(os.path.join(ckpt, "context", "model.yaml"))
    finally:
        manager.shutdown()


def test_async_wrapper_keeps_separate_queues(nemo, tmp_path):
    io, fallback, base, manager, _, _, _ = _io_stack(nemo, tmp_path)
    try:
        with pytest.raises(ValueError):
            nemo["checkpoint_io"].MLFlashpointAsyncFinalizableCheckpointIO(fallback)
        wrapped = nemo["checkpoint_io"].MLFlashpointAsyncFinalizableCheckpointIO(io)
        assert wrapped.maybe_finalize_save_checkpoint() is False
        extra = []
        wrapped.save_checkpoint({"w": torch.ones(2)}, os.path.join(base, "step-2_ckpt"), {"finalize_fn": lambda: extra.append("mlf")})
        wrapped.save_checkpoint({"w": torch.ones(2)}, str(tmp_path / "longterm" / "s2"), {"finalize_fn": lambda: extra.append("alt")})
        assert wrapped._mlf_async_calls_queue.get_num_unfinalized_calls() == 1
        assert wrapped._alt_async_calls_queue.get_num_unfinalized_calls() == 1
        assert wrapped._mlf_async_calls_queue.persistent and not wrapped._alt_async_calls_queue.persistent
        assert wrapped.maybe_finalize_save_checkpoint(blocking=True) is True
        assert extra == ["mlf", "alt"] and os.path.exists(os.path.join(base, "step-2_ckpt", ".metadata"))
        wrapped.teardown()
        assert wrapped._mlf_async_calls_queue.closed
    finally:
        manager.shutdown()


def test_callback_train_end_drains_and_cleans_up(nemo, tmp_path):
    io, _, base, manager, replication, _, trainer = _io_stack(nemo, tmp_path)
    try:
        wrapped = nemo["checkpoint_io"].MLFlashpointAsyncFinalizableCheckpointIO(io)
        trainer.strategy.checkpoint_io = wrapped
        cb = nemo["checkpoint_callback"].MLFlashpointCheckpointCallback(base, every_n_steps=1)
        cb.replication_manager = replication
        wrapped.save_checkpoint({"w": torch.ones(2)}, os.path.join(base, "step-1_ckpt"))
        wrapped.remove_checkpoint = io.remove_checkpoint
        cb.on_train_end(trainer, None)
        assert trainer.strategy.barriers == ["mlf_cleanup_barrier"] and replication.down
        assert not os.path.exists(base)  # removed unless keep_mlf_checkpoint_on_train_end
    finally:
        manager.shutdown()


def test_auto_resume_prefers_flashpoint_then_falls_back(nemo, tmp_path):
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId

    found = CheckpointContainerId(str(tmp_path / "mlf" / "step-8_ckpt"))
    os.makedirs(found.data)

    class _Loader:
        calls = 0

        def __init__(self, answer):
            self.answer = answer

        def get_latest_complete_checkpoint(self, base):
            _Loader.calls += 1
            return self.answer

    resume = nemo["auto_resume"].MLFlashpointAutoResume(
        checkpoint_base_container=CheckpointContainerId(str(tmp_path / "mlf")), checkpoint_loader=_Loader(found), resume_if_exists=True
    )
    assert resume.get_trainer_ckpt_path() == Path(found.data)
    assert json.load(open(os.path.join(found.data, "metadata.json"))) == {"sharded_backend": ""}
    assert resume.get_trainer_ckpt_path() == Path(found.data) and _Loader.calls == 1  # cached, the search is collective
    none = nemo["auto_resume"].MLFlashpointAutoResume(
        checkpoint_base_container=CheckpointContainerId(str(tmp_path / "mlf")), checkpoint_loader=_Loader(None), fallback_path=Path("/long/term")
    )
    assert none.get_trainer_ckpt_path() == Path("/long/term")


def test_nemo_loader_adds_context_files_to_the_retrieval_plan(nemo, tmp_path):
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId

    ckpt = CheckpointContainerId(str(tmp_path / "step-1_ckpt"))
    os.makedirs(os.path.join(ckpt.data, "context", "sub"))
    for rel in ("context/model.yaml", "context/sub/io.json"):
        open(os.path.join(ckpt.data, rel), "w").close()

    def loader(recover):
        return nemo["nemo_checkpoint_loader"].NeMoMLFlashpointCheckpointLoader(
            CheckpointObjectManager(), None, global_rank_getter=lambda: 0, local_rank_getter=lambda: 0,
            broadcast_object_list_func=None, all_gather_object_func=None, world_size_getter=lambda: 1,
            recover_context=recover, copy_engine=NumpyCopyEngine(),
        )

    assert loader(False)._get_extra_local_objects(Path(ckpt.data)) == []
    extra = loader(True)._get_extra_local_objects(Path(ckpt.data))
    assert sorted(Path(str(o)).name for o in extra) == ["io.json", "model.yaml"]
    listing = {0: extra + [CheckpointObjectId.from_container(ckpt, "__0__0_src0.distcp")]}
    assert loader(True)._get_extra_needed_objects(ckpt, listing) == {str(o) for o in extra}
    assert loader(False)._get_extra_needed_objects(ckpt, listing) == set()


def test_wrapping_a_trainer(nemo, tmp_path, monkeypatch):
    import sys

    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.replication.replication_manager import ReplicationManager

    wu = nemo["wrapper_util"]
    monkeypatch.setattr(ReplicationManager, "initialize", lambda self, **kw: None)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    for fn in ("get_world_size", "all_gather_object", "barrier"):
        monkeypatch.setattr(torch.distributed, fn, lambda *a, **k: 1)
    pl_mod = sys.modules["nemo.lightning.io.pl"]
    strategies = sys.modules["nemo.lightning.pytorch.strategies"]
    trainer_cls = sys.modules["nemo.lightning.pytorch.trainer"].Trainer
    async_wrap = sys.modules["nemo.utils.callbacks.dist_ckpt_io"].AsyncFinalizableCheckpointIO
    base = str(tmp_path / "mlf")
    cb = nemo["checkpoint_callback"].MLFlashpointCheckpointCallback(base, every_n_steps=2)

    plain = trainer_cls(strategies.MegatronStrategy(pl_mod.MegatronCheckpointIO()), callbacks=[])
    wu.wrap_trainer_checkpoint_io_with_mlflashpoint(plain, base, CheckpointObjectManager(), ReplicationManager(), True, object())
    assert isinstance(plain.strategy.checkpoint_io, pl_mod.MegatronCheckpointIO)  # no callback: left alone

    trainer = trainer_cls(strategies.MegatronStrategy(async_wrap(pl_mod.MegatronCheckpointIO())), callbacks=[cb])
    resume = wu.wrap_trainer_and_auto_resume_with_mlflashpoint(
        trainer, base, async_save=True, default_auto_resume=sys.modules["nemo.lightning"].AutoResume(resume_if_exists=True),
        initial_write_buffer_size_bytes=1 << 20,
    )
    io = trainer.strategy.checkpoint_io
    assert isinstance(io, nemo["checkpoint_io"].MLFlashpointAsyncFinalizableCheckpointIO)
    assert isinstance(io.checkpoint_io.fallback_checkpoint_io, pl_mod.MegatronCheckpointIO)
    assert type(io.checkpoint_io.save_strategy).__name__ == "FullyParallelSaveStrategyWrapper"
    assert cb.replication_manager is not None and resume.resume_if_exists is True
    assert str(resume.checkpoint_base_container) == base
    before = trainer.strategy.checkpoint_io
    wu.wrap_trainer_checkpoint_io_with_mlflashpoint(trainer, base, CheckpointObjectManager(), ReplicationManager(), True, object())
    assert trainer.strategy.checkpoint_io is before  # idempotent
    with pytest.raises(ValueError, match="async_save is False"):
        wu.wrap_trainer_checkpoint_io_with_mlflashpoint(trainer, base, CheckpointObjectManager(), ReplicationManager(), False, object())
    with pytest.raises(ValueError, match="MegatronStrategy"):
        wu.wrap_trainer_checkpoint_io_with_mlflashpoint(trainer_cls(object(), callbacks=[cb]), base, CheckpointObjectManager(), ReplicationManager(), True, object())
    for bad in (dict(write_thread_count=0), dict(initial_write_buffer_size_bytes=0)):
        with pytest.raises(ValueError):
            wu.wrap_trainer_checkpoint_io_with_mlflashpoint(trainer, base, CheckpointObjectManager(), ReplicationManager(), True, object(), **bad)
    CheckpointObjectManager._worker_pool = None


def test_event_logging_callback_logs_every_hook(nemo, caplog):
    import logging

    cb = nemo["event_logging_callback"].EventLoggingCallback()
    seen = []
    cb._log_event = seen.append
    cb.on_train_start(None, None)
    cb.on_train_batch_end(None, None, None, None, 0)
    cb.on_before_optimizer_step(None, None, None)
    assert seen == ["on_train_start", "on_train_batch_end", "on_before_optimizer_step"]
