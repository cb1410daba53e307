"""Replication strategies, manager bookkeeping and recovery discovery, all on the host.

Failures are injected on the host only: a transfer future that carries an exception, a missing
object, a dirty marker, a rank that reports nothing."""

import concurrent.futures
import os
import pickle

import pytest
from torch.distributed.checkpoint.filesystem import _StorageInfo
from torch.distributed.checkpoint.metadata import Metadata, MetadataIndex

from helpers import NumpyCopyEngine, make_loader, make_saver
from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.replication import replication_manager as rm
from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferResult


def test_ring_strategy():
    addrs = [f"h:{p}" for p in range(4)]
    ring = rm.RingReplicationStrategy(addrs)
    assert [ring.get_destination_addresses(r) for r in range(4)] == [["h:1"], ["h:2"], ["h:3"], ["h:0"]]
    assert rm.RingReplicationStrategy(addrs, offset=4).get_destination_addresses(0) == []
    assert rm.RingReplicationStrategy(["only"]).get_destination_addresses(0) == []
    with pytest.raises(ValueError):
        ring.get_destination_addresses(4)
    with pytest.raises(ValueError):
        rm.RingReplicationStrategy([])
    assert ring.get_replication_service_addresses() == addrs


def test_pairwise_strategy(monkeypatch):
    addrs = [f"h:{p}" for p in range(8)]
    monkeypatch.setenv("NNODES", "4")
    pair = rm.PairwiseReplicationStrategy(addrs, processes_per_node=2)
    assert [pair.get_destination_addresses(r)[0] for r in range(8)] == ["h:2", "h:3", "h:0", "h:1", "h:6", "h:7", "h:4", "h:5"]
    with pytest.raises(ValueError):
        pair.get_destination_addresses(8)
    monkeypatch.setenv("NNODES", "1")
    assert rm.PairwiseReplicationStrategy(addrs, processes_per_node=8).get_destination_addresses(3) == []
    monkeypatch.setenv("NNODES", "3")
    with pytest.raises(ValueError, match="even"):
        rm.PairwiseReplicationStrategy(addrs[:6], processes_per_node=2)
    monkeypatch.setenv("NNODES", "2")
    with pytest.raises(ValueError, match="divisible"):
        rm.PairwiseReplicationStrategy(addrs[:7], processes_per_node=2)
    with pytest.raises(ValueError):
        rm.PairwiseReplicationStrategy([], processes_per_node=2)


class _FakeTransfer:
    def __init__(self, fail=False):
        self.puts, self.gets, self.fail = [], [], fail

    def _done(self):
        f = concurrent.futures.Future()
        if self.fail:
            f.set_exception(RuntimeError("peer unreachable"))
        else:
            f.set_result(TransferResult("t", True, ""))
        return f

    def async_put(self, ptr, size, address, obj):
        self.puts.append((ptr, size, address, obj))
        return self._done()

    def async_get(self, remote, address, local):
        self.gets.append((remote, address, local))
        return self._done()

    def shutdown(self):
        self.down = True


def _manager(tmp_path, monkeypatch, transfer, strategy):
    monkeypatch.setattr(rm.dist, "get_rank", lambda: 0)
    mgr = rm.ReplicationManager()
    mgr.initialize(CheckpointObjectManager(), replication_transfer_service=transfer, repl_strategy=strategy)
    return mgr


def _object(tmp_path):
    com = CheckpointObjectManager()
    oid = CheckpointObjectId(str(tmp_path / "step-1_ckpt" / "o_src0.distcp"))
    with com.acquire_buffer(oid, 64) as w:
        w.write(b"payload")
    return com, oid


@pytest.mark.parametrize("fail", [False, True])
def test_async_replicate_puts_whole_object_and_closes_buffer(tmp_path, monkeypatch, fail):
    transfer = _FakeTransfer(fail)
    mgr = _manager(tmp_path, monkeypatch, transfer, rm.RingReplicationStrategy(["a:1", "b:2"]))
    com, oid = _object(tmp_path)
    buf = com.get_buffer(oid)
    ptr, cap = buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity()
    futures = mgr.async_replicate(buf)
    assert transfer.puts == [(ptr, cap, "b:2", str(oid))]
    assert len(futures) == 1 and buf.closed  # closed by the aggregate callback, also after a failure
    assert isinstance(futures[0].exception(), RuntimeError) == fail
    mgr.shutdown()
    assert transfer.down


def test_async_replicate_without_destination_closes_at_once(tmp_path, monkeypatch):
    transfer = _FakeTransfer()
    mgr = _manager(tmp_path, monkeypatch, transfer, rm.RingReplicationStrategy(["solo:1"]))
    com, oid = _object(tmp_path)
    buf = com.get_buffer(oid)
    assert mgr.async_replicate(buf) == [] and buf.closed and transfer.puts == []


def test_sync_bulk_retrieve(tmp_path, monkeypatch):
    ok = _manager(tmp_path, monkeypatch, _FakeTransfer(), rm.RingReplicationStrategy(["a:1", "b:2"]))
    objs = [CheckpointObjectId("/c/step-1_ckpt/x"), CheckpointObjectId("/c/step-1_ckpt/y")]
    assert ok.sync_bulk_retrieve(1, objs, []) is True
    assert ok._transfer_service.gets == [("/c/step-1_ckpt/x", "b:2", "/c/step-1_ckpt/x"), ("/c/step-1_ckpt/y", "b:2", "/c/step-1_ckpt/y")]
    assert ok.sync_bulk_retrieve(5, objs, []) is False  # unknown rank
    assert ok.sync_bulk_retrieve(1, objs, [], retrieved_object_ids=objs[:1]) is False  # length mismatch
    bad = _manager(tmp_path, monkeypatch, _FakeTransfer(fail=True), rm.RingReplicationStrategy(["a:1", "b:2"]))
    assert bad.sync_bulk_retrieve(1, objs, []) is False
    assert rm.ReplicationManager().sync_bulk_retrieve(0, objs, []) is False  # never initialised


def test_aggregate_callback_fires_once():
    calls = []
    futs = [concurrent.futures.Future() for _ in range(3)]
    rm.ReplicationManager._add_aggregate_callback(futs, lambda fs: calls.append(len(fs)))
    for f in futs[:2]:
        f.set_result(1)
    assert calls == []
    futs[2].set_exception(RuntimeError("x"))
    assert calls == [3]
    rm.ReplicationManager._add_aggregate_callback([], lambda fs: calls.append("empty"))
    assert calls[-1] == "empty"


# ------------------------------------------------------------------ recovery discovery
class _Cluster:
    """Per-rank loaders whose collectives are answered from the other ranks' local views."""

    def __init__(self, roots, monkeypatch, nodes):
        monkeypatch.setenv("NNODES", str(nodes))
        self.roots = roots
        self.world = len(roots)

    def loader(self, rank, retrieved):
        cluster = self

        class _Repl:
            def sync_bulk_retrieve(self, source_global_rank, object_ids_to_retrieve, container_ids_to_retrieve):
                for obj in object_ids_to_retrieve:
                    retrieved.append((rank, source_global_rank, str(obj)))
                return True

        return make_loader(CheckpointObjectManager(), copy_engine=NumpyCopyEngine(), rank=rank, world=self.world, replication_manager=_Repl())


def _touch(path, data=b"x"):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "wb") as f:
        f.write(data)


def test_candidates_skip_dirty_and_non_common_checkpoints(tmp_path):
    base = tmp_path / "ckpts"
    for step in (1, 2, 3):
        os.makedirs(base / f"step-{step}_ckpt")
    _touch(str(base / "step-3_ckpt__0__unfinished"))
    os.makedirs(base / "other")
    loader = make_loader(CheckpointObjectManager(), copy_engine=NumpyCopyEngine(), world=2)
    mine = [str(base / "step-1_ckpt"), str(base / "step-2_ckpt")]
    loader._all_gather_object_func = lambda out, obj: out.__setitem__(slice(None), [obj, [str(base / "step-1_ckpt")]])
    got = loader.get_candidate_checkpoints(CheckpointContainerId(str(base)))
    assert [str(c) for c in got] == [str(base / "step-1_ckpt")]
    loader._all_gather_object_func = lambda out, obj: out.__setitem__(slice(None), [obj, None])  # a rank with nothing to say
    got = loader.get_candidate_checkpoints(CheckpointContainerId(str(base)))
    assert [str(c) for c in got] == [str(base / "step-2_ckpt"), str(base / "step-1_ckpt")]
    assert sorted(mine) == sorted(str(c) for c in got)
    loader._all_gather_object_func = lambda out, obj: out.__setitem__(slice(None), [[], []])
    assert loader.get_candidate_checkpoints(CheckpointContainerId(str(tmp_path / "none"))) == []


def test_retrieval_plan(tmp_path, monkeypatch):
    monkeypatch.setenv("NNODES", "2")
    ckpt = CheckpointContainerId(str(tmp_path / "step-7_ckpt"))
    os.makedirs(ckpt.data)
    storage = {
        MetadataIndex("a"): _StorageInfo("__0__0_src0.distcp", 0, 10),
        MetadataIndex("b"): _StorageInfo("__1__0_src1.distcp", 0, 10),
        MetadataIndex("c"): _StorageInfo("__2__0_src2.distcp", 0, 10),
        MetadataIndex("d"): _StorageInfo("__3__0_src3.distcp", 0, 10),
    }
    with open(os.path.join(ckpt.data, ".metadata"), "wb") as f:
        pickle.dump(Metadata(state_dict_metadata={}, storage_data=storage), f)
    loader = make_loader(CheckpointObjectManager(), copy_engine=NumpyCopyEngine(), world=4)

    def obj(name):
        return CheckpointObjectId.from_container(ckpt, name)

    full = {
        0: [obj("__0__0_src0.distcp"), obj(".metadata"), obj("common.pt")],
        1: [obj("__1__0_src1.distcp")],
        2: [obj("__2__0_src2.distcp"), obj(".metadata"), obj("common.pt")],
        3: [obj("__3__0_src3.distcp")],
    }
    assert loader._compute_retrieval_plan(ckpt, full) == {}
    # node 1 (ranks 2, 3) was replaced: it holds nothing, its objects survive as replicas on node 0
    lost = {0: full[0] + [obj("__2__0_src2.distcp")], 1: full[1] + [obj("__3__0_src3.distcp")], 2: [], 3: []}
    plan = loader._compute_retrieval_plan(ckpt, lost)
    assert sorted(plan) == [2, 3]
    assert sorted(plan[2]) == sorted([(0, str(obj("__2__0_src2.distcp"))), (0, str(obj(".metadata"))), (0, str(obj("common.pt")))])
    assert plan[3] == [(1, str(obj("__3__0_src3.distcp")))]
    # an object nobody holds makes the checkpoint unusable
    gone = {0: full[0], 1: full[1], 2: [], 3: []}
    assert loader._compute_retrieval_plan(ckpt, gone) is None
    # unreadable metadata likewise
    os.remove(os.path.join(ckpt.data, ".metadata"))
    assert loader._compute_retrieval_plan(ckpt, full) is None


def test_latest_complete_checkpoint_walks_back_to_a_recoverable_step(tmp_path, monkeypatch):
    monkeypatch.setenv("NNODES", "1")
    base = tmp_path / "job"
    new, old = base / "step-20_ckpt", base / "step-10_ckpt"
    for ckpt, complete in ((new, False), (old, True)):
        storage = {MetadataIndex("a"): _StorageInfo("__0__0_src0.distcp", 0, 4)}
        _touch(str(ckpt / ".metadata"), pickle.dumps(Metadata(state_dict_metadata={}, storage_data=storage)))
        _touch(str(ckpt / "common.pt"))
        if complete:
            _touch(str(ckpt / "__0__0_src0.distcp"))
    loader = make_loader(CheckpointObjectManager(), copy_engine=NumpyCopyEngine(), world=1)
    loader._broadcast_object_list_func = lambda box, src=0: None
    found = loader.get_latest_complete_checkpoint(CheckpointContainerId(str(base)))
    assert str(found) == str(old)  # step 20 lacks its only object everywhere
    _touch(str(base / "step-10_ckpt__0__unfinished"))
    assert loader.get_latest_complete_checkpoint(CheckpointContainerId(str(base))) is None


def test_missing_object_is_fetched_from_the_rank_that_holds_it(tmp_path):
    fetched = []

    class _Repl:
        def sync_bulk_retrieve(self, source_global_rank, object_ids_to_retrieve, container_ids_to_retrieve):
            fetched.append((source_global_rank, [str(o) for o in object_ids_to_retrieve]))
            _touch(str(object_ids_to_retrieve[0]))
            return True

    loader = make_loader(CheckpointObjectManager(), copy_engine=NumpyCopyEngine(), replication_manager=_Repl())
    ckpt = CheckpointContainerId(str(tmp_path / "step-1_ckpt"))
    oid = CheckpointObjectId.from_container(ckpt, "o_src0.distcp")
    os.makedirs(ckpt.data)
    assert loader._try_retrieve_object_if_missing(oid) is False  # nobody is known to hold it
    loader._available_objects_cache[ckpt] = {str(oid): [3, 1]}
    assert loader._try_retrieve_object_if_missing(oid) is True
    assert fetched == [(3, [str(oid)])]
    assert loader._try_retrieve_object_if_missing(oid) is True and len(fetched) == 1  # present now


def test_replica_namespace_maps_and_lists_back(tmp_path):
    """Replicas of ranks that share a filesystem live under ``<root>/src<sender>/<object path>``; the
    reverse listing reports them under their original paths (what a loader advertises in recovery)."""
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import ReplicaNamespace

    space = ReplicaNamespace(str(tmp_path / "replicas"))
    container = "/job/ckpt/step-5_ckpt"
    assert space.held_objects(container) == []  # nothing received yet, the root does not even exist
    a = space(f"{container}/__0__0_src0.distcp", 0)
    b = space(f"{container}/__3__0_src3.distcp", 3)
    assert a == str(tmp_path / "replicas" / "src0" / "job/ckpt/step-5_ckpt/__0__0_src0.distcp")
    for path in (a, b, b + ".tmp", space("/job/ckpt/step-4_ckpt/__0__0_src0.distcp", 0)):
        _touch(path)
    assert sorted(space.held_objects(container)) == [f"{container}/__0__0_src0.distcp", f"{container}/__3__0_src3.distcp"]

    loader = make_loader(CheckpointObjectManager(), copy_engine=NumpyCopyEngine(), rank=1, world=2)
    loader._replica_namespace = space
    import pathlib

    extra = loader._get_extra_local_objects(pathlib.Path(container))
    assert sorted(str(o) for o in extra) == sorted(space.held_objects(container))
