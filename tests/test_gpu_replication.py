"""Object replication over the GPU transport: copy kernel into the peer's HBM, peer drains to a file.

Two ``TransferService`` instances talk over 127.0.0.1, as the reference's own point-to-point tests
do with its TCP service. Inside one process the peers exchange raw device pointers; across processes
(``test_replication_between_processes``) the landing buffer travels as a CUDA IPC handle. Failures
are injected on the host only (dead address, missing object, shutdown with work pending)."""

import ast
import hashlib
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

import cases
import conftest
from helpers import case_to_device, make_loader, make_saver
from helpers import tensor_bytes as oracle_bytes

pytestmark = pytest.mark.gpu
GOLDEN = conftest.GOLDEN_DIR


def _save_object(root, engine, name="views"):
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId

    case = case_to_device(cases.CASES[name](), "cuda")
    saver, com = make_saver(copy_engine=engine)
    ckpt = CheckpointContainerId(str(root / "step-1_ckpt"))
    saver.initialize_checkpoint(ckpt)
    items, resolver = cases.write_items_and_resolver(case)
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=1)
    saver.write_data(ckpt, buckets, replicate_after_write=False)
    return com, buckets[0].object_id


@pytest.fixture
def services(shm_path):
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    replica_root = str(shm_path / "replicas")

    def mapper(object_id, source_rank):
        return os.path.join(replica_root, f"src{source_rank}", object_id.lstrip("/"))

    a, b = TransferService(), TransferService(replica_path_mapper=mapper)
    assert a.initialize(0, threads=4, global_rank=0) > 0
    assert b.initialize(0, threads=4, global_rank=1) > 0
    yield a, b, mapper
    a.shutdown()
    b.shutdown()


@pytest.mark.parametrize("resident", [True, False])
def test_put_then_get_round_trip(shm_path, services, resident):
    from ml_flashpoint.core import gpu_engine

    a, b, mapper = services
    engine = gpu_engine.default_engine()
    com, oid = _save_object(shm_path, engine)
    primary = open(str(oid), "rb").read()
    if not resident:
        engine.drop_resident_images()  # as after a later save reused the HBM image: source is the host mapping
    else:
        assert gpu_engine.resident_image(str(oid), len(primary) - 4096) is not None
    buf = com.get_buffer(oid)
    result = a.async_put(buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity(), b.address, str(oid)).result(timeout=60)
    assert result.success and result.task_id
    replica_path = mapper(str(oid), 0)
    assert open(replica_path, "rb").read() == primary
    assert not os.path.exists(replica_path + ".tmp")
    # recovery direction: rank 0 lost the object and asks rank 1, which serves its replica
    back = str(shm_path / "restored" / "obj.distcp")
    os.makedirs(os.path.dirname(back))
    got = a.async_get(str(oid), b.address, back).result(timeout=60)
    assert got.success and open(back, "rb").read() == primary
    buf.close()


def test_replica_lands_in_a_page_locked_pool_file(shm_path):
    """With a landing pool the receiver drains by one copy-engine transfer into a pool file; the
    replica is a symlink to it and frees the pool buffer when it is deleted."""
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.core.buffer_pool import BufferPool
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    pool = BufferPool(str(shm_path / "replica_pool"), rank=1, num_buffers=1, buffer_size=1 << 20, register_cuda=True)
    replica = str(shm_path / "replicas" / "obj.distcp")
    a, b = TransferService(), TransferService(replica_path_mapper=lambda obj, src: replica, landing_pool=pool)
    a.initialize(0, threads=2, global_rank=0)
    b.initialize(0, threads=2, global_rank=1)
    try:
        com, oid = _save_object(shm_path, gpu_engine.default_engine(), name="mixed")
        primary = open(str(oid), "rb").read()
        for _ in range(2):  # the second round reuses the pool buffer freed by deleting the replica
            buf = com.get_buffer(oid)
            assert a.async_put(buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity(), b.address, str(oid)).result(timeout=60).success
            buf.close()
            assert os.path.islink(replica) and os.path.dirname(os.path.realpath(replica)) == os.path.realpath(pool.pool_dir)
            assert open(replica, "rb").read() == primary
            os.remove(replica)
    finally:
        a.shutdown()
        b.shutdown()
        pool.teardown()


def test_failures_surface_on_the_future(shm_path, services):
    a, b, _ = services
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        dead = f"127.0.0.1:{s.getsockname()[1]}"
    src = torch.zeros(8192, dtype=torch.uint8).numpy()
    with pytest.raises(RuntimeError, match="cannot reach"):
        a.async_put(src.ctypes.data, src.nbytes, dead, "/x/y").result(timeout=60)
    with pytest.raises(RuntimeError, match="not held here"):
        a.async_get("/no/such/object", b.address, str(shm_path / "nothing")).result(timeout=60)
    with pytest.raises(RuntimeError):
        a.async_put(0, 0, b.address, "/x/y").result(timeout=60)
    a.shutdown()
    with pytest.raises(RuntimeError, match="not running"):
        a.async_put(src.ctypes.data, src.nbytes, b.address, "/x/y").result(timeout=5)


def test_manager_ring_replication_end_to_end(shm_path, services, monkeypatch):
    """ReplicationManager + RingReplicationStrategy over the real service, as the saver drives it."""
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.replication import replication_manager as rm

    a, b, mapper = services
    monkeypatch.setattr(rm.dist, "get_rank", lambda: 0)
    com, oid = _save_object(shm_path, gpu_engine.default_engine(), name="mixed")
    mgr = rm.ReplicationManager()
    mgr.initialize(com, replication_transfer_service=a, repl_strategy=rm.RingReplicationStrategy([a.address, b.address]))
    futures = mgr.async_replicate(com.get_buffer(oid))
    assert len(futures) == 1 and futures[0].result(timeout=60).success
    assert open(mapper(str(oid), 0), "rb").read() == open(str(oid), "rb").read()


def _peer_process(role, root, port_file, digest_file):
    import sys
    import time

    here = os.path.dirname(os.path.abspath(__file__))
    repo = os.path.dirname(here)
    for p in (here, os.path.join(here, "golden"), os.path.join(repo, "oracle"), os.path.join(repo, "ml-flashpoint_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MLFLASHPOINT_LOG_LEVEL"] = "ERROR"
    import pathlib

    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    torch.cuda.set_device((0 if role == "receiver" else 1) % torch.cuda.device_count())
    if role == "receiver":
        svc = TransferService(replica_path_mapper=lambda obj, src: os.path.join(root, "replica.distcp"))
        port = svc.initialize(0, threads=2, global_rank=1)
        with open(port_file + ".tmp", "w") as f:
            f.write(str(port))
        os.rename(port_file + ".tmp", port_file)
        deadline = time.time() + 120
        while not os.path.exists(digest_file) and time.time() < deadline:
            time.sleep(0.05)
        svc.shutdown()
        return
    deadline = time.time() + 120
    while not os.path.exists(port_file) and time.time() < deadline:
        time.sleep(0.05)
    port = int(open(port_file).read())
    svc = TransferService()
    svc.initialize(0, threads=2, global_rank=0)
    com, oid = _save_object(pathlib.Path(root), gpu_engine.default_engine(), name="gpt2_tiny")
    buf = com.get_buffer(oid)
    ok = svc.async_put(buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity(), f"127.0.0.1:{port}", str(oid)).result(timeout=120).success
    digest = hashlib.sha256(open(str(oid), "rb").read()).hexdigest()
    with open(digest_file + ".tmp", "w") as f:
        f.write(repr({"ok": ok, "sha": digest}))
    os.rename(digest_file + ".tmp", digest_file)
    svc.shutdown()


def test_replication_between_processes(shm_path):
    """Sender and receiver are separate processes (on two GPUs when present, else sharing one):
    the landing buffer crosses as a CUDA IPC handle and is written by the sender's copy kernel."""
    ctx = mp.get_context("spawn")
    port_file, digest_file = str(shm_path / "port"), str(shm_path / "digest")
    procs = [ctx.Process(target=_peer_process, args=(role, str(shm_path), port_file, digest_file)) for role in ("receiver", "sender")]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    outcome = ast.literal_eval(open(digest_file).read())
    assert outcome["ok"]
    assert hashlib.sha256(open(str(shm_path / "replica.distcp"), "rb").read()).hexdigest() == outcome["sha"]


def _pooled_saver(root, engine, rank, manager=None, buffer_bytes=8 << 20):
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig

    pool = BufferPoolConfig(str(root / f"buffer_pool_{rank}"), rank, 2, buffer_bytes, register_cuda=True)
    return make_saver(copy_engine=engine, rank=rank, pool_config=pool, replication_manager=manager)


@pytest.mark.parametrize("overlapped", [False, True])
def test_replication_starts_with_the_pack_kernel_when_the_object_is_pooled(shm_path, services, monkeypatch, overlapped):
    """``replicate_after_write=True`` on a pool buffer: the push is queued with the pack kernel and
    sends the HBM image while the copy engine still drains it; the replica equals the primary and
    the golden object, and the device-timed path starts at the save's own start event."""
    from helpers import golden_object_bytes, load_golden
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.replication import replication_manager as rm

    a, b, mapper = services
    monkeypatch.setattr(rm.dist, "get_rank", lambda: 0)
    engine = gpu_engine.default_engine()
    mgr = rm.ReplicationManager()
    saver, com = _pooled_saver(shm_path, engine, 0)
    mgr.initialize(com, replication_transfer_service=a, repl_strategy=rm.RingReplicationStrategy([a.address, b.address]))
    saver._replication_manager = mgr
    try:
        case = case_to_device(cases.CASES["mixed"](), "cuda")
        ckpt = CheckpointContainerId(str(shm_path / "step-3_ckpt"))
        saver.initialize_checkpoint(ckpt)
        items, resolver = cases.write_items_and_resolver(case)
        buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=1)
        started = []
        real = mgr.async_replicate
        monkeypatch.setattr(mgr, "async_replicate", lambda buf: started.append(real(buf)) or started[-1])
        if overlapped:
            pending = saver.write_data_async(ckpt, buckets, replicate_after_write=True)
            assert len(started) == 1  # queued before result() is called
            pending.result()
            futures = pending.replication_futures
        else:
            saver.write_data(ckpt, buckets, replicate_after_write=True)
            futures = started[0]
        assert len(started) == 1 and len(futures) == 1 and futures[0].result(timeout=60).success
        gold = load_golden(GOLDEN, "mixed.json")["objects"][0]
        primary = open(str(buckets[0].object_id), "rb").read()
        assert primary == golden_object_bytes(GOLDEN, gold)
        assert open(mapper(str(buckets[0].object_id), 0), "rb").read() == primary
        stats = a.last_put_stats
        assert stats["from_hbm_image"] and stats["since_save_start_ms"] is not None and stats["since_save_start_ms"] > 0
    finally:
        com.teardown_pool()  # the pool is process-wide: later tests must not inherit this one


def test_put_falls_back_to_the_host_copy_when_the_image_is_gone(shm_path, services):
    """A later save or a restore may take the arena between the look-up of the resident image and its
    lease: the put then sends the object from its host mapping instead of failing."""
    from ml_flashpoint.core import gpu_engine

    a, b, mapper = services
    engine = gpu_engine.default_engine()
    com, oid = _save_object(shm_path, engine)
    primary = open(str(oid), "rb").read()
    real = gpu_engine.resident_image

    def lease_then_lose(object_id, nbytes):
        lease = real(object_id, nbytes)
        engine.staging(1 << 20)  # what a restore does: every resident image is given up
        return lease

    gpu_engine.resident_image = lease_then_lose
    try:
        buf = com.get_buffer(oid)
        assert a.async_put(buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity(), b.address, str(oid)).result(timeout=60).success
        buf.close()
    finally:
        gpu_engine.resident_image = real
    assert a.last_put_stats["from_hbm_image"] is False
    assert open(mapper(str(oid), 0), "rb").read() == primary


class _TwoRankCollectives:
    """all_gather / broadcast for two loaders that run as threads of one process."""

    def __init__(self):
        import threading

        self._barrier = threading.Barrier(2)
        self._slots = [None, None]
        self._box = None

    def all_gather(self, rank):
        def gather(out, obj):
            self._slots[rank] = obj
            self._barrier.wait(timeout=120)
            out[:] = list(self._slots)
            self._barrier.wait(timeout=120)

        return gather

    def broadcast(self, rank):
        def bcast(box, src=0):
            if rank == src:
                self._box = list(box)
            self._barrier.wait(timeout=120)
            box[:] = self._box
            self._barrier.wait(timeout=120)

        return bcast


def test_recovery_of_a_lost_object_through_the_cuda_transport(shm_path, golden_dir, monkeypatch):
    """Save on rank 0, replicate to rank 1, lose the primary (a host-side fault: the file is deleted),
    then recover the way a restarted job does: ``get_latest_complete_checkpoint`` on both ranks
    (discovery, retrieval plan, ``retrieve_checkpoint`` -> ``sync_bulk_retrieve`` -> get over the
    GPU transport) and ``read_data`` into the unpack kernel, checked against the reference-generated
    narrow reads. A second loss after discovery goes through ``_try_retrieve_object_if_missing``."""
    import pickle
    import threading

    from helpers import load_golden
    from torch.distributed.checkpoint.metadata import Metadata, MetadataIndex
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.replication import replication_manager as rm
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import ReplicaNamespace, TransferService

    monkeypatch.setenv("NNODES", "1")
    engine = gpu_engine.default_engine()
    spaces = [ReplicaNamespace(str(shm_path / f"replicas_of_rank{r}")) for r in range(2)]
    services = [TransferService(replica_path_mapper=spaces[r]) for r in range(2)]
    for r, s in enumerate(services):
        assert s.initialize(0, threads=4, global_rank=r) > 0
    addresses = [s.address for s in services]
    managers = []
    for r in range(2):
        m = rm.ReplicationManager()
        m.initialize(CheckpointObjectManager(), replication_transfer_service=services[r], repl_strategy=rm.RingReplicationStrategy(addresses))
        managers.append(m)
    try:
        # ---- rank 0 saves (the narrow-read sources) and replicates to rank 1
        monkeypatch.setattr(rm.dist, "get_rank", lambda: 0)
        tensors = {f"n.{i}": cases.narrow_source(i).cuda() for i in range(len(cases.NARROW_CASES))}
        saver, com = make_saver(copy_engine=engine, replication_manager=managers[0])
        base = shm_path / "job"
        ckpt = CheckpointContainerId(str(base / "step-7_ckpt"))
        saver.initialize_checkpoint(ckpt)
        items, resolver = cases.write_items_and_resolver({"tensors": tensors, "blobs": {}, "bucket_count": 1})
        buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=1)
        results = saver.write_data(ckpt, buckets, replicate_after_write=False)
        for f in saver.async_replicate_object(buckets[0].object_id):
            assert f.result(timeout=60).success
        storage = {r.index: r.storage_data for r in results}
        saver.write_metadata(ckpt, Metadata(state_dict_metadata={}, storage_data=storage))
        open(os.path.join(ckpt.data, "common.pt"), "wb").close()
        saver.finalize_checkpoint(ckpt)
        oid = buckets[0].object_id
        primary = open(str(oid), "rb").read()
        os.remove(str(oid))  # the fault

        # ---- both ranks look for the latest complete checkpoint
        net = _TwoRankCollectives()
        loaders = [
            make_loader(CheckpointObjectManager(), copy_engine=engine, rank=r, world=2, replication_manager=managers[r])
            for r in range(2)
        ]
        found = [None, None]
        for r, loader in enumerate(loaders):
            loader._replica_namespace = spaces[r]
            loader._all_gather_object_func = net.all_gather(r)
            loader._broadcast_object_list_func = net.broadcast(r)

        def discover(r):
            found[r] = loaders[r].get_latest_complete_checkpoint(CheckpointContainerId(str(base)))

        threads = [threading.Thread(target=discover, args=(r,)) for r in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=180)
        assert [str(f) for f in found] == [str(ckpt), str(ckpt)]
        assert open(str(oid), "rb").read() == primary  # came back over the GPU transport

        # ---- lost again after discovery: read_data fetches it on its own, then unpacks
        os.remove(str(oid))
        rows = load_golden(golden_dir, "narrow.json")
        for row in rows:
            shape, dtype, offs, lens = cases.NARROW_CASES[row["i"]]
            idx = MetadataIndex(f"n.{row['i']}", torch.Size([0] * len(shape)))
            target = torch.zeros(lens, dtype=dtype, device="cuda")
            req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * len(lens)), idx, torch.Size(offs), torch.Size(lens))

            class _Planner:
                def resolve_tensor(self, r):
                    return target

                def commit_tensor(self, r, t):
                    pass

            loaders[0].read_data(oid, [req], _Planner(), {idx: storage[idx]})
            assert oracle_bytes(target).hex() == row["hex"], row["i"]
        assert open(str(oid), "rb").read() == primary
    finally:
        for s in services:
            s.shutdown()


def test_two_devices_in_one_process_pack_replicate_and_restore(shm_path):
    """A process that drives two GPUs: an engine on device 1 packs and unpacks after device 0 has
    (per-device kernel attributes), and an object saved on device 0 is pushed into device 1's HBM
    over NVLink by the copy kernel and drained there."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import ReplicaNamespace, TransferService

    engines = [CudaCopyEngine(device=torch.device("cuda", d)) for d in range(2)]
    objects = []
    for d, engine in enumerate(engines):
        with torch.cuda.device(d):
            case = case_to_device(cases.CASES["views"](), f"cuda:{d}")
            saver, com = make_saver(copy_engine=engine, rank=d)
            from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId

            ckpt = CheckpointContainerId(str(shm_path / f"dev{d}" / "step-1_ckpt"))
            saver.initialize_checkpoint(ckpt)
            items, resolver = cases.write_items_and_resolver(case)
            buckets = saver.prepare_write_data(ckpt, items, resolver, f"__{d}_", bucket_count=1)
            results = saver.write_data(ckpt, buckets, replicate_after_write=False)
            objects.append((com, buckets[0].object_id, results, case))
            # restore on the same device, strided targets
            loader = make_loader(com, copy_engine=engine, rank=d)
            from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

            targets = {}
            reqs = []
            for r in results:
                t = case["tensors"][r.index.fqn]
                if t.numel() == 0:
                    continue
                targets[r.index.fqn] = torch.zeros(t.shape, dtype=t.dtype, device=f"cuda:{d}")
                reqs.append(ReadItem(LoadItemType.TENSOR, r.index, torch.Size([0] * t.dim()), r.index, torch.Size([0] * t.dim()), torch.Size(t.shape)))

            class _Planner:
                def resolve_tensor(self, req):
                    return targets[req.dest_index.fqn]

                def commit_tensor(self, req, tensor):
                    pass

            loader.read_data(buckets[0].object_id, reqs, _Planner(), {r.index: r.storage_data for r in results})
            for fqn, target in targets.items():
                assert oracle_bytes(target) == oracle_bytes(case["tensors"][fqn]), (d, fqn)
    first, second = (open(str(o[1]), "rb").read() for o in objects)
    assert first[4096:] == second[4096:]  # same case, same bytes, whichever device packed them

    # ---- device 0 -> device 1 over NVLink
    space = ReplicaNamespace(str(shm_path / "replicas"))
    services = []
    for d in range(2):
        with torch.cuda.device(d):
            s = TransferService(replica_path_mapper=space)
            assert s.initialize(0, threads=2, global_rank=d) > 0
            services.append(s)
    try:
        gpu_engine.set_default_engine(engines[0])
        com, oid, _, case0 = objects[0]
        # the restore above gave the arena to its own image; save once more so that the push below
        # finds the object's image resident in device 0's HBM
        with torch.cuda.device(0):
            saver0, com = make_saver(copy_engine=engines[0], rank=0)
            ckpt0 = CheckpointContainerId(os.path.dirname(str(oid)))
            items0, resolver0 = cases.write_items_and_resolver(case0)
            again = saver0.prepare_write_data(ckpt0, items0, resolver0, "__0_", bucket_count=1)
            saver0.write_data(ckpt0, again, replicate_after_write=False)
            assert str(again[0].object_id) == str(oid) and open(str(oid), "rb").read() == first
        buf = com.get_buffer(oid)
        assert services[0].async_put(buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity(), services[1].address, str(oid)).result(timeout=60).success
        buf.close()
        assert services[0].last_put_stats["from_hbm_image"]
        assert open(space(str(oid), 0), "rb").read() == first
        assert space.held_objects(os.path.dirname(str(oid))) == [str(oid)]
    finally:
        gpu_engine.set_default_engine(None)
        for s in services:
            s.shutdown()


@pytest.mark.parametrize("resident", [True, False])
@pytest.mark.parametrize("pooled_landing", [False, True])
def test_replication_through_a_two_slot_landing_ring(shm_path, resident, pooled_landing):
    """With ``landing_chunk_bytes`` the receiver holds two small slots instead of a buffer the size of
    the object: the sender's copy kernel fills one while the other drains to the file. Same replica
    bytes whether the source is the save's HBM image or the host mapping, into a plain file or a
    page-locked pool file, and the get direction (recovery) works through the same ring."""
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.core.buffer_pool import BufferPool
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import ReplicaNamespace, TransferService

    chunk = 64 << 10
    space = ReplicaNamespace(str(shm_path / "replicas"))
    pool = BufferPool(str(shm_path / "replica_pool"), rank=1, num_buffers=1, buffer_size=1 << 20, register_cuda=True) if pooled_landing else None
    a = TransferService(landing_chunk_bytes=chunk)
    b = TransferService(replica_path_mapper=space, landing_pool=pool, landing_chunk_bytes=chunk)
    assert a.initialize(0, threads=4, global_rank=0) > 0 and b.initialize(0, threads=4, global_rank=1) > 0
    try:
        engine = gpu_engine.default_engine()
        com, oid = _save_object(shm_path, engine, name="gpt2_tiny")  # 839 KB: thirteen chunks
        primary = open(str(oid), "rb").read()
        if not resident:
            engine.drop_resident_images()
        buf = com.get_buffer(oid)
        assert a.async_put(buf.buffer_obj.get_data_ptr(), buf.buffer_obj.get_capacity(), b.address, str(oid)).result(timeout=60).success
        buf.close()
        stats = a.last_put_stats
        assert stats["chunks"] == -(-len(primary) // chunk) and stats["from_hbm_image"] is resident
        assert open(space(str(oid), 0), "rb").read() == primary
        assert not os.path.exists(space(str(oid), 0) + ".tmp")
        assert b.held_device_bytes() == 2 * chunk  # not the object's 839 KB
        back = str(shm_path / "restored" / "obj.distcp")
        os.makedirs(os.path.dirname(back))
        assert a.async_get(str(oid), b.address, back).result(timeout=60).success
        assert open(back, "rb").read() == primary
    finally:
        a.shutdown()
        b.shutdown()
        if pool is not None:
            pool.teardown()
