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
from helpers import case_to_device, make_saver

pytestmark = pytest.mark.gpu


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
