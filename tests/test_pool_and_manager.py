"""BufferPool / PooledBufferIO / CheckpointObjectManager host logic (no GPU needed)."""

import os

import pytest

from ml_flashpoint.checkpoint_object_manager.buffer_io import BufferIO
from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE
from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core.buffer_pool import BufferPool, BufferPoolConfig, PooledBufferIO
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId


@pytest.fixture(autouse=True)
def _fresh_pool_registry():
    CheckpointObjectManager._worker_pool = None
    yield
    pool, CheckpointObjectManager._worker_pool = CheckpointObjectManager._worker_pool, None
    if pool:
        pool.teardown()


def test_config_validation():
    with pytest.raises(ValueError):
        BufferPoolConfig("", 0, 1, 1)
    with pytest.raises(ValueError):
        BufferPoolConfig("/x", -1, 1, 1)
    with pytest.raises(ValueError):
        BufferPoolConfig("/x", 0, 1, -5)
    with pytest.raises(ValueError):
        BufferPool("/x", num_buffers=0, buffer_size=10)
    with pytest.raises(ValueError):
        BufferPool("/x", num_buffers=1, buffer_size=0)


def test_pool_preallocates_links_collects_and_exhausts(tmp_path):
    pool = BufferPool(str(tmp_path / "pool"), rank=3, num_buffers=2, buffer_size=METADATA_SIZE + 64)
    assert sorted(os.listdir(tmp_path / "pool")) == ["buffer_3_0.dist", "buffer_3_1.dist"]
    a = pool.acquire(str(tmp_path / "objA"))
    assert isinstance(a, PooledBufferIO) and os.path.islink(tmp_path / "objA")
    assert os.path.realpath(tmp_path / "objA") == os.path.realpath(a.buffer_obj.get_id())
    b = pool.acquire(str(tmp_path / "objB"))
    with pytest.raises(RuntimeError, match="exhausted"):
        pool.acquire(str(tmp_path / "objC"))
    a.write(b"first")
    a.close()
    assert a.closed and not a._buffer_io.closed  # the pooled file stays open
    os.remove(tmp_path / "objA")  # checkpoint deleted -> buffer becomes reusable
    c = pool.acquire(str(tmp_path / "objC"))
    assert c.tell() == 0 and c._buffer_io._metadata.len_written_data == 0
    assert c.buffer_obj.get_id() == a.buffer_obj.get_id()
    # a failed link leaves the buffer in the free list
    os.remove(tmp_path / "objB")
    with pytest.raises(OSError):
        pool.acquire(str(tmp_path / "no" / "such" / "dir" / "obj"))
    assert len(pool.free_buffers) == 1
    pool.teardown()
    assert not pool.free_buffers and not pool.active_buffers
    del b


def test_pooled_buffer_grows_on_demand_and_trims_on_close(tmp_path):
    pool = BufferPool(str(tmp_path / "pool"), rank=0, num_buffers=1, buffer_size=METADATA_SIZE + 16)
    w = pool.acquire(str(tmp_path / "obj"))
    w.write(b"x" * 10)
    w.write(b"y" * 100)  # beyond capacity: grows by max(10 %, need + 1 MiB)
    assert w.buffer_obj.get_capacity() >= METADATA_SIZE + 110 + 1024 * 1024
    piece = w.next_buffer_slice(3 * 1024 * 1024)
    assert len(piece) == 3 * 1024 * 1024
    total = 110 + 3 * 1024 * 1024
    w.close()
    assert os.path.getsize(tmp_path / "obj") == METADATA_SIZE + total
    with open(tmp_path / "obj", "rb") as f:
        f.seek(METADATA_SIZE)
        assert f.read(12) == b"x" * 10 + b"yy"
    # exact sizing in one step
    os.remove(tmp_path / "obj")
    w2 = pool.acquire(str(tmp_path / "obj2"))
    w2.ensure_total_size(METADATA_SIZE + 500)
    assert w2.buffer_obj.get_capacity() == METADATA_SIZE + 500
    w2.next_buffer_slice(500)
    w2.close()
    assert os.path.getsize(tmp_path / "obj2") == METADATA_SIZE + 500


def test_manager_prefers_pool_then_falls_back_to_standalone_files(tmp_path):
    cfg = BufferPoolConfig(str(tmp_path / "pool"), rank=0, num_buffers=1, buffer_size=METADATA_SIZE + 32)
    com = CheckpointObjectManager(cfg)
    ckpt = CheckpointContainerId(str(tmp_path / "step-1_ckpt"))
    one = CheckpointObjectId.from_container(ckpt, "a.distcp")
    two = CheckpointObjectId.from_container(ckpt, "b.distcp")
    with pytest.raises(ValueError):
        com.acquire_buffer(one, 0)
    w1 = com.acquire_buffer(one, 1000)
    assert isinstance(w1, PooledBufferIO) and os.path.islink(str(one))
    w2 = com.acquire_buffer(two, 1000)  # pool exhausted -> plain file of the requested size + metadata
    assert isinstance(w2, BufferIO) and not os.path.islink(str(two))
    assert os.path.getsize(str(two)) == 1000 + METADATA_SIZE
    w1.write(b"pooled")
    w2.write(b"alone")
    w1.close()
    w2.close()
    r = com.get_buffer(one)
    assert r.is_readonly and r.read() == b"pooled"
    com.close_buffer(r, skip_close_if_symlink=True)
    assert not r.closed  # objects that are symlinks into the pool are left open on request
    com.close_buffer(r)
    assert r.closed
    com.close_buffer(r)  # closing twice is ignored
    assert com.get_buffer(CheckpointObjectId.from_container(ckpt, "missing")) is None
    assert com.get_buffer(CheckpointObjectId(str(tmp_path / "step-1_ckpt"))) is None  # a directory
    # overwrite semantics
    with pytest.raises(FileExistsError):
        com.acquire_buffer(two, 10, overwrite=False)
    com.delete_object(two)
    com.delete_object(two)  # missing: warning only
    com.delete_container(ckpt)
    assert not os.path.exists(str(ckpt))
    com.delete_container(ckpt)  # missing: warning only
    com.teardown_pool()
    assert CheckpointObjectManager._worker_pool is None


def test_manager_without_pool_creates_standalone_files(tmp_path):
    com = CheckpointObjectManager()
    obj = CheckpointObjectId(str(tmp_path / "c" / "o.distcp"))
    with com.acquire_buffer(obj, 64) as w:
        w.write(b"abc")
    assert os.path.getsize(str(obj)) == METADATA_SIZE + 3
