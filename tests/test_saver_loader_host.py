"""Saver / loader host logic with the numpy stand-in engine: naming, bucketing, cursors, results,
markers, metadata, legacy format. Object bytes are still checked against the reference's golden
files, which pins the layout planner (``plan_object_layout``) independently of the CUDA path."""

import hashlib
import io
import os
import pickle
import time

import pytest
import torch
from torch.distributed.checkpoint.metadata import Metadata, MetadataIndex
from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

import cases
import mlf_oracle as oracle
from helpers import NumpyCopyEngine, golden_object_bytes, load_golden, make_loader, make_saver, tensor_bytes
from ml_flashpoint.core import gpu_engine
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId


def _save(case, root, **kw):
    saver, com = make_saver(copy_engine=NumpyCopyEngine(), **kw)
    ckpt = CheckpointContainerId(str(root / "step-5_ckpt"))
    saver.initialize_checkpoint(ckpt)
    items, resolver = cases.write_items_and_resolver(case)
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=case["bucket_count"])
    results = saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=case["bucket_count"])
    return saver, com, ckpt, buckets, results


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_layout_planner_reproduces_reference_objects(name, tmp_path, golden_dir):
    gold = load_golden(golden_dir, f"{name}.json")
    _, _, ckpt, buckets, results = _save(cases.CASES[name](), tmp_path)
    assert [b.object_name for b in buckets] == [o["name"] for o in gold["objects"]]
    for bucket, g in zip(buckets, gold["objects"]):
        data = open(str(bucket.object_id), "rb").read()
        assert len(data) == g["size"] and hashlib.sha256(data).hexdigest() == g["sha256"]
        if "file" in g:
            assert data == golden_object_bytes(golden_dir, g)
    got = sorted((r.storage_data.relative_path, r.storage_data.offset, r.storage_data.length, r.index.fqn) for r in results)
    assert got == [(w["relative_path"], w["offset"], w["length"], w["index"]["fqn"]) for w in gold["write_results"]]
    assert all(r.size_in_bytes == r.storage_data.length for r in results)


def test_layout_records_chunks_and_placements():
    a = torch.arange(6, dtype=torch.int16).reshape(2, 3)
    empty = torch.zeros(0, dtype=torch.float32)
    layout = gpu_engine.plan_object_layout([("a", a), ("e", empty)], [("b", io.BytesIO(b"xyz")), ("n", b"")], start_offset=7)
    ha = len(oracle.header_bytes("int16", (2, 3)))
    he = len(oracle.header_bytes("float32", (0,)))
    assert [(r.item, r.offset, r.length) for r in layout.records] == [
        ("a", 7, ha + 12),
        ("e", 7 + ha + 12, he),
        ("b", 7 + ha + 12 + he, 3),
        ("n", 7 + ha + 12 + he + 3, 0),
    ]
    assert layout.total_bytes == ha + 12 + he + 3 and layout.payload_bytes == 12
    assert [(p.payload_offset, tuple(p.tensor.shape)) for p in layout.tensors] == [(7 + ha, (2, 3))]
    assert [c.offset for c in layout.host_chunks] == [7, 7 + ha + 12, 7 + ha + 12 + he]
    assert layout.host_chunks[0].data == oracle.header_bytes("int16", (2, 3))
    assert gpu_engine.c_strides((4, 1, 3, 0, 5)) == [15, 15, 5, 5, 1]  # a zero extent counts as one
    assert gpu_engine.c_strides((2, 3, 4)) == [12, 4, 1] and gpu_engine.c_strides(()) == []


def test_dirty_marker_metadata_and_finalize(tmp_path):
    saver, com, ckpt, buckets, results = _save(cases.CASES["mixed"](), tmp_path)
    marker = str(tmp_path / "step-5_ckpt__0__unfinished")
    assert os.path.exists(marker)
    md = Metadata(state_dict_metadata={}, storage_data={r.index: r.storage_data for r in results})
    saver.write_metadata(ckpt, md)
    assert not os.path.exists(os.path.join(ckpt.data, ".metadata.tmp"))
    assert pickle.load(open(os.path.join(ckpt.data, ".metadata"), "rb")).storage_data == md.storage_data
    os.makedirs(tmp_path / "step-3_ckpt")
    os.makedirs(tmp_path / "step-9_ckpt")
    os.makedirs(tmp_path / "unrelated")
    barrier_calls = []
    saver._barrier_func = lambda: barrier_calls.append(1)
    proc = saver.finalize_checkpoint(ckpt)
    assert barrier_calls == [1] and not os.path.exists(marker)
    proc.wait(timeout=30)
    assert sorted(os.listdir(tmp_path)) == ["step-5_ckpt", "step-9_ckpt", "unrelated"]
    assert saver.finalize_checkpoint(ckpt) is None  # nothing older left; missing marker only warns
    saver._local_rank_getter = lambda: 1
    assert saver.finalize_checkpoint(ckpt) is None  # only local rank 0 deletes


def test_writer_errors_surface_and_saver_pickles_without_engine(tmp_path):
    class _Boom:
        def pack_async(self, *a, **k):
            raise OSError("disk on fire")

    saver, _ = make_saver(copy_engine=_Boom())
    ckpt = CheckpointContainerId(str(tmp_path / "step-1_ckpt"))
    items, resolver = cases.write_items_and_resolver(cases.CASES["two_buckets"]())
    buckets = saver.prepare_write_data(ckpt, items, resolver, "p", bucket_count=2)
    with pytest.raises(OSError, match="disk on fire"):
        saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=2)
    state = saver.__getstate__()  # what crosses into a writer process
    assert "_replication_manager" not in state and state["_copy_engine"] is None
    clone = object.__new__(type(saver))
    clone.__setstate__(state)
    assert clone._replication_manager is None and clone._copy_engine is None
    with pytest.raises(RuntimeError, match="ReplicationManager is not available"):
        clone.async_replicate_object(buckets[0].object_id)
    # standalone buffers cannot grow: a bucket larger than the initial size is an error, as upstream
    small, _ = make_saver(copy_engine=NumpyCopyEngine(), initial_buffer_size_bytes=64)
    with pytest.raises(ValueError, match="exceeds buffer capacity"):
        small.write_data(ckpt, buckets[:1], replicate_after_write=False)


def _read_all(loader, buckets, results, case, device="cpu"):
    storage = {r.index: r.storage_data for r in results}
    by_fqn = {r.index.fqn: r.index for r in results}
    targets, blobs, committed = {}, {}, []

    class _Planner:
        def resolve_tensor(self, req):
            return targets[req.dest_index.fqn]

        def commit_tensor(self, req, tensor):
            committed.append(req.dest_index.fqn)

        def load_bytes(self, req, value):
            blobs[req.dest_index.fqn] = value.read()

    per_object = {}
    for fqn, t in case["tensors"].items():
        idx = by_fqn[fqn]
        targets[fqn] = torch.zeros(t.shape, dtype=t.dtype, device=device)
        req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * t.dim()), idx, torch.Size([0] * t.dim()), torch.Size(t.shape))
        per_object.setdefault(storage[idx].relative_path, []).append(req)
    for fqn in case["blobs"]:
        idx = by_fqn[fqn]
        per_object.setdefault(storage[idx].relative_path, []).append(ReadItem(LoadItemType.BYTE_IO, idx, None, idx, None, None))
    for b in buckets:
        loader.read_data(b.object_id, per_object.get(b.object_name, []), _Planner(), storage)
    return targets, blobs, committed


@pytest.mark.parametrize("name", ["mixed", "views", "two_buckets"])
def test_loader_round_trip_including_zero_element_tensors(name, tmp_path):
    case = cases.CASES[name]()
    _, com, ckpt, buckets, results = _save(case, tmp_path)
    loader = make_loader(com, copy_engine=NumpyCopyEngine())
    targets, blobs, committed = _read_all(loader, buckets, results, case)
    for fqn, t in case["tensors"].items():
        assert tensor_bytes(targets[fqn]) == tensor_bytes(t), fqn
    assert blobs == dict(case["blobs"])
    assert sorted(committed) == sorted(case["tensors"])


def test_loader_narrow_reads_match_reference(tmp_path, golden_dir):
    rows = load_golden(golden_dir, "narrow.json")
    tensors = {f"n.{i}": cases.narrow_source(i) for i in range(len(cases.NARROW_CASES))}
    _, com, ckpt, buckets, results = _save({"tensors": tensors, "blobs": {}, "bucket_count": 1}, tmp_path)
    loader = make_loader(com, copy_engine=NumpyCopyEngine())
    storage = {r.index: r.storage_data for r in results}
    for row in rows:
        shape, dtype, offs, lens = cases.NARROW_CASES[row["i"]]
        idx = MetadataIndex(f"n.{row['i']}", torch.Size([0] * len(shape)))
        target = torch.zeros(lens, dtype=dtype)
        req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * len(lens)), idx, torch.Size(offs), torch.Size(lens))

        class _Planner:
            def resolve_tensor(self, r):
                return target

            def commit_tensor(self, r, t):
                pass

        loader.read_data(buckets[0].object_id, [req], _Planner(), {idx: storage[idx]})
        assert tensor_bytes(target).hex() == row["hex"]
    # a block that leaves the stored extent is refused before any byte moves
    idx = MetadataIndex("n.0", torch.Size([0, 0]))
    bad = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0, 0]), idx, torch.Size([10, 0]), torch.Size([16, 24]))

    class _P2:
        def resolve_tensor(self, r):
            return torch.zeros(16, 24)

        def commit_tensor(self, r, t):
            pass

    with pytest.raises(IndexError):
        loader.read_data(buckets[0].object_id, [bad], _P2(), {idx: storage[idx]})


def test_missing_object_and_metadata_errors(tmp_path):
    _, com = make_saver(copy_engine=NumpyCopyEngine())
    loader = make_loader(com, copy_engine=NumpyCopyEngine())
    with pytest.raises(FileNotFoundError, match="does not exist on any node"):
        loader.read_data(CheckpointObjectId(str(tmp_path / "step-1_ckpt" / "x.distcp")), [], None, {})
    with pytest.raises(FileNotFoundError):
        loader.read_metadata(CheckpointContainerId(str(tmp_path / "step-1_ckpt")))


def test_legacy_torch_save_format_round_trip(tmp_path):
    case = cases.CASES["two_buckets"]()
    case["bucket_count"] = 1
    _, com, ckpt, buckets, results = _save(case, tmp_path, use_optimized_save=False)
    raw = open(str(buckets[0].object_id), "rb").read()
    assert raw[8:16] == b"TORCH___"
    loader = make_loader(com, copy_engine=NumpyCopyEngine())
    targets, blobs, _ = _read_all(loader, buckets, results, case)
    for fqn, t in case["tensors"].items():
        assert torch.equal(targets[fqn], t)
    assert blobs == dict(case["blobs"])


def test_overlapped_save_api_publishes_the_same_objects(tmp_path, golden_dir):
    """``write_data_async`` + ``PendingSave.result`` must leave exactly what ``write_data`` leaves."""
    gold = load_golden(golden_dir, "two_buckets.json")
    case = cases.CASES["two_buckets"]()
    saver, com = make_saver(copy_engine=NumpyCopyEngine())
    ckpt = CheckpointContainerId(str(tmp_path / "step-5_ckpt"))
    saver.initialize_checkpoint(ckpt)
    items, resolver = cases.write_items_and_resolver(case)
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=2)
    pending = saver.write_data_async(ckpt, buckets)
    pending.wait_safe_to_mutate()
    assert pending.done() and pending.safe_to_mutate_event is not None
    results = pending.result()
    assert pending.result() is results  # idempotent
    for bucket, g in zip(buckets, gold["objects"]):
        assert open(str(bucket.object_id), "rb").read() == golden_object_bytes(golden_dir, g)
    got = sorted((r.storage_data.relative_path, r.storage_data.offset, r.storage_data.length) for r in results)
    assert got == [(w["relative_path"], w["offset"], w["length"]) for w in gold["write_results"]]


def test_load_converts_to_the_target_dtype(tmp_path):
    """The reference ends a read in ``target.copy_(tensor)``, which converts dtypes (fp32 checkpoint
    into bf16 parameters): the loader unpacks in the stored dtype and converts afterwards."""
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    src = torch.randn(6, 10)
    _, com, ckpt, buckets, results = _save({"tensors": {"w": src}, "blobs": {}, "bucket_count": 1}, tmp_path)
    loader = make_loader(com, copy_engine=NumpyCopyEngine())
    idx = results[0].index
    target = torch.zeros(2, 10, dtype=torch.bfloat16)
    req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0, 0]), idx, torch.Size([1, 0]), torch.Size([2, 10]))

    class _P:
        def resolve_tensor(self, r):
            return target

        def commit_tensor(self, r, t):
            pass

    loader.read_data(buckets[0].object_id, [req], _P(), {idx: results[0].storage_data})
    assert torch.equal(target, src[1:3].to(torch.bfloat16))


def test_replication_follows_the_write_unless_the_process_wide_cuda_engine_moves_the_bytes(tmp_path, golden_dir):
    """Replication may only start together with the pack kernel when the transfer service can find
    the save in the process-wide CUDA engine. With any other engine (here the numpy double), pool
    buffer or not, ``async_replicate`` is called once per object, after the object is complete."""
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig

    gold = load_golden(golden_dir, "mixed.json")["objects"][0]
    seen = []

    class _Repl:
        def async_replicate(self, buffer_io):
            seen.append(bytes(memoryview(buffer_io.buffer_obj)))
            buffer_io.close()
            return []

    case = cases.CASES["mixed"]()
    for pooled in (False, True):
        seen.clear()
        pool = BufferPoolConfig(str(tmp_path / f"pool{pooled}"), 0, 2, 1 << 20) if pooled else None
        saver, com = make_saver(copy_engine=NumpyCopyEngine(), pool_config=pool, replication_manager=_Repl())
        try:
            ckpt = CheckpointContainerId(str(tmp_path / f"run{pooled}" / "step-1_ckpt"))
            saver.initialize_checkpoint(ckpt)
            items, resolver = cases.write_items_and_resolver(case)
            buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=1)
            assert saver._can_replicate_early(com.acquire_buffer(CheckpointObjectId(str(tmp_path / f"probe{pooled}.distcp")), 1 << 16)) is False
            saver.write_data(ckpt, buckets, replicate_after_write=True)
            assert seen == [golden_object_bytes(golden_dir, gold)]
            seen.clear()
            ckpt2 = CheckpointContainerId(str(tmp_path / f"run{pooled}" / "step-2_ckpt"))
            saver.initialize_checkpoint(ckpt2)
            buckets = saver.prepare_write_data(ckpt2, items, resolver, "__0_", bucket_count=1)
            pending = saver.write_data_async(ckpt2, buckets, replicate_after_write=True)
            assert seen == []  # nothing before result()
            pending.result()
            assert seen == [golden_object_bytes(golden_dir, gold)] and pending.replication_futures == []
        finally:
            com.teardown_pool()
