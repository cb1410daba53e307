"""Generates the golden vectors under tests/golden/ by running the reference implementation.

Run where a checkout of the reference project is available and pass its root:

    python tests/golden/generate_golden.py /path/to/ml-flashpoint

The reference's two compiled extension modules cannot be built offline, so two small
stand-ins are registered in ``sys.modules`` before the reference package is imported: a
file-backed ``BufferObject`` over ``mmap`` and an inert ``TransferService``. Everything that
produces bytes (bucketing, header pickling, cursor arithmetic, ``copy_`` into the mapping,
metadata block, truncation, the loader's slicing) is the reference's own Python code.

Outputs (all deterministic for a fixed torch version):
  <case>.json          object names/sizes/sha256 and the WriteResults of ``write_data``
  <case>__<obj>.bin    the object file bytes, for objects up to 128 KiB
  headers.json         pickled TensorHeader bytes for a dtype x shape matrix
  narrow.json          bytes the reference loader delivers for sub-block reads
"""

from __future__ import annotations

import hashlib
import json
import mmap
import os
import shutil
import sys
import tempfile
import types

HERE = os.path.dirname(os.path.abspath(__file__))
MAX_INLINE_OBJECT = 128 * 1024


class _FileBufferObject:
    """Stand-in for the reference's compiled ``BufferObject`` (same constructor forms and methods)."""

    def __init__(self, object_id, capacity=None, overwrite=False):
        self._id = object_id
        if capacity is None:
            self._fd = os.open(object_id, os.O_RDONLY)
            size = os.fstat(self._fd).st_size
            if size == 0:
                os.close(self._fd)
                raise RuntimeError("zero-sized file")
            self._map = mmap.mmap(self._fd, size, prot=mmap.PROT_READ)
            self._readonly = True
        else:
            if capacity <= 0:
                raise RuntimeError("capacity must be positive")
            os.makedirs(os.path.dirname(object_id), exist_ok=True)
            mode = os.O_TRUNC if overwrite else os.O_EXCL
            self._fd = os.open(object_id, os.O_CREAT | os.O_RDWR | mode, 0o666)
            os.ftruncate(self._fd, capacity)
            self._map = mmap.mmap(self._fd, capacity)
            self._readonly = False
        self._closed = False

    def __buffer__(self, flags):
        view = memoryview(self._map)
        return view.toreadonly() if self._readonly else view

    closed = property(lambda self: self._closed)
    is_readonly = property(lambda self: self._readonly)

    def get_id(self):
        return self._id

    def get_capacity(self):
        return 0 if self._closed else len(self._map)

    def get_data_ptr(self):
        return 0

    def resize(self, new_capacity):
        os.ftruncate(self._fd, new_capacity)
        self._map = mmap.mmap(self._fd, new_capacity)

    def close(self, truncate_size=None):
        if self._closed:
            return
        if truncate_size is not None and not self._readonly:
            os.ftruncate(self._fd, truncate_size)
        os.close(self._fd)  # exported views keep the old mapping alive; the file is already final
        self._closed = True


def _install_reference(ref_root: str) -> None:
    buf = types.ModuleType("ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext")
    buf.BufferObject = _FileBufferObject
    sys.modules[buf.__name__] = buf
    xfer = types.ModuleType("ml_flashpoint.replication.transfer_service.transfer_service_ext")
    xfer.TransferService = type("TransferService", (), {})
    xfer.TransferResult = type("TransferResult", (), {})
    sys.modules[xfer.__name__] = xfer
    sys.path.insert(0, os.path.join(ref_root, "src"))
    os.environ.setdefault("MLFLASHPOINT_LOG_LEVEL", "ERROR")


def _index_to_json(index) -> dict:
    return {
        "fqn": index.fqn,
        "offset": None if index.offset is None else list(index.offset),
        "index": index.index,
    }


def _save_case(name: str, case: dict, workdir: str) -> dict:
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver

    sys.path.insert(0, HERE)
    import cases

    saver = DefaultMLFlashpointCheckpointSaver(
        global_rank_getter=lambda: 0,
        local_rank_getter=lambda: 0,
        global_barrier_func=lambda: None,
        ckpt_obj_manager=CheckpointObjectManager(),
        replication_manager=None,
        initial_buffer_size_bytes=8 * 1024 * 1024,
    )
    ckpt = CheckpointContainerId(os.path.join(workdir, name, "step-1_ckpt"))
    saver.initialize_checkpoint(ckpt)
    items, resolver = cases.write_items_and_resolver(case)
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=case["bucket_count"])
    results = saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=1)

    objects = []
    for bucket in buckets:
        with open(str(bucket.object_id), "rb") as f:
            data = f.read()
        entry = {
            "name": bucket.object_name,
            "size": len(data),
            "sha256": hashlib.sha256(data).hexdigest(),
            "item_order": [_index_to_json(wi.index) for wi, _ in bucket.tensor_data]
            + [_index_to_json(wi.index) for wi, _ in bucket.bytesio_data],
        }
        if len(data) <= MAX_INLINE_OBJECT:
            entry["file"] = f"{name}__{bucket.object_name}.bin"
            with open(os.path.join(HERE, entry["file"]), "wb") as f:
                f.write(data)
        else:
            # enough of the head to debug a mismatch without storing megabytes
            entry["head_hex"] = data[: 4096 + 512].hex()
        objects.append(entry)

    write_results = [
        {
            "index": _index_to_json(r.index),
            "size_in_bytes": r.size_in_bytes,
            "relative_path": r.storage_data.relative_path,
            "offset": r.storage_data.offset,
            "length": r.storage_data.length,
        }
        for r in results
    ]
    write_results.sort(key=lambda r: (r["relative_path"], r["offset"]))
    return {"case": name, "bucket_count": case["bucket_count"], "objects": objects, "write_results": write_results}


def _headers() -> list:
    import torch
    from ml_flashpoint.core.tensor_header import TensorHeader

    sys.path.insert(0, HERE)
    import cases

    out = []
    for dtype, shape in cases.HEADER_MATRIX:
        raw = TensorHeader(dtype=dtype, shape=torch.Size(shape)).to_bytes()
        out.append({"dtype": str(dtype), "shape": list(shape), "hex": raw.hex()})
    return out


def _narrow(workdir: str) -> list:
    import torch
    from torch.distributed.checkpoint.filesystem import _StorageInfo
    from torch.distributed.checkpoint.metadata import MetadataIndex
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.core.checkpoint_loader import DefaultMLFlashpointCheckpointLoader
    from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver

    sys.path.insert(0, HERE)
    import cases

    com = CheckpointObjectManager()
    saver = DefaultMLFlashpointCheckpointSaver(
        global_rank_getter=lambda: 0,
        local_rank_getter=lambda: 0,
        global_barrier_func=lambda: None,
        ckpt_obj_manager=com,
        replication_manager=None,
        initial_buffer_size_bytes=1024 * 1024,
    )
    loader = DefaultMLFlashpointCheckpointLoader(
        com,
        None,
        global_rank_getter=lambda: 0,
        local_rank_getter=lambda: 0,
        broadcast_object_list_func=lambda *a, **k: None,
        all_gather_object_func=lambda *a, **k: None,
        world_size_getter=lambda: 1,
    )
    ckpt = CheckpointContainerId(os.path.join(workdir, "narrow", "step-1_ckpt"))
    saver.initialize_checkpoint(ckpt)
    tensors = {f"n.{i}": cases.narrow_source(i) for i in range(len(cases.NARROW_CASES))}
    items, resolver = cases.write_items_and_resolver({"tensors": tensors, "blobs": {}})
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=1)
    results = saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=1)
    storage = {r.index: r.storage_data for r in results}

    out = []
    for i, (shape, dtype, offs, lens) in enumerate(cases.NARROW_CASES):
        idx = MetadataIndex(f"n.{i}", torch.Size([0] * len(shape)))
        target = torch.zeros(lens, dtype=dtype)
        req = ReadItem(
            type=LoadItemType.TENSOR,
            dest_index=idx,
            dest_offsets=torch.Size([0] * len(lens)),
            storage_index=idx,
            storage_offsets=torch.Size(offs),
            lengths=torch.Size(lens),
        )

        class _Planner:
            def resolve_tensor(self, read_item):
                return target

            def commit_tensor(self, read_item, tensor):
                pass

        loader.read_data(buckets[0].object_id, [req], _Planner(), {idx: storage[idx]})
        raw = target.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        out.append(
            {
                "i": i,
                "shape": list(shape),
                "dtype": str(dtype),
                "storage_offsets": list(offs),
                "lengths": list(lens),
                "hex": raw.hex(),
            }
        )
    return out


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MLF_REFERENCE_ROOT")
    if not ref_root:
        sys.exit("usage: generate_golden.py /path/to/ml-flashpoint   (or set MLF_REFERENCE_ROOT)")
    _install_reference(ref_root)
    sys.path.insert(0, HERE)
    import cases

    workdir = tempfile.mkdtemp(prefix="mlf_golden_")
    try:
        for name, make in cases.CASES.items():
            record = _save_case(name, make(), workdir)
            with open(os.path.join(HERE, f"{name}.json"), "w") as f:
                json.dump(record, f, indent=1)
            print(name, [(o["name"], o["size"]) for o in record["objects"]])
        with open(os.path.join(HERE, "headers.json"), "w") as f:
            json.dump(_headers(), f, indent=0)
        with open(os.path.join(HERE, "narrow.json"), "w") as f:
            json.dump(_narrow(workdir), f, indent=1)
    finally:
        shutil.rmtree(workdir, ignore_errors=True)


if __name__ == "__main__":
    main()
