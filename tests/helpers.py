"""Test-side helpers: golden loading, a saver/loader factory and a numpy stand-in for the CUDA engine.

``NumpyCopyEngine`` executes the product's layouts and read lists with the CPU oracle's byte
routines. It exists so that host logic (naming, bucketing, cursors, metadata, collectives) can be
tested without a GPU; it is test infrastructure and never part of the product path.
"""

import ctypes
import json
import os

import numpy as np
import torch

import mlf_oracle as oracle


def load_golden(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return json.load(f)


def golden_object_bytes(golden_dir, entry):
    with open(os.path.join(golden_dir, entry["file"]), "rb") as f:
        return f.read()


class _FiredEvent:
    def synchronize(self):
        pass

    def query(self):
        return True


class _FinishedTicket:
    """What ``pack_async`` returns when the work is already done (the stand-in engine is synchronous)."""

    mutate_event = _FiredEvent()
    done_event = _FiredEvent()

    def wait(self):
        pass


class NumpyCopyEngine:
    """Drop-in for ``CudaCopyEngine`` in CPU tests: same ``pack`` / ``pack_async`` / ``unpack`` signatures."""

    def pack_async(self, layout, buffer_io, start_pos=0, object_id=None):
        self.pack(layout, buffer_io, start_pos, object_id)
        return _FinishedTicket()

    def pack(self, layout, buffer_io, start_pos=0, object_id=None):
        base = buffer_io.host_address(start_pos)
        image = (ctypes.c_ubyte * max(layout.total_bytes, 1)).from_address(base)
        view = memoryview(image).cast("B")
        for chunk in layout.host_chunks:
            view[chunk.offset : chunk.offset + len(chunk.data)] = chunk.data
        for placement in layout.tensors:
            raw = oracle.tensor_payload(placement.tensor.cpu())
            view[placement.payload_offset : placement.payload_offset + len(raw)] = raw

    def unpack(self, reads, buffer_io):
        for target, image_off, stored_shape, storage_offsets in reads:
            if target.numel() == 0:
                continue
            esize = target.element_size()
            numel = int(np.prod(stored_shape, dtype=np.int64)) if len(stored_shape) else 1
            raw = (ctypes.c_ubyte * (numel * esize)).from_address(buffer_io.host_address(image_off))
            arr = np.frombuffer(raw, dtype=np.uint8).reshape(tuple(stored_shape) + (esize,))
            index = tuple(slice(int(o), int(o) + int(n)) for o, n in zip(storage_offsets, target.shape))
            block = np.ascontiguousarray(arr[index]).reshape(-1)
            flat = torch.from_numpy(block.copy())
            carrier = torch.empty(target.shape, dtype=target.dtype)
            carrier.view(torch.uint8).reshape(-1).copy_(flat) if carrier.dim() else carrier.reshape(1).view(torch.uint8).copy_(flat)
            target.copy_(carrier)


def make_saver(copy_engine=None, rank=0, pool_config=None, initial_buffer_size_bytes=8 * 1024 * 1024, replication_manager=None, **kw):
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver

    com = CheckpointObjectManager(pool_config)
    saver = DefaultMLFlashpointCheckpointSaver(
        global_rank_getter=lambda: rank,
        local_rank_getter=lambda: rank,
        global_barrier_func=lambda: None,
        ckpt_obj_manager=com,
        replication_manager=replication_manager,
        initial_buffer_size_bytes=initial_buffer_size_bytes,
        copy_engine=copy_engine,
        **kw,
    )
    return saver, com


def make_loader(com, copy_engine=None, rank=0, world=1, replication_manager=None):
    from ml_flashpoint.core.checkpoint_loader import DefaultMLFlashpointCheckpointLoader

    return DefaultMLFlashpointCheckpointLoader(
        com,
        replication_manager,
        global_rank_getter=lambda: rank,
        local_rank_getter=lambda: rank,
        broadcast_object_list_func=lambda *a, **k: None,
        all_gather_object_func=lambda out, obj: out.__setitem__(slice(None), [obj] * len(out)),
        world_size_getter=lambda: world,
        copy_engine=copy_engine,
    )


def case_to_device(case, device):
    """Moves a case's tensors to ``device`` keeping shape AND strides (views stay views)."""
    moved = {}
    for name, t in case["tensors"].items():
        if t.numel() == 0 or t.is_contiguous():
            moved[name] = t.to(device)
            continue
        # rebuild the same strided view over a device copy of the minimal covering storage
        span = 1 + sum((s - 1) * st for s, st in zip(t.shape, t.stride()))
        flat = torch.as_strided(t, (span,), (1,)).to(device)
        moved[name] = torch.as_strided(flat, tuple(t.shape), tuple(t.stride()))
    return {"tensors": moved, "blobs": case["blobs"], "bucket_count": case["bucket_count"]}


def tensor_bytes(t: torch.Tensor) -> bytes:
    return oracle.tensor_payload(t.detach().cpu())
