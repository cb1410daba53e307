"""The reference's CPU save / restore path, restated for timing (TEST INFRASTRUCTURE).

Only the benchmark's CPU-baseline leg and the tests may import this module. It follows what the
reference does on the host, step by step, with the same torch calls:

  save     stage every tensor with ``tensor.to("cpu", non_blocking=True)`` + one synchronize
           (adapter/pytorch/memory_storage_writer.py:211-233), then per tensor write the header and
           ``torch.frombuffer(slice).reshape(shape).copy_(tensor)`` into the object mapping
           (core/checkpoint_saver.py:764-800) with torch's intra-op thread count set to
           ``cpus // 2 // ranks // writer_threads`` (:443-450), then truncate to the written size.
  restore  per tensor ``read()`` the bytes, ``torch.frombuffer``, reshape, narrow, ``target.copy_``
           (core/checkpoint_loader.py:177-219, :331-336).

Header bytes come from ``mlf_oracle.header_bytes`` so that this module does not depend on the
product package. Objects written here are byte-identical to the product's (checked in tests).
"""

from __future__ import annotations

import mmap
import os
import struct
from typing import Dict, List, Sequence, Tuple

import torch

import mlf_oracle as oracle


def reference_thread_count(ranks_on_host: int, writer_threads: int = 1) -> int:
    return max(1, (os.cpu_count() or 1) // 2 // max(ranks_on_host, 1) // max(writer_threads, 1))


def stage_to_cpu(tensors: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    staged = [t.to(device="cpu", non_blocking=True) for t in tensors]
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    return staged


def write_object(path: str, tensors: Sequence[torch.Tensor], capacity: int) -> List[Tuple[int, int]]:
    """Writes CPU ``tensors`` into a fresh object file; returns ``(offset, length)`` per tensor."""
    fd = os.open(path, os.O_CREAT | os.O_RDWR | os.O_TRUNC, 0o666)
    try:
        os.ftruncate(fd, capacity)
        mapping = mmap.mmap(fd, capacity)
        view = memoryview(mapping)
        pos = oracle.METADATA_SIZE
        records = []
        dest = None
        for t in tensors:
            begin = pos
            header = oracle.header_bytes(str(t.dtype).split(".")[-1], tuple(t.shape))
            view[pos : pos + len(header)] = header
            pos += len(header)
            nbytes = t.numel() * t.element_size()
            if nbytes:
                dest = torch.frombuffer(view[pos : pos + nbytes], dtype=t.dtype, count=t.numel()).reshape(t.shape)
                dest.copy_(t)
                pos += nbytes
            records.append((begin - oracle.METADATA_SIZE, pos - begin))
        written = pos - oracle.METADATA_SIZE
        view[0:16] = struct.pack("<Q", written) + oracle.SIGNATURE_MLF
        dest = None
        view.release()
        mapping.close()
        os.ftruncate(fd, pos)
    finally:
        os.close(fd)
    return records


def read_object(path: str, records: Sequence[Tuple[int, int]], targets: Sequence[torch.Tensor]) -> None:
    """Restores whole tensors from an object into ``targets`` (CPU or CUDA), the reference way."""
    fd = os.open(path, os.O_RDONLY)
    try:
        size = os.fstat(fd).st_size
        mapping = mmap.mmap(fd, size, prot=mmap.PROT_READ)
        view = memoryview(mapping)
        for (offset, length), target in zip(records, targets):
            item = view[oracle.METADATA_SIZE + offset : oracle.METADATA_SIZE + offset + length]
            dtype_name, shape, used = oracle.parse_header(bytes(item[:4096]))
            data = item[used:].tobytes()  # the reference materialises a bytes object per tensor
            if not data:
                continue
            stored = torch.frombuffer(data, dtype=getattr(torch, dtype_name)).reshape(shape)
            target.copy_(stored)
            item.release()
        view.release()
        mapping.close()
    finally:
        os.close(fd)


def timed_save(tensors: Sequence[torch.Tensor], path: str, ranks_on_host: int = 1) -> Dict[str, float]:
    """One reference-style save of ``tensors`` (on any device). Returns wall seconds per phase."""
    import time

    capacity = oracle.METADATA_SIZE + sum(t.numel() * t.element_size() + 256 for t in tensors)
    before = torch.get_num_threads()
    torch.set_num_threads(reference_thread_count(ranks_on_host))
    try:
        t0 = time.perf_counter()
        staged = stage_to_cpu(tensors)
        t1 = time.perf_counter()
        records = write_object(path, staged, capacity)
        t2 = time.perf_counter()
    finally:
        torch.set_num_threads(before)
    return {"stage_s": t1 - t0, "write_s": t2 - t1, "total_s": t2 - t0, "records": records}
