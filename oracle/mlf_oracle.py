"""CPU oracle for the checkpoint object format (TEST INFRASTRUCTURE, not product code).

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this module;
the product package never does. It restates, in numpy and plain Python, what the reference
implementation (google/ml-flashpoint) does on the save / restore data path, citing the
reference file and line for each step. Parity is pinned: ``tests/golden/`` holds object files,
write results, header bytes and loader outputs produced by running the reference's own
Python code (see ``tests/golden/generate_golden.py``) and ``tests/test_oracle_golden.py``
checks every function here against them.

Deliberately independent of the product: header bytes are assembled opcode by opcode from the
pickle protocol-4 specification instead of calling ``pickle.dumps`` on the product's
``TensorHeader`` class, and strided gathers go through numpy rather than torch ``copy_``.
"""

from __future__ import annotations

import struct
from typing import Iterable, List, Sequence, Tuple

import numpy as np

METADATA_SIZE = 4096  # checkpoint_object_manager/buffer_metadata.py:17
SIGNATURE_MLF = b"MLF_TENS"  # core/defaults.py:27
HEADER_MODULE = "ml_flashpoint.core.tensor_header"  # module path embedded by pickle (core/tensor_header.py:23)
HEADER_CLASS = "TensorHeader"

# torch dtype name -> (itemsize, numpy dtype used to carry the raw bytes)
DTYPES = {
    "float32": (4, np.uint32),
    "bfloat16": (2, np.uint16),
    "float16": (2, np.uint16),
    "float64": (8, np.uint64),
    "int64": (8, np.uint64),
    "int32": (4, np.uint32),
    "int16": (2, np.uint16),
    "int8": (1, np.uint8),
    "uint8": (1, np.uint8),
    "bool": (1, np.uint8),
    "complex64": (8, np.uint64),
    "complex128": (16, None),
}


# --------------------------------------------------------------------------------------
# Header: [u32 LE length][pickle(TensorHeader(dtype, shape))]      core/tensor_header.py:30-39
# --------------------------------------------------------------------------------------
def _short_str(s: str) -> bytes:
    raw = s.encode("utf-8")
    assert len(raw) < 256
    return b"\x8c" + bytes([len(raw)]) + raw + b"\x94"  # SHORT_BINUNICODE + MEMOIZE


def _pickle_int(v: int) -> bytes:
    """Protocol-4 integer encodings in the order CPython's pickler tries them."""
    if 0 <= v < 256:
        return b"K" + bytes([v])  # BININT1
    if 0 <= v < 65536:
        return b"M" + struct.pack("<H", v)  # BININT2
    if -(2**31) <= v < 2**31:
        return b"J" + struct.pack("<i", v)  # BININT
    nbytes = (v.bit_length() >> 3) + 1
    enc = v.to_bytes(nbytes, "little", signed=True)
    if v < 0 and nbytes > 1 and enc[-1] == 0xFF and (enc[-2] & 0x80):
        enc = enc[:-1]
    return b"\x8a" + bytes([len(enc)]) + enc  # LONG1


def _pickle_int_tuple(dims: Sequence[int]) -> bytes:
    body = b"".join(_pickle_int(int(d)) for d in dims)
    if len(dims) == 0:
        return b")"  # EMPTY_TUPLE is never memoized
    if len(dims) <= 3:
        return body + (b"\x85", b"\x86", b"\x87")[len(dims) - 1] + b"\x94"
    return b"(" + body + b"t\x94"  # MARK ... TUPLE


def header_bytes(dtype_name: str, shape: Sequence[int]) -> bytes:
    """Bytes ``TensorHeader(dtype, shape).to_bytes()`` yields (core/tensor_header.py:30-39).

    The pickle of a dataclass instance is NEWOBJ of its class with the instance ``__dict__`` as
    state; ``torch.dtype`` pickles as the global ``torch.<name>`` and ``torch.Size`` reduces to
    ``torch.Size(tuple)``.
    """
    body = (
        _short_str(HEADER_MODULE)
        + _short_str(HEADER_CLASS)
        + b"\x93\x94"  # STACK_GLOBAL
        + b")\x81\x94"  # EMPTY_TUPLE NEWOBJ
        + b"}\x94("  # EMPTY_DICT MARK
        + _short_str("dtype")
        + _short_str("torch")
        + _short_str(dtype_name)
        + b"\x93\x94"
        + _short_str("shape")
        + _short_str("torch")
        + _short_str("Size")
        + b"\x93\x94"
        + _pickle_int_tuple(shape)
        + b"\x85\x94R\x94"  # TUPLE1 REDUCE
        + b"ub."  # SETITEMS BUILD STOP
    )
    pickled = b"\x80\x04\x95" + struct.pack("<Q", len(body)) + body  # PROTO 4, FRAME
    return struct.pack("<I", len(pickled)) + pickled


def parse_header(buf: bytes) -> Tuple[str, Tuple[int, ...], int]:
    """Inverse of :func:`header_bytes`: ``(dtype_name, shape, bytes_consumed)``.

    Follows the loader's framing (core/checkpoint_loader.py:194-205): 4-byte LE length, then
    that many pickle bytes. Walks only the opcodes the header can contain.
    """
    (hlen,) = struct.unpack_from("<I", buf, 0)
    p = bytes(buf[4 : 4 + hlen])
    assert p[:2] == b"\x80\x04", "not a protocol-4 pickle"
    i = 2
    strings: List[str] = []
    ints: List[int] = []
    while i < len(p):
        op = p[i : i + 1]
        i += 1
        if op == b"\x95":
            i += 8
        elif op == b"\x8c":
            n = p[i]
            strings.append(p[i + 1 : i + 1 + n].decode())
            i += 1 + n
        elif op == b"K":
            ints.append(p[i])
            i += 1
        elif op == b"M":
            ints.append(struct.unpack_from("<H", p, i)[0])
            i += 2
        elif op == b"J":
            ints.append(struct.unpack_from("<i", p, i)[0])
            i += 4
        elif op == b"\x8a":
            n = p[i]
            ints.append(int.from_bytes(p[i + 1 : i + 1 + n], "little", signed=True))
            i += 1 + n
        elif op == b".":
            break
        # every other opcode in a header carries no operand bytes
    assert strings[:2] == [HEADER_MODULE, HEADER_CLASS], strings
    dtype_name = strings[strings.index("dtype") + 2]
    return dtype_name, tuple(ints), 4 + hlen


# --------------------------------------------------------------------------------------
# Tensor payload: logical C-order bytes whatever the source strides (checkpoint_saver.py:764-800)
# --------------------------------------------------------------------------------------
def tensor_payload(tensor) -> bytes:
    """Raw little-endian bytes of ``tensor`` in logical C order.

    ``tensor`` is a CPU torch tensor (possibly a strided view). The strided gather is done by
    numpy on an integer view of the same item size, so no torch copy kernel is involved.
    """
    import torch

    name = str(tensor.dtype).split(".")[-1]
    itemsize, carrier = DTYPES[name]
    if tensor.numel() == 0:
        return b""
    t = tensor.detach()
    if carrier is None:  # complex128: two float64 halves, innermost and contiguous
        t = torch.view_as_real(t)
        carrier, itemsize = np.uint64, 8
    torch_carrier = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[itemsize]
    if t.dtype == torch.bool:
        t = t.view(torch.uint8)
    elif t.dtype != torch_carrier:
        t = t.view(torch_carrier)  # same item size: legal for any strides
    base = t.numpy() if t.dim() else t.reshape(1).numpy()
    return np.ascontiguousarray(base).view(np.uint8).tobytes()


# --------------------------------------------------------------------------------------
# Bucketing (torch/distributed/checkpoint/filesystem.py `_split_by_size_and_type`, the function the
# reference calls at core/checkpoint_saver.py:407)
# --------------------------------------------------------------------------------------
def split_by_size_and_type(bins: int, items: Sequence[Tuple[str, bool, int]]) -> List[List[int]]:
    """``items[i] = (name, is_bytes, tensor_nbytes)``; returns item indices per bucket.

    One bin keeps plan order. Otherwise blobs go round-robin and tensors, largest first
    (stable), each to the currently lightest bucket (lowest index on ties).
    """
    if bins == 1:
        return [list(range(len(items)))]
    blobs = [i for i, it in enumerate(items) if it[1]]
    tensors = [i for i, it in enumerate(items) if not it[1]]
    buckets: List[List[int]] = [[] for _ in range(bins)]
    sizes = [0] * bins
    tensors.sort(key=lambda i: items[i][2], reverse=True)
    for k, i in enumerate(blobs):
        buckets[k % bins].append(i)
    for i in tensors:
        b = min(range(bins), key=lambda j: sizes[j])
        buckets[b].append(i)
        sizes[b] += items[i][2]
    return buckets


# --------------------------------------------------------------------------------------
# Whole object: metadata block + data section            checkpoint_saver.py:621-707, buffer_io.py
# --------------------------------------------------------------------------------------
def pack_object(tensors: Iterable[Tuple[str, object]], blobs: Iterable[Tuple[str, bytes]]):
    """Serialises one bucket. Returns ``(object_bytes, records)``.

    Layout (buffer_metadata.py:18-37, checkpoint_saver.py:662-698):
      [0,8) u64 LE length of the data section; [8,16) ``MLF_TENS``; [16,4096) zero;
      then every tensor in bucket order as header + payload, then every blob, unpadded.
    ``records`` = ``(name, offset, length)`` with offsets relative to byte 4096, exactly the
    ``_StorageInfo`` fields the saver reports (checkpoint_saver.py:675-681, 690-696).
    """
    data = bytearray()
    records = []
    for name, tensor in tensors:
        start = len(data)
        dtype_name = str(tensor.dtype).split(".")[-1]
        data += header_bytes(dtype_name, tuple(tensor.shape))
        data += tensor_payload(tensor)
        records.append((name, start, len(data) - start))
    for name, blob in blobs:
        start = len(data)
        data += blob
        records.append((name, start, len(data) - start))
    meta = struct.pack("<Q", len(data)) + SIGNATURE_MLF + bytes(METADATA_SIZE - 16)
    return bytes(meta) + bytes(data), records


def object_sha256(tensors: Sequence[Tuple[str, object]], blobs: Sequence[Tuple[str, bytes]] = ()) -> Tuple[str, int]:
    """SHA-256 and size of the object ``pack_object`` would produce, without building it.

    Meant for objects too large to hold in host memory a second time. The metadata block at offset 0
    carries the length of the data section, so a first pass adds that length up from shapes and
    dtypes alone; the second pass feeds the hash piece by piece: metadata block, then header and
    payload of every tensor in bucket order, then the blobs. Tensors may live on any device; each
    is brought to the host only while its payload is hashed.
    """
    import hashlib

    length = 0
    for _, tensor in tensors:
        length += len(header_bytes(str(tensor.dtype).split(".")[-1], tuple(tensor.shape)))
        length += tensor.numel() * tensor.element_size()
    length += sum(len(b) for _, b in blobs)
    digest = hashlib.sha256()
    digest.update(struct.pack("<Q", length) + SIGNATURE_MLF + bytes(METADATA_SIZE - 16))
    for _, tensor in tensors:
        digest.update(header_bytes(str(tensor.dtype).split(".")[-1], tuple(tensor.shape)))
        host = tensor if tensor.device.type == "cpu" else tensor.cpu()
        digest.update(tensor_payload(host))
        del host
    for _, blob in blobs:
        digest.update(blob)
    return digest.hexdigest(), METADATA_SIZE + length


def save_case(case: dict, prefix: str = "__0_", rank: int = 0):
    """Runs bucketing + naming + packing for a ``tests/golden/cases.py`` case.

    Returns ``[(object_name, object_bytes, records)]``. Object names follow
    ``{prefix}_{bucket}_src{rank}.distcp`` (checkpoint_saver.py:382-388); empty buckets get no
    object and do not consume an index (checkpoint_saver.py:409-420).
    """
    names = list(case["tensors"].keys()) + list(case["blobs"].keys())
    objs = list(case["tensors"].values()) + list(case["blobs"].values())
    items = [
        (n, isinstance(o, (bytes, bytearray)), 0 if isinstance(o, (bytes, bytearray)) else o.numel() * o.element_size())
        for n, o in zip(names, objs)
    ]
    out = []
    k = 0
    for bucket in split_by_size_and_type(max(case["bucket_count"], 1), items):
        if not bucket:
            continue
        tens = [(names[i], objs[i]) for i in bucket if not items[i][1]]
        blobs = [(names[i], objs[i]) for i in bucket if items[i][1]]
        data, records = pack_object(tens, blobs)
        out.append((f"{prefix}_{k}_src{rank}.distcp", data, records))
        k += 1
    return out


# --------------------------------------------------------------------------------------
# Restore: header parse + N-d narrow                        core/checkpoint_loader.py:177-219
# --------------------------------------------------------------------------------------
def read_item(object_bytes: bytes, offset: int, length: int, storage_offsets: Sequence[int], lengths: Sequence[int]):
    """Bytes (C order) of the sub-block the loader hands to ``target.copy_``.

    ``offset``/``length`` are the item's ``_StorageInfo`` (relative to byte 4096). The stored tensor
    is reshaped to its header shape and narrowed per dimension by ``storage_offsets``/``lengths``
    (torch ``narrow_tensor_by_index``, called at checkpoint_loader.py:219).
    Returns ``(dtype_name, bytes)``.
    """
    view = memoryview(object_bytes)[METADATA_SIZE + offset : METADATA_SIZE + offset + length]
    dtype_name, shape, used = parse_header(bytes(view[:4096]) if len(view) > 4096 else bytes(view))
    itemsize = DTYPES[dtype_name][0]
    payload = np.frombuffer(view[used:], dtype=np.uint8)
    numel = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    assert payload.size == numel * itemsize
    arr = payload.reshape(tuple(shape) + (itemsize,))
    index = tuple(slice(int(o), int(o) + int(n)) for o, n in zip(storage_offsets, lengths))
    return dtype_name, np.ascontiguousarray(arr[index]).tobytes()


def read_blob(object_bytes: bytes, offset: int, length: int) -> bytes:
    """BYTE_IO items are returned verbatim (checkpoint_loader.py:325-328)."""
    return bytes(object_bytes[METADATA_SIZE + offset : METADATA_SIZE + offset + length])
