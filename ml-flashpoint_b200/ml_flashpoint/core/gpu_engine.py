"""GPU data mover for checkpoint objects: layout planning plus the CUDA pack / unpack engine.

Two halves:

* ``plan_object_layout`` is pure host arithmetic. It reproduces the byte layout the reference
  saver produces for one object (core/checkpoint_saver.py:667-698 with ``_save_tensor_optimized``
  :764-800): every tensor in bucket order as ``[u32 len][pickled TensorHeader][C-order bytes]``,
  then every BYTE_IO item, no padding. It yields the storage records and, per tensor, the box-copy
  descriptor the kernel needs. It touches no CUDA API.

* ``CudaCopyEngine`` executes layouts. Save: ONE gather-pack kernel per object reads all tensors
  (any strides) plus a pinned blob holding headers and byte items and writes the finished data
  section, either straight into the page-locked object mapping ("direct") or into an HBM image
  that a copy engine then drains to the mapping ("staged", the default: training may resume as
  soon as the kernel is done, a few milliseconds, while the PCIe transfer continues).
  Restore: the mirror scatter-unpack kernel, fed from an HBM copy of the needed image range.

There is no CPU data path: without the native library or a CUDA device the engine raises.
"""

from __future__ import annotations

import ctypes
import dataclasses
import threading
from collections import OrderedDict
from typing import Any, List, Optional, Sequence, Tuple

import torch

from ml_flashpoint import _native
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.tensor_header import TensorHeader
from ml_flashpoint.core.utils import get_env_val_int, get_env_val_str

_LOGGER = get_logger(__name__)

MAX_DIMS = _native.MLF_MAX_DIMS


# ======================================================================================
# Layout planning (host only)
# ======================================================================================
@dataclasses.dataclass
class LayoutRecord:
    """Where one item landed: the fields of the ``_StorageInfo`` / ``WriteResult`` for it."""

    item: Any  # the WriteItem (or any caller token)
    offset: int  # relative to the start of the data section
    length: int  # header + payload for tensors, byte count for blobs


@dataclasses.dataclass
class TensorPlacement:
    tensor: torch.Tensor
    payload_offset: int  # data-section offset of the first payload byte


@dataclasses.dataclass
class HostChunk:
    offset: int  # data-section offset
    data: bytes


@dataclasses.dataclass
class ObjectLayout:
    total_bytes: int
    records: List[LayoutRecord]
    tensors: List[TensorPlacement]
    host_chunks: List[HostChunk]
    payload_bytes: int

    def host_blob_size(self) -> int:
        return sum(len(c.data) for c in self.host_chunks)


_HEADER_CACHE: dict = {}


def _header_bytes(dtype: torch.dtype, shape: torch.Size) -> bytes:
    """Pickled header for (dtype, shape); identical inputs pickle to identical bytes, so cache them."""
    key = (dtype, tuple(shape))
    cached = _HEADER_CACHE.get(key)
    if cached is None:
        if len(_HEADER_CACHE) > 65536:
            _HEADER_CACHE.clear()
        cached = _HEADER_CACHE[key] = TensorHeader(dtype=dtype, shape=shape).to_bytes()
    return cached


def plan_object_layout(
    tensor_items: Sequence[Tuple[Any, torch.Tensor]],
    bytes_items: Sequence[Tuple[Any, Any]],
    start_offset: int = 0,
) -> ObjectLayout:
    """Lays out one object's data section: tensors first (bucket order), then byte items.

    ``bytes_items`` values are ``io.BytesIO``-likes (read from position 0) or ``bytes``.
    Zero-element tensors get a header and no payload, as in the reference (:789).
    """
    pos = start_offset
    records: List[LayoutRecord] = []
    placements: List[TensorPlacement] = []
    chunks: List[HostChunk] = []
    payload_total = 0
    for item, tensor in tensor_items:
        begin = pos
        header = _header_bytes(tensor.dtype, tensor.shape)
        chunks.append(HostChunk(pos, header))
        pos += len(header)
        nbytes = tensor.numel() * tensor.element_size()
        if nbytes:
            placements.append(TensorPlacement(tensor, pos))
            pos += nbytes
            payload_total += nbytes
        records.append(LayoutRecord(item, begin, pos - begin))
    for item, blob in bytes_items:
        if hasattr(blob, "seek"):
            blob.seek(0)
            data = blob.read()
        else:
            data = bytes(blob)
        if data:
            chunks.append(HostChunk(pos, data))
        records.append(LayoutRecord(item, pos, len(data)))
        pos += len(data)
    return ObjectLayout(pos - start_offset, records, placements, chunks, payload_total)


def split_layout(layout: ObjectLayout, piece_limit: int) -> Tuple[int, List[Tuple[int, int, List[TensorPlacement], List[HostChunk]]]]:
    """Cuts a layout into consecutive image ranges for a save through a bounded arena.

    Returns ``(slot_bytes, [(lo, hi, tensors, host_chunks)])``: every range holds whole items only (a
    header, a tensor's payload or a byte item is never cut), ranges follow one another without gaps
    in image order, and none is longer than ``slot_bytes`` = ``max(piece_limit, largest item)``.
    """
    items = [(p.payload_offset, p.tensor.numel() * p.tensor.element_size(), 0, p) for p in layout.tensors]
    items += [(c.offset, len(c.data), 1, c) for c in layout.host_chunks]
    items.sort(key=lambda it: (it[0], it[2]))
    slot = max([piece_limit] + [n for _, n, _, _ in items])
    pieces = []
    lo = hi = None
    tensors, chunks = [], []
    for off, n, kind, obj in items:
        if lo is not None and off + n - lo > slot:
            pieces.append((lo, hi, tensors, chunks))
            lo, tensors, chunks = None, [], []
        if lo is None:
            lo = off
        hi = off + n
        (chunks if kind else tensors).append(obj)
    if lo is not None:
        pieces.append((lo, hi, tensors, chunks))
    return slot, pieces


def c_strides(shape: Sequence[int]) -> List[int]:
    out = [1] * len(shape)
    for d in range(len(shape) - 2, -1, -1):
        out[d] = out[d + 1] * max(int(shape[d + 1]), 1)
    return out


def fill_desc(
    desc: _native.CopyDesc,
    tensor_ptr: int,
    image_off: int,
    elem_size: int,
    shape: Sequence[int],
    tensor_stride: Sequence[int],
    image_stride: Sequence[int],
) -> None:
    if len(shape) > MAX_DIMS:
        raise ValueError(f"tensors with more than {MAX_DIMS} dimensions are not supported, got {len(shape)}")
    desc.tensor_ptr = tensor_ptr
    desc.image_off = image_off
    desc.elem_size = elem_size
    desc.ndim = len(shape)
    for d in range(len(shape)):
        desc.shape[d] = int(shape[d])
        desc.tensor_stride[d] = int(tensor_stride[d])
        desc.image_stride[d] = int(image_stride[d])


def default_host_threads(share: float = 0.5) -> int:
    """CPU threads for the bounce ring: ``share`` of the cores, divided between the ranks on this host."""
    import os

    local_world = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1") or 1))
    return max(2, int((os.cpu_count() or 2) * share) // local_world)


def default_restore_lock_run_mib() -> int:
    """Whether a restore runs its lock lane by default, and with which run size: it does not.
    Measured on B200 hosts, page-locking pieces of the object while the pread() threads issue their
    copies slows both down (the driver serialises the calls inside a process); the lane stays
    available through ``MLFLASHPOINT_GPU_RESTORE_LOCK_RUN_MIB`` for hosts where cores are scarcer."""
    return 0


# ======================================================================================
# CUDA engine
# ======================================================================================
class _PinnedBlob:
    """Page-locked, device-mapped host scratch for headers and byte items (kernel reads it in place)."""

    def __init__(self, nbytes: int):
        self.nbytes = max(nbytes, 1)
        ptr = ctypes.c_void_p()
        _native.check(_native.lib().mlf_host_alloc(self.nbytes, ctypes.byref(ptr)))
        self.ptr = int(ptr.value)

    def fill(self, chunks: Sequence[HostChunk]) -> None:
        packed = b"".join(c.data for c in chunks)
        ctypes.memmove(self.ptr, packed, len(packed))

    def __del__(self):
        try:
            _native.lib().mlf_host_free(ctypes.c_void_p(self.ptr))
        except Exception:
            pass


class _Plan:
    def __init__(self, descs, n: int, direction: int):
        handle = ctypes.c_void_p()
        _native.check(_native.lib().mlf_plan_create(descs, n, direction, ctypes.byref(handle)))
        self.handle = handle
        self.extent = int(_native.lib().mlf_plan_image_extent(handle))
        self.payload = int(_native.lib().mlf_plan_payload_bytes(handle))

    def launch(self, image_base: int, capacity: int, stream: int, max_ctas: int = 0) -> None:
        _native.check(
            _native.lib().mlf_plan_launch(
                self.handle, ctypes.c_void_p(image_base), capacity, ctypes.c_void_p(stream), max_ctas
            )
        )

    def status(self) -> None:
        _native.check(_native.lib().mlf_plan_status(self.handle))

    def __del__(self):
        try:
            _native.lib().mlf_plan_destroy(self.handle)
        except Exception:
            pass


@dataclasses.dataclass
class _CachedPack:
    plan: _Plan
    blob: _PinnedBlob
    keepalive: list  # device copies of CPU tensors referenced by the plan
    last_kernel: Optional["torch.cuda.Event"] = None  # the last launch that read ``blob``


@dataclasses.dataclass
class _CachedCappedPack:
    """Plans of a save that goes through the bounded arena piece by piece."""

    slot_bytes: int
    pieces: list  # (lo, hi, _Plan)
    blob: _PinnedBlob
    keepalive: list
    last_kernel: Optional["torch.cuda.Event"] = None

    @property
    def plan(self):  # status of the last piece's plan stands for the save (every piece is checked in wait)
        return self

    def status(self) -> None:
        for _, _, plan in self.pieces:
            plan.status()


@dataclasses.dataclass(eq=False)
class _Image:
    """One object image inside the engine's HBM arena."""

    offset: int
    nbytes: int
    done: "torch.cuda.Event"  # fires when the transfer out of the region has finished
    object_id: Optional[str]
    ready: Optional["torch.cuda.Event"] = None  # fires when the pack kernel has written the whole image
    start: Optional["torch.cuda.Event"] = None  # recorded right before the pack kernel (timing)

    def overlaps(self, offset: int, nbytes: int) -> bool:
        return self.offset < offset + nbytes and offset < self.offset + self.nbytes


class PackTicket:
    """Handle of an in-flight save of one object.

    ``mutate_event`` fires when the pack kernel has read every source tensor: from then on the
    training loop may overwrite parameters and optimizer state. ``done_event`` fires when the last
    byte has reached the object mapping. ``wait()`` blocks on the latter and surfaces kernel status.
    """

    def __init__(self, engine: "CudaCopyEngine", cached: _CachedPack, start_event, mutate_event, done_event, nbytes: int):
        self._engine = engine
        self._cached = cached
        self.start_event = start_event
        self.mutate_event = mutate_event
        self.done_event = done_event
        self.nbytes = nbytes

    def wait(self) -> None:
        self.done_event.synchronize()
        self._cached.plan.status()

    def kernel_ms(self) -> float:
        """Device time of the pack kernel (valid after ``wait``)."""
        return self.start_event.elapsed_time(self.mutate_event)

    def total_ms(self) -> float:
        """Device time from kernel start to the last byte reaching the object mapping."""
        return self.start_event.elapsed_time(self.done_event)


class CudaCopyEngine:
    """Runs pack and unpack plans on one CUDA device.

    ``mode`` is ``"staged"`` (kernel writes an HBM image, a copy engine moves it to the object
    mapping) or ``"direct"`` (kernel writes the page-locked mapping itself). Environment override:
    ``MLFLASHPOINT_GPU_PACK_MODE``. ``host_ctas`` bounds the grid of kernels that write to or read
    from host memory, where a handful of CTAs saturate the link (``MLFLASHPOINT_GPU_HOST_CTAS``).
    """

    def __init__(self, device: Optional[torch.device] = None, mode: Optional[str] = None, plan_cache_size: int = 8,
                 arena_limit_bytes: Optional[int] = None):
        _native.lib()  # fail here, loudly, if the native library is absent
        if not torch.cuda.is_available():
            raise RuntimeError(
                "CudaCopyEngine needs a CUDA device: checkpoint bytes are moved by CUDA kernels and there is "
                "no CPU data path in this package."
            )
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.mode = (mode or get_env_val_str("GPU_PACK_MODE", "staged")).lower()
        if self.mode not in ("staged", "direct"):
            raise ValueError(f"unknown pack mode '{self.mode}' (expected 'staged' or 'direct')")
        self.host_ctas = get_env_val_int("GPU_HOST_CTAS", 32)
        # Upper bound on the HBM image arena (0 = none: the arena holds the whole save, which lets
        # training resume after the few milliseconds of the pack kernels and leaves a resident image
        # for replication). With a bound, a larger save is packed and drained piece by piece through
        # two arena halves: the tensors stay read-locked until the last piece is packed, i.e. for most
        # of the host transfer, and replication sends from the host mapping.
        self.arena_limit = int(arena_limit_bytes if arena_limit_bytes is not None else get_env_val_int("GPU_ARENA_LIMIT_BYTES", 0))
        self._slot_free: list = [None, None]  # bounded mode: event after which arena half k may be rewritten
        # CPU threads feeding the bounce ring when host memory is not page-locked (0 = half the cores)
        self.host_threads = get_env_val_int("GPU_HOST_THREADS", default_host_threads())
        # a restore runs before training starts, with the host otherwise idle: it may use every core
        self.restore_threads = get_env_val_int("GPU_RESTORE_THREADS", default_host_threads(1.0))
        # MiB the restore's lock lane page-locks at a time (0 = no lane, CPU threads only); see
        # ``mlf_buf_read_to_device_hybrid``. -1 = decide from the ranks that share this host's cores.
        self.restore_lock_run_mib = get_env_val_int("GPU_RESTORE_LOCK_RUN_MIB", -1)
        if self.restore_lock_run_mib < 0:
            self.restore_lock_run_mib = default_restore_lock_run_mib()
        self.last_lock_lane_bytes = 0
        self._lock = threading.RLock()
        self._cache: "OrderedDict[tuple, _CachedPack]" = OrderedDict()
        self._cache_size = plan_cache_size
        # HBM arena holding the images of the objects being saved (and the image of a restore).
        # Regions are handed out front to back within one save (``begin_save``), so the buckets of a
        # multi-object save are packed back to back while earlier ones still drain to the host.
        self._arena: Optional[torch.Tensor] = None
        self._arena_goal = 0  # bytes the arena should hold: the largest save announced so far
        self._cursor = 0
        self._images: List[_Image] = []  # regions whose contents are still valid, oldest first
        # object id -> event of the latest transfer into that object's mapping (kept after the image is reused)
        self._drains: "OrderedDict[str, torch.cuda.Event]" = OrderedDict()
        self._active_read: Optional["_ObjectRead"] = None  # a restore's image being filled right now
        self.last_ticket: Optional[PackTicket] = None  # most recent save, for timing queries
        self.last_unpack_ms: Optional[Tuple[float, float]] = None  # (host-to-HBM ms, kernel ms) of the last restore
        with torch.cuda.device(self.device):
            self._bind()
            self.pack_stream = torch.cuda.Stream(device=self.device)
            self.copy_stream = torch.cuda.Stream(device=self.device)

    # ------------------------------------------------------------------ helpers
    def _bind(self) -> None:
        _native.check(_native.lib().mlf_set_device(self.device.index))

    @staticmethod
    def _is_registered(buffer_io) -> bool:
        obj = getattr(buffer_io, "buffer_obj", None)
        return bool(getattr(obj, "is_cuda_registered", False))

    _ARENA_ALIGN = 256

    def _ensure_arena(self, nbytes: int) -> None:
        """Makes the arena at least ``nbytes`` (and the announced goal) large. Growing it waits for
        every transfer that still reads the old one: the allocator knows nothing about those streams."""
        want = max(nbytes, self._arena_goal, 1 << 20)
        if self._arena is not None and self._arena.numel() >= want:
            return
        for image in self._images:
            image.done.synchronize()
        for event in self._slot_free:
            if event is not None:
                event.synchronize()
        self._slot_free = [None, None]
        self._images = []
        self._cursor = 0
        self._arena = None
        self._arena = torch.empty(want, dtype=torch.uint8, device=self.device)

    def begin_save(self, total_bytes: int) -> None:
        """Announces a save whose object images take ``total_bytes`` in all: the arena is sized for
        the whole save and its objects are placed from the front, so none waits for another's transfer."""
        with self._lock, torch.cuda.device(self.device):
            goal = int(total_bytes) + self._ARENA_ALIGN * 64
            if self.arena_limit and goal > self.arena_limit:
                goal = self.arena_limit  # the save goes through the arena piece by piece
            self._arena_goal = max(self._arena_goal, goal)
            self._cursor = 0

    def _reserve_image(self, nbytes: int, stream: "torch.cuda.Stream") -> Tuple[torch.Tensor, int]:
        """Region of ``nbytes`` for a new object image. Work queued on ``stream`` afterwards runs
        after the transfers out of any older image the region overlaps; those images are forgotten."""
        if self._active_read is not None:
            self._active_read.wait()  # a restore's image occupies the arena until it has arrived
            self._active_read = None
        self._ensure_arena(nbytes)
        for event in self._slot_free:  # halves of a piecewise save that may still be draining
            if event is not None:
                stream.wait_event(event)
        self._slot_free = [None, None]
        if self._cursor + nbytes > self._arena.numel():
            self._cursor = 0
        offset = self._cursor
        kept = []
        for image in self._images:
            if image.overlaps(offset, nbytes):
                stream.wait_event(image.done)
            else:
                kept.append(image)
        self._images = kept
        self._cursor = (offset + nbytes + self._ARENA_ALIGN - 1) // self._ARENA_ALIGN * self._ARENA_ALIGN
        return self._arena[offset : offset + nbytes], offset

    def staging(self, nbytes: int) -> torch.Tensor:
        """The front of the arena for a restore's image; every resident object image is given up
        (after the transfers out of them have finished)."""
        self._ensure_arena(nbytes)
        for image in self._images:
            image.done.synchronize()
        for event in self._slot_free:
            if event is not None:
                event.synchronize()
        self._slot_free = [None, None]
        self._images = []
        self._cursor = 0
        return self._arena[:nbytes]

    def release_device_memory(self) -> None:
        """Gives the HBM arena back to the allocator (after the transfers out of it have finished);
        the next save or restore allocates a new one."""
        with self._lock:
            if self._active_read is not None:
                self._active_read.wait()
                self._active_read = None
            for image in self._images:
                image.done.synchronize()
            self._images = []
            self._cursor = 0
            self._arena = None

    def drop_resident_images(self) -> None:
        """Forgets the object images kept in HBM after their saves (they stay valid until reused)."""
        with self._lock:
            for image in self._images:
                image.object_id = None

    @staticmethod
    def _tensor_key(t: torch.Tensor) -> tuple:
        return (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, t.device.type)

    def _build_pack(self, layout: ObjectLayout) -> _CachedPack:
        keepalive = []
        n = len(layout.tensors) + len(layout.host_chunks)
        descs = (_native.CopyDesc * max(n, 1))()
        blob = _PinnedBlob(layout.host_blob_size())
        k = 0
        for placement in layout.tensors:
            t = placement.tensor
            if t.device.type != "cuda":
                # host-resident tensors ride through HBM like everything else
                t = t.to(self.device, non_blocking=False)
                keepalive.append(t)
            elif t.device != self.device:
                raise ValueError(f"tensor lives on {t.device}, engine on {self.device}")
            fill_desc(descs[k], t.data_ptr(), placement.payload_offset, t.element_size(), t.shape, t.stride(), c_strides(t.shape))
            k += 1
        at = blob.ptr
        for chunk in layout.host_chunks:
            fill_desc(descs[k], at, chunk.offset, 1, (len(chunk.data),), (1,), (1,))
            at += len(chunk.data)
            k += 1
        return _CachedPack(_Plan(descs, n, _native.MLF_PACK), blob, keepalive)

    def _pack_entry(self, layout: ObjectLayout) -> _CachedPack:
        has_host_tensor = any(p.tensor.device.type != "cuda" for p in layout.tensors)
        key = (
            tuple(self._tensor_key(p.tensor) + (p.payload_offset,) for p in layout.tensors),
            tuple((c.offset, len(c.data)) for c in layout.host_chunks),
        )
        entry = None if has_host_tensor else self._cache.get(key)
        if entry is None:
            entry = self._build_pack(layout)
            if not has_host_tensor:
                self._cache[key] = entry
                while len(self._cache) > self._cache_size:
                    self._cache.popitem(last=False)
        else:
            self._cache.move_to_end(key)
        if entry.last_kernel is not None:
            # the previous launch of this plan may still be reading the pinned blob about to be refilled
            entry.last_kernel.synchronize()
        entry.blob.fill(layout.host_chunks)
        return entry

    # ------------------------------------------------------------------ save through a bounded arena
    def _capped(self, nbytes: int) -> bool:
        return bool(self.arena_limit) and self.mode == "staged" and nbytes > self.arena_limit

    def _capped_pack_entry(self, layout: ObjectLayout) -> _CachedCappedPack:
        has_host_tensor = any(p.tensor.device.type != "cuda" for p in layout.tensors)
        key = (
            "capped",
            self.arena_limit,
            tuple(self._tensor_key(p.tensor) + (p.payload_offset,) for p in layout.tensors),
            tuple((c.offset, len(c.data)) for c in layout.host_chunks),
        )
        entry = None if has_host_tensor else self._cache.get(key)
        if entry is None:
            slot_bytes, ranges = split_layout(layout, max(self.arena_limit // 2, 4096))
            blob = _PinnedBlob(layout.host_blob_size())
            blob_at = {}
            at = blob.ptr
            for chunk in layout.host_chunks:  # the blob keeps the layout's chunk order (see _PinnedBlob.fill)
                blob_at[chunk.offset] = at
                at += len(chunk.data)
            keepalive, pieces = [], []
            for lo, hi, tensors, chunks in ranges:
                descs = (_native.CopyDesc * max(len(tensors) + len(chunks), 1))()
                k = 0
                for placement in tensors:
                    t = placement.tensor
                    if t.device.type != "cuda":
                        t = t.to(self.device, non_blocking=False)
                        keepalive.append(t)
                    elif t.device != self.device:
                        raise ValueError(f"tensor lives on {t.device}, engine on {self.device}")
                    fill_desc(descs[k], t.data_ptr(), placement.payload_offset - lo, t.element_size(), t.shape, t.stride(), c_strides(t.shape))
                    k += 1
                for chunk in chunks:
                    fill_desc(descs[k], blob_at[chunk.offset], chunk.offset - lo, 1, (len(chunk.data),), (1,), (1,))
                    k += 1
                pieces.append((lo, hi, _Plan(descs, k, _native.MLF_PACK)))
            entry = _CachedCappedPack(slot_bytes, pieces, blob, keepalive)
            if not has_host_tensor:
                self._cache[key] = entry
                while len(self._cache) > self._cache_size:
                    self._cache.popitem(last=False)
        else:
            self._cache.move_to_end(key)
        if entry.last_kernel is not None:
            entry.last_kernel.synchronize()
        entry.blob.fill(layout.host_chunks)
        return entry

    def _claim_whole_arena(self, nbytes: int, stream: "torch.cuda.Stream") -> None:
        """Bounded mode uses the arena as two halves of its own: images of earlier saves are given
        up (work on ``stream`` waits for the transfers out of them) and a restore in flight is awaited."""
        if self._active_read is not None:
            self._active_read.wait()
            self._active_read = None
        self._arena_goal = max(self._arena_goal, nbytes)
        self._ensure_arena(nbytes)
        for image in self._images:
            stream.wait_event(image.done)
        self._images = []
        self._cursor = 0

    def _pack_capped(self, layout: ObjectLayout, buffer_io, start_pos: int, object_id: Optional[str]) -> PackTicket:
        entry = self._capped_pack_entry(layout)
        slot_bytes = (entry.slot_bytes + self._ARENA_ALIGN - 1) // self._ARENA_ALIGN * self._ARENA_ALIGN
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        self.pack_stream.wait_event(ready)
        self._claim_whole_arena(2 * slot_bytes, self.pack_stream)
        start_event = torch.cuda.Event(enable_timing=True)
        mutate_event = torch.cuda.Event(enable_timing=True)
        done_event = torch.cuda.Event(enable_timing=True)
        registered = self._is_registered(buffer_io)
        start_event.record(self.pack_stream)
        for k, (lo, hi, plan) in enumerate(entry.pieces):
            half = k % 2
            slot = self._arena[half * slot_bytes : half * slot_bytes + (hi - lo)]
            if self._slot_free[half] is not None:
                self.pack_stream.wait_event(self._slot_free[half])  # the piece before last has left this half
            plan.launch(slot.data_ptr(), hi - lo, self.pack_stream.cuda_stream)
            packed = torch.cuda.Event()
            packed.record(self.pack_stream)
            if registered:
                self.copy_stream.wait_event(packed)
                _native.check(
                    _native.lib().mlf_memcpy_async(
                        ctypes.c_void_p(buffer_io.host_address(start_pos + lo)),
                        ctypes.c_void_p(slot.data_ptr()),
                        hi - lo,
                        _native.MLF_COPY_D2H,
                        ctypes.c_void_p(self.copy_stream.cuda_stream),
                    )
                )
                drained = torch.cuda.Event()
                drained.record(self.copy_stream)
            else:
                packed.synchronize()
                _native.check(
                    _native.lib().mlf_bounce_copy(
                        ctypes.c_void_p(slot.data_ptr()), ctypes.c_void_p(buffer_io.host_address(start_pos + lo)), hi - lo, 0, self.host_threads
                    )
                )
                drained = packed
            self._slot_free[half] = drained
        mutate_event.record(self.pack_stream)
        if registered:
            done_event.record(self.copy_stream)
        else:
            done_event.record(self.pack_stream)
        if object_id is not None:
            self._drains[str(object_id)] = done_event
            self._drains.move_to_end(str(object_id))
        entry.last_kernel = mutate_event
        self.last_ticket = PackTicket(self, entry, start_event, mutate_event, done_event, layout.total_bytes)
        return self.last_ticket

    # ------------------------------------------------------------------ save
    def pack_async(self, layout: ObjectLayout, buffer_io, start_pos: int = 0, object_id: Optional[str] = None) -> PackTicket:
        """Starts writing ``layout`` at stream position ``start_pos`` of ``buffer_io``.

        The bytes must already be claimed in ``buffer_io`` (its cursor moved past them). Source
        tensors are read on a side stream ordered after the caller's current stream. If
        ``object_id`` is given and the save is staged, the HBM image stays registered under that id
        until the next save or restore reuses the buffer, so that replication can send it from
        HBM (``resident_image``).
        """
        with self._lock, torch.cuda.device(self.device):
            self._bind()
            if self._capped(layout.total_bytes):
                return self._pack_capped(layout, buffer_io, start_pos, object_id)
            entry = self._pack_entry(layout)
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(self.device))
            self.pack_stream.wait_event(ready)
            start_event = torch.cuda.Event(enable_timing=True)
            mutate_event = torch.cuda.Event(enable_timing=True)
            done_event = torch.cuda.Event(enable_timing=True)
            total = layout.total_bytes
            if total == 0:
                start_event.record(self.pack_stream)
                mutate_event.record(self.pack_stream)
                done_event.record(self.pack_stream)
                return PackTicket(self, entry, start_event, mutate_event, done_event, 0)
            if self.mode == "direct":
                start_event.record(self.pack_stream)
                base = buffer_io.device_address(start_pos)
                entry.plan.launch(base, total, self.pack_stream.cuda_stream, self.host_ctas)
                mutate_event.record(self.pack_stream)
                done_event.record(self.pack_stream)
            else:
                # the region may hold an older image: the kernel is ordered after the transfer out of it
                image, offset = self._reserve_image(total, self.pack_stream)
                start_event.record(self.pack_stream)
                entry.plan.launch(image.data_ptr(), total, self.pack_stream.cuda_stream)
                mutate_event.record(self.pack_stream)
                if self._is_registered(buffer_io):
                    # page-locked destination: one asynchronous copy-engine transfer
                    self.copy_stream.wait_event(mutate_event)
                    _native.check(
                        _native.lib().mlf_memcpy_async(
                            ctypes.c_void_p(buffer_io.host_address(start_pos)),
                            ctypes.c_void_p(image.data_ptr()),
                            total,
                            _native.MLF_COPY_D2H,
                            ctypes.c_void_p(self.copy_stream.cuda_stream),
                        )
                    )
                    done_event.record(self.copy_stream)
                else:
                    # pageable destination (a standalone object file): drain through the page-locked
                    # bounce ring, several CPU threads wide. This part blocks the caller.
                    mutate_event.synchronize()
                    _native.check(
                        _native.lib().mlf_bounce_copy(
                            ctypes.c_void_p(image.data_ptr()),
                            ctypes.c_void_p(buffer_io.host_address(start_pos)),
                            total,
                            0,
                            self.host_threads,
                        )
                    )
                    done_event.record(self.pack_stream)
                resident_id = str(object_id) if object_id is not None and start_pos == 0 else None
                self._images.append(_Image(offset, total, done_event, resident_id, mutate_event, start_event))
            if object_id is not None:
                self._drains[str(object_id)] = done_event
                self._drains.move_to_end(str(object_id))
                while len(self._drains) > 64:
                    self._drains.popitem(last=False)
            entry.last_kernel = mutate_event
            self.last_ticket = PackTicket(self, entry, start_event, mutate_event, done_event, total)
            return self.last_ticket

    def pack(self, layout: ObjectLayout, buffer_io, start_pos: int = 0, object_id: Optional[str] = None) -> None:
        self.pack_async(layout, buffer_io, start_pos, object_id).wait()

    def resident_image(self, object_id: str, nbytes: int) -> Optional["_ResidentLease"]:
        """Lease on the HBM image of ``object_id``'s data section, if a staged save left one of
        exactly ``nbytes`` that has not been reused since. While the lease is held no save or restore
        can reuse the arena."""
        with self._lock:
            for image in reversed(self._images):
                if image.object_id == str(object_id) and image.nbytes == nbytes:
                    return _ResidentLease(self, image)
        return None

    def wait_object_on_host(self, object_id: str) -> None:
        """Blocks until every save of ``object_id`` that this engine still knows of has reached the
        object's host mapping. Callers that read the mapping while a save may still be draining
        (replication started right after the pack kernel) call this first."""
        with self._lock:
            event = self._drains.get(str(object_id))
        if event is not None:
            event.synchronize()

    def held_device_bytes(self) -> int:
        """HBM this engine holds beyond the caller's tensors: the image arena."""
        with self._lock:
            return 0 if self._arena is None else int(self._arena.numel())

    def _fill_image(self, image: torch.Tensor, buffer_io, lo: int, nbytes: int, stream: "torch.cuda.Stream") -> None:
        """Brings data-section bytes ``[lo, lo + nbytes)`` of ``buffer_io`` into ``image``. Asynchronous on
        ``stream`` for a page-locked mapping, blocking (CPU threads feeding the bounce ring) otherwise."""
        if self._is_registered(buffer_io):
            _native.check(
                _native.lib().mlf_memcpy_async(
                    ctypes.c_void_p(image.data_ptr()),
                    ctypes.c_void_p(buffer_io.host_address(lo)),
                    nbytes,
                    _native.MLF_COPY_H2D,
                    ctypes.c_void_p(stream.cuda_stream),
                )
            )
            return
        # read-only object mappings cannot be page-locked: feed HBM through the bounce ring,
        # reading the file descriptor so that the mapping's pages are never faulted in
        stream.synchronize()
        reader = getattr(getattr(buffer_io, "buffer_obj", None), "read_to_device", None)
        if reader is not None:
            from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE

            self.last_lock_lane_bytes = reader(
                METADATA_SIZE + lo, image.data_ptr(), nbytes, self.restore_threads, self.restore_lock_run_mib
            ) or 0
        else:
            _native.check(
                _native.lib().mlf_bounce_copy(
                    ctypes.c_void_p(image.data_ptr()),
                    ctypes.c_void_p(buffer_io.host_address(lo)),
                    nbytes,
                    1,
                    self.restore_threads,
                )
            )

    def _unpack_capped(self, prepared, buffer_io) -> None:
        _unpack_capped_impl(self, prepared, buffer_io)

    def object_read(self, buffer_io, lo: int, hi: int) -> "_ObjectRead":
        """Context manager that starts moving data-section bytes ``[lo, hi)`` of ``buffer_io`` into HBM
        at once, on a helper thread, so that the caller can parse headers and plan the restore while
        the bytes travel. Pass the object to ``unpack(..., prefetched=...)`` inside the ``with`` block.
        The engine is reserved for the calling thread until the block ends."""
        return _ObjectRead(self, buffer_io, lo, hi)

    def unpack(
        self,
        reads: Sequence[Tuple[torch.Tensor, int, Sequence[int], Sequence[int]]],
        buffer_io,
        prefetched: Optional["_ObjectRead"] = None,
    ) -> None:
        """Scatters stored tensors (or sub-blocks) from ``buffer_io`` into target tensors.

        Each read is ``(target, image_off, stored_shape, storage_offsets)``: ``image_off`` is the
        data-section offset of the stored tensor's first payload byte, ``stored_shape`` its shape as
        saved, ``storage_offsets`` where the wanted block starts in it; the block's extent is
        ``target.shape``. Targets may be strided; host targets are filled through a device
        temporary. ``prefetched`` is an ``object_read`` of the same buffer that is already bringing
        the bytes into HBM. Returns when all targets hold their data.
        """
        reads = [r for r in reads if r[0].numel() > 0]
        if not reads:
            return
        with self._lock, torch.cuda.device(self.device):
            self._bind()
            lo = None
            hi = 0
            prepared = []
            for target, image_off, stored_shape, storage_offsets in reads:
                esize = target.element_size()
                istr = c_strides(stored_shape)
                first = image_off + sum(int(o) * s for o, s in zip(storage_offsets, istr)) * esize
                span = sum((int(n) - 1) * s for n, s in zip(target.shape, istr)) + 1
                lo = first if lo is None else min(lo, first)
                hi = max(hi, first + span * esize)
                prepared.append((target, first, istr))
            lo -= lo % 16  # keep image offsets congruent mod 16 between the mapping and the HBM copy
            if self._capped(hi - lo) and not (prefetched is not None and prefetched.covers(buffer_io, lo, hi)):
                self._unpack_capped(prepared, buffer_io)
                return
            use_prefetch = prefetched is not None and prefetched.covers(buffer_io, lo, hi)
            if use_prefetch:
                lo, hi = prefetched.lo, prefetched.hi
            elif self._active_read is not None:
                self._active_read.wait()  # its image is about to be given up
                self._active_read = None
            # the plan (tables uploaded once) is built before the bytes have arrived
            descs = (_native.CopyDesc * len(prepared))()
            host_targets = []
            for k, (target, first, istr) in enumerate(prepared):
                dev_target = target
                if target.device.type != "cuda":
                    dev_target = torch.empty(target.shape, dtype=target.dtype, device=self.device)
                    host_targets.append((target, dev_target))
                elif target.device != self.device:
                    raise ValueError(f"target lives on {target.device}, engine on {self.device}")
                fill_desc(descs[k], dev_target.data_ptr(), first - lo, dev_target.element_size(), dev_target.shape, dev_target.stride(), istr)
            plan = _Plan(descs, len(prepared), _native.MLF_UNPACK)
            stream = self.pack_stream
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(self.device))
            stream.wait_event(ready)
            if use_prefetch:
                image = prefetched.image
                fill_ms = prefetched.wait()
            else:
                image = self.staging(hi - lo)
                t_begin = torch.cuda.Event(enable_timing=True)
                t_copied = torch.cuda.Event(enable_timing=True)
                t_begin.record(stream)
                self._fill_image(image, buffer_io, lo, hi - lo, stream)
                t_copied.record(stream)
                fill_ms = None
            t_launch = torch.cuda.Event(enable_timing=True)
            t_launch.record(stream)
            plan.launch(image.data_ptr(), hi - lo, stream.cuda_stream)
            done = torch.cuda.Event(enable_timing=True)
            done.record(stream)
            done.synchronize()
            plan.status()
            if fill_ms is None:
                fill_ms = t_begin.elapsed_time(t_copied)
            self.last_unpack_ms = (fill_ms, t_launch.elapsed_time(done))
            for target, dev_target in host_targets:
                target.copy_(dev_target)
            # later work on the caller's stream must see the restored values
            torch.cuda.current_stream(self.device).wait_event(done)


def _unpack_capped_impl(engine: "CudaCopyEngine", prepared, buffer_io) -> None:
    """Restore through the bounded arena: the reads are grouped, in image order, into pieces that fit
    half the arena; each piece is brought into its half and scattered by a launch of its own while
    the next piece travels into the other half."""
    spans = []
    for target, first, istr in prepared:
        span = sum((int(n) - 1) * s for n, s in zip(target.shape, istr)) + 1
        spans.append((first, first + span * target.element_size(), target, istr))
    spans.sort(key=lambda x: x[0])
    limit = max(engine.arena_limit // 2, 4096)
    slot_bytes = max([limit] + [hi - (lo - lo % 16) for lo, hi, _, _ in spans])
    pieces, current, p_lo, p_hi = [], [], None, None
    for lo, hi, target, istr in spans:
        if current and max(hi, p_hi) - p_lo > slot_bytes:
            pieces.append((p_lo, p_hi, current))
            current, p_lo, p_hi = [], None, None
        if p_lo is None:
            p_lo, p_hi = lo - lo % 16, hi
        p_hi = max(p_hi, hi)
        current.append((target, lo, istr))
    if current:
        pieces.append((p_lo, p_hi, current))
    slot_bytes = (slot_bytes + engine._ARENA_ALIGN - 1) // engine._ARENA_ALIGN * engine._ARENA_ALIGN
    stream = engine.pack_stream
    ready = torch.cuda.Event()
    ready.record(torch.cuda.current_stream(engine.device))
    stream.wait_event(ready)
    engine._claim_whole_arena(2 * slot_bytes, stream)
    for event in engine._slot_free:  # halves of an earlier piecewise save
        if event is not None:
            event.synchronize()
    engine._slot_free = [None, None]
    host_targets, plans = [], []
    scattered = [None, None]
    fill_ms = kernel_ms = 0.0
    timers = []
    for k, (p_lo, p_hi, group) in enumerate(pieces):
        descs = (_native.CopyDesc * len(group))()
        for j, (target, first, istr) in enumerate(group):
            dev_target = target
            if target.device.type != "cuda":
                dev_target = torch.empty(target.shape, dtype=target.dtype, device=engine.device)
                host_targets.append((target, dev_target))
            elif target.device != engine.device:
                raise ValueError(f"target lives on {target.device}, engine on {engine.device}")
            fill_desc(descs[j], dev_target.data_ptr(), first - p_lo, dev_target.element_size(), dev_target.shape, dev_target.stride(), istr)
        plan = _Plan(descs, len(group), _native.MLF_UNPACK)
        plans.append(plan)
        half = k % 2
        slot = engine._arena[half * slot_bytes : half * slot_bytes + (p_hi - p_lo)]
        if scattered[half] is not None:
            scattered[half].synchronize()  # the bounce ring writes the half outside any stream
        t0, t1, t2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        t0.record(stream)
        engine._fill_image(slot, buffer_io, p_lo, p_hi - p_lo, stream)
        t1.record(stream)
        plan.launch(slot.data_ptr(), p_hi - p_lo, stream.cuda_stream)
        t2.record(stream)
        scattered[half] = t2
        timers.append((t0, t1, t2))
    stream.synchronize()
    for plan in plans:
        plan.status()
    for t0, t1, t2 in timers:
        fill_ms += t0.elapsed_time(t1)
        kernel_ms += t1.elapsed_time(t2)
    engine.last_unpack_ms = (fill_ms, kernel_ms)
    for target, dev_target in host_targets:
        target.copy_(dev_target)
    done = torch.cuda.Event()
    done.record(stream)
    torch.cuda.current_stream(engine.device).wait_event(done)


class _ObjectRead:
    """An object's bytes on their way into the engine's HBM arena (see ``CudaCopyEngine.object_read``)."""

    def __init__(self, engine: CudaCopyEngine, buffer_io, lo: int, hi: int):
        self._engine = engine
        self._buffer_io = buffer_io
        self.lo = lo - lo % 16
        self.hi = hi
        self.image: Optional[torch.Tensor] = None
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self._ms = 0.0
        self._events = None
        self._entered = False

    def covers(self, buffer_io, lo: int, hi: int) -> bool:
        return self.image is not None and buffer_io is self._buffer_io and self.lo <= lo and hi <= self.hi

    def __enter__(self) -> "_ObjectRead":
        engine = self._engine
        engine._lock.acquire()
        self._entered = True
        try:
            if self.hi <= self.lo or engine._capped(self.hi - self.lo):
                return self  # nothing to fetch ahead, or the restore goes through the bounded arena piece by piece
            with torch.cuda.device(engine.device):
                engine._bind()
                if engine._active_read is not None:
                    engine._active_read.wait()
                self.image = engine.staging(self.hi - self.lo)
                stream = engine.pack_stream
                if engine._is_registered(self._buffer_io):
                    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    begin.record(stream)
                    engine._fill_image(self.image, self._buffer_io, self.lo, self.hi - self.lo, stream)
                    end.record(stream)
                    self._events = (begin, end)
                else:
                    stream.synchronize()
                    self._events = None
                    self._thread = threading.Thread(target=self._run, name="mlf-object-read", daemon=True)
                    self._thread.start()
            engine._active_read = self
            return self
        except BaseException:
            self._entered = False
            engine._lock.release()
            raise

    def _run(self) -> None:
        import time

        engine = self._engine
        started = time.perf_counter()
        try:
            with torch.cuda.device(engine.device):
                engine._bind()
                engine._fill_image(self.image, self._buffer_io, self.lo, self.hi - self.lo, engine.pack_stream)
        except BaseException as e:  # surfaces in wait()
            self._error = e
        self._ms = (time.perf_counter() - started) * 1e3

    def wait(self) -> float:
        """Blocks until the bytes are in HBM (or queued ahead of later work on the engine's stream);
        returns the milliseconds the transfer took."""
        if self._thread is not None:
            self._thread.join()
            self._thread = None
            if self._error is not None:
                raise self._error
        elif self._events is not None:
            self._events[1].synchronize()
            self._ms = self._events[0].elapsed_time(self._events[1])
            self._events = None
        return self._ms

    def __exit__(self, *exc) -> None:
        engine = self._engine
        try:
            if self._thread is not None:
                self._thread.join()
                self._thread = None
            if engine._active_read is self:
                engine._active_read = None
        finally:
            if self._entered:
                self._entered = False
                engine._lock.release()


class _ResidentLease:
    """Context manager yielding the device address of a resident object image (see ``resident_image``).

    Entering waits for the pack kernel that writes the image, not for the transfer that drains it to
    the host: the image is complete from the "safe to mutate" moment on, so a replication hop can
    run over NVLink while the copy engine is still moving the same bytes over PCIe."""

    def __init__(self, engine: CudaCopyEngine, image: _Image):
        self._engine = engine
        self._image = image

    @property
    def start_event(self):
        """CUDA event recorded right before the pack kernel of this image (None if unknown)."""
        return self._image.start

    def __enter__(self) -> int:
        engine = self._engine
        engine._lock.acquire()
        if not any(held is self._image for held in engine._images) or self._image.object_id is None:
            engine._lock.release()
            raise RuntimeError("the resident image was overwritten before it could be leased")
        (self._image.ready or self._image.done).synchronize()
        return engine._arena.data_ptr() + self._image.offset

    def __exit__(self, *exc) -> None:
        self._engine._lock.release()


class _HostBytesView:
    """Adapter that lets ``CudaCopyEngine.unpack`` read a payload held in a ``bytes`` object."""

    def __init__(self, data: bytes):
        self._keep = (ctypes.c_char * max(len(data), 1)).from_buffer_copy(data or b"\0")
        self._addr = ctypes.addressof(self._keep)

    def host_address(self, pos: int = 0) -> int:
        return self._addr + pos


def unpack_payload_bytes(engine: CudaCopyEngine, payload: bytes, dtype: torch.dtype, stored_shape, storage_offsets, lengths) -> torch.Tensor:
    """The sub-block ``[storage_offsets, storage_offsets + lengths)`` of a stored tensor whose raw
    C-order bytes are ``payload``, as a new host tensor (scattered by the unpack kernel)."""
    out = torch.empty(tuple(lengths), dtype=dtype, device=engine.device)
    engine.unpack([(out, 0, tuple(stored_shape), tuple(storage_offsets))], _HostBytesView(payload))
    return out.cpu()


_default_engine: Optional[CudaCopyEngine] = None
_default_engine_lock = threading.Lock()


def default_engine() -> CudaCopyEngine:
    """Process-wide engine on the current CUDA device, created on first use."""
    global _default_engine
    with _default_engine_lock:
        if _default_engine is None:
            _default_engine = CudaCopyEngine()
        return _default_engine


def peek_default_engine() -> Optional[CudaCopyEngine]:
    """The process-wide engine if one exists already (never creates one)."""
    return _default_engine


def set_default_engine(engine: Optional[CudaCopyEngine]) -> None:
    """Makes ``engine`` the process-wide engine (for callers that configure their own)."""
    global _default_engine
    with _default_engine_lock:
        _default_engine = engine


def resident_image(object_id: str, nbytes: int) -> Optional[_ResidentLease]:
    """``CudaCopyEngine.resident_image`` of the process-wide engine, or None if there is no engine yet."""
    engine = _default_engine
    return None if engine is None else engine.resident_image(object_id, nbytes)


def wait_object_on_host(object_id: str) -> None:
    """``CudaCopyEngine.wait_object_on_host`` of the process-wide engine (no-op without one)."""
    engine = _default_engine
    if engine is not None:
        engine.wait_object_on_host(object_id)
