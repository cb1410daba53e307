"""Checkpoint restore pipeline.

Public surface and semantics follow the reference's core/checkpoint_loader.py
(``MLFlashpointCheckpointLoader`` :57-118, ``DefaultMLFlashpointCheckpointLoader`` :121-712):
metadata read, per-object reads with N-d narrowing, newest-complete-checkpoint search across ranks,
retrieval plan and peer retrieval.

The data path differs. The reference materialises every stored tensor as ``bytes``, wraps it with
``frombuffer``, narrows and ``copy_``s on the host (:177-219, :331-336). Here all tensor reads of one
object become ONE scatter-unpack kernel launch: the needed byte range is brought into HBM by a
copy engine and the kernel writes every target (any strides, any sub-block) directly
(``gpu_engine.CudaCopyEngine.unpack``). Results are bit-identical.
"""

import abc
import contextlib
import fcntl
import io
import logging
import os
import pickle
import re
import struct
from collections import defaultdict
from pathlib import Path
from typing import IO, Callable, List, Optional, Set, Tuple, TypeVar, cast

import torch
from torch.distributed._shard._utils import narrow_tensor_by_index
from torch.distributed.checkpoint import Metadata
from torch.distributed.checkpoint.filesystem import _StorageInfo
from torch.distributed.checkpoint.planner import LoadItemType, LoadPlanner, ReadItem
from torch.distributed.checkpoint.utils import _create_file_view

from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core import gpu_engine
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.defaults import (
    COMMON_STATE_FNAME,
    DIRTY_MARKER_SUFFIX,
    GLOBAL_RANK_PATTERN,
    CheckpointFormat,
    default_metadata_object_name,
)
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import get_num_of_nodes, log_execution_time
from ml_flashpoint.replication.replication_manager import ReplicationManager

M = TypeVar("M")

_LOGGER = get_logger(__name__)

_MAX_HEADER_BYTES = 1024 * 1024  # a longer "header" means the item is not in the MLF_TENS format


class MLFlashpointCheckpointLoader(abc.ABC):
    @abc.abstractmethod
    def read_metadata(
        self,
        checkpoint_id: CheckpointContainerId,
        object_name: str = default_metadata_object_name(),
    ) -> Metadata:
        """Unpickles ``{checkpoint_id}/{object_name}``."""

    @abc.abstractmethod
    def read_data(
        self,
        checkpoint_object_id: CheckpointObjectId,
        read_items: List[ReadItem],
        planner: LoadPlanner,
        storage_data: dict[int, _StorageInfo],
    ) -> None:
        """Loads ``read_items`` from one object into the planner's targets."""

    @abc.abstractmethod
    def get_latest_complete_checkpoint(
        self, checkpoint_base_container: CheckpointContainerId
    ) -> Optional[CheckpointContainerId]:
        """Newest ``step-<N>_ckpt`` under the base that every rank can fully load, or None."""


class DefaultMLFlashpointCheckpointLoader(MLFlashpointCheckpointLoader):
    def __init__(
        self,
        checkpoint_object_manager: CheckpointObjectManager,
        replication_manager: ReplicationManager,
        *,
        global_rank_getter: Callable[[], int],
        local_rank_getter: Callable[[], int],
        broadcast_object_list_func: Callable[..., None],
        all_gather_object_func: Callable[..., None],
        world_size_getter: Callable[[], int],
        copy_engine: Optional["gpu_engine.CudaCopyEngine"] = None,
        replica_namespace=None,
    ):
        """``copy_engine`` moves the bytes (default: the process-wide CUDA engine, created on first
        use). ``replica_namespace`` (a ``transfer_service_ext.ReplicaNamespace``) is for ranks whose
        replication partners share their filesystem: the replicas this rank holds for others are then
        reported during recovery as objects it can serve. The other arguments are as in the reference
        (:126-160)."""
        self._replica_namespace = replica_namespace
        self._checkpoint_object_manager = checkpoint_object_manager
        self._replication_manager = replication_manager
        self._global_rank_getter = global_rank_getter
        self._local_rank_getter = local_rank_getter
        self._broadcast_object_list_func = broadcast_object_list_func
        self._all_gather_object_func = all_gather_object_func
        self._world_size_getter = world_size_getter
        self._copy_engine = copy_engine
        # container -> {object path -> ranks that hold it}, filled by get_checkpoint_objects_by_rank
        self._available_objects_cache: dict[CheckpointContainerId, dict[str, List[int]]] = {}

    def _engine(self) -> "gpu_engine.CudaCopyEngine":
        if self._copy_engine is None:
            self._copy_engine = gpu_engine.default_engine()
        return self._copy_engine

    # ------------------------------------------------------------------ metadata
    @log_execution_time(logger=_LOGGER, name="read_metadata")
    def read_metadata(
        self,
        checkpoint_id: CheckpointContainerId,
        object_name: str = default_metadata_object_name(),
    ) -> Metadata:
        path = Path(checkpoint_id.data) / object_name
        try:
            with open(path, "rb") as f:
                return pickle.load(f)
        except Exception:
            _LOGGER.exception("Error reading metadata from '%s'", path)
            raise

    # ------------------------------------------------------------------ data
    @staticmethod
    def _parse_stored_header(stream, offset: int, length: int):
        """Header of the item stored at ``[offset, offset + length)``.

        Returns ``(dtype, shape, header_bytes)`` or None if the bytes there are not an MLF_TENS item.
        """
        stream.seek(offset)
        prefix = stream.read(min(4, length))
        if len(prefix) != 4:
            return None
        (header_len,) = struct.unpack("<I", prefix)
        if header_len >= _MAX_HEADER_BYTES or 4 + header_len > length:
            return None
        try:
            header = pickle.loads(stream.read(header_len))
            return header.dtype, header.shape, 4 + header_len
        except Exception:
            _LOGGER.exception("Failed to parse tensor header")
            raise

    def read_tensor(self, buffer_slice: IO[bytes], req: ReadItem, use_optimized_loader: bool = False) -> torch.Tensor:
        """One stored tensor from a file view, narrowed to the request, as a host tensor.

        ``read_data`` does not come through here for ``MLF_TENS`` objects (it scatters all items of an
        object with one kernel launch); this per-item form is kept for callers of the reference API
        and for objects in the ``TORCH___`` format, whose items are opaque ``torch.save`` streams.
        With ``use_optimized_loader`` an ``MLF_TENS`` item is narrowed by the unpack kernel; anything
        that does not parse as such an item falls back to ``torch.load``.
        """
        start = buffer_slice.tell()
        if use_optimized_loader:
            prefix = buffer_slice.read(4)
            if len(prefix) == 4:
                (header_len,) = struct.unpack("<I", prefix)
                if header_len < _MAX_HEADER_BYTES:
                    try:
                        header = pickle.loads(buffer_slice.read(header_len))
                        payload = buffer_slice.read()
                    except Exception:
                        _LOGGER.exception("Failed to parse tensor header")
                        raise
                    return gpu_engine.unpack_payload_bytes(
                        self._engine(), payload, header.dtype, header.shape, req.storage_offsets, req.lengths
                    )
        buffer_slice.seek(start)
        tensor = cast(torch.Tensor, torch.load(cast(IO[bytes], buffer_slice), map_location="cpu", weights_only=True))
        return narrow_tensor_by_index(tensor, req.storage_offsets, req.lengths)

    @log_execution_time(logger=_LOGGER, name="read_data", level=logging.INFO)
    def read_data(
        self,
        checkpoint_object_id: CheckpointObjectId,
        read_items: List[ReadItem],
        planner: LoadPlanner,
        storage_data: dict[int, _StorageInfo],
    ) -> None:
        """A locally missing object is first fetched from a peer that holds a replica."""
        if not self._try_retrieve_object_if_missing(checkpoint_object_id):
            error_msg = f"Checkpoint object '{checkpoint_object_id.data}' does not exist on any node in the cluster"
            _LOGGER.error(error_msg)
            raise FileNotFoundError(error_msg)

        with contextlib.ExitStack() as scope:
            stream = scope.enter_context(self._checkpoint_object_manager.get_buffer(checkpoint_object_id))
            optimized = stream.format_signature == CheckpointFormat.MLF_FORMAT
            scatter = []  # (target, payload offset, stored shape, storage offsets)
            commits = []  # (req, target)
            converts = []  # (target, temporary in the stored dtype)
            # The bytes start moving into HBM now; headers are parsed and the plan is built meanwhile.
            prefetched = None
            tensor_items = [storage_data[req.storage_index] for req in read_items if req.type != LoadItemType.BYTE_IO]
            start_read = getattr(self._engine(), "object_read", None) if optimized and tensor_items else None
            if start_read is not None:
                lo = min(md.offset for md in tensor_items)
                hi = max(md.offset + md.length for md in tensor_items)
                prefetched = scope.enter_context(start_read(stream, lo, hi))
            for req in read_items:
                item_md = storage_data[req.storage_index]
                if req.type == LoadItemType.BYTE_IO:
                    stream.seek(item_md.offset)
                    planner.load_bytes(req, io.BytesIO(stream.read(item_md.length)))
                    continue
                target = planner.resolve_tensor(req).detach()
                header = self._parse_stored_header(stream, item_md.offset, item_md.length) if optimized else None
                if header is None:
                    view = cast(IO[bytes], _create_file_view(stream, item_md.offset, item_md.length))
                    tensor = self.read_tensor(view, req)
                    assert target.size() == tensor.size(), (
                        f"req {req.storage_index} mismatch sizes {target.size()} vs {tensor.size()}"
                    )
                    target.copy_(tensor)
                    planner.commit_tensor(req, target)
                    continue
                dtype, shape, header_bytes = header
                assert tuple(target.size()) == tuple(req.lengths), (
                    f"req {req.storage_index} mismatch sizes {target.size()} vs {torch.Size(req.lengths)}"
                )
                for off, n, full in zip(req.storage_offsets, req.lengths, shape):
                    if off < 0 or off + n > full:
                        raise IndexError(f"req {req.storage_index}: block [{off}, {off + n}) outside stored extent {full}")
                landing = target
                if target.dtype != dtype:
                    # the reference ends in ``target.copy_(tensor)`` (:331-336), which converts: the block
                    # is unpacked in its stored dtype into a device temporary and converted from there
                    landing = torch.empty(tuple(req.lengths), dtype=dtype, device=getattr(self._engine(), "device", target.device))
                    converts.append((target, landing))
                scatter.append((landing, item_md.offset + header_bytes, tuple(shape), tuple(req.storage_offsets)))
                commits.append((req, target))
            if scatter:
                if prefetched is not None:
                    self._engine().unpack(scatter, stream, prefetched=prefetched)
                else:
                    self._engine().unpack(scatter, stream)
            for target, landing in converts:
                target.copy_(landing)
            for req, target in commits:
                planner.commit_tensor(req, target)

    def _try_retrieve_object_if_missing(self, checkpoint_object_id: CheckpointObjectId) -> bool:
        """True if the object is (now) present locally. Needs the location cache filled by
        ``get_latest_complete_checkpoint`` to know which rank holds a replica."""
        path = checkpoint_object_id.data
        if os.path.exists(path):
            return True
        if not self._replication_manager:
            _LOGGER.error("ReplicationManager is not initialized.")
            return False
        holders = self._available_objects_cache.get(checkpoint_object_id.get_parent(), {}).get(path)
        if not holders:
            return False
        source_rank = holders[0]
        _LOGGER.debug("Object '%s' missing locally but found on rank %s. Attempting retrieval.", path, source_rank)
        try:
            with open(f"{path}.lock", "w") as lock_file:
                fcntl.flock(lock_file, fcntl.LOCK_EX)
                try:
                    if os.path.exists(path):  # another local rank fetched it while we waited
                        return True
                    ok = self._replication_manager.sync_bulk_retrieve(
                        source_global_rank=source_rank,
                        object_ids_to_retrieve=[checkpoint_object_id],
                        container_ids_to_retrieve=[],
                    )
                    if not ok:
                        _LOGGER.error("Failed to retrieve '%s'", path)
                    return bool(ok)
                finally:
                    fcntl.flock(lock_file, fcntl.LOCK_UN)
        except Exception:
            _LOGGER.exception("Error during retrieval/locking for '%s'", path)
            return False

    # ------------------------------------------------------------------ discovery
    @log_execution_time(logger=_LOGGER, name="get_latest_complete_checkpoint", level=logging.INFO)
    def get_latest_complete_checkpoint(
        self, checkpoint_base_container: CheckpointContainerId
    ) -> Optional[CheckpointContainerId]:
        """Walks candidates newest first. For each: gather who holds which objects; the lowest rank
        holding ``.metadata`` computes a retrieval plan and broadcasts it; None = not recoverable,
        empty = complete everywhere, otherwise every rank fetches its share and all must succeed."""
        rank = self._global_rank_getter()
        candidates = self.get_candidate_checkpoints(checkpoint_base_container)
        if not candidates:
            _LOGGER.warning("No candidate checkpoints found.")
            return None
        md_name = default_metadata_object_name()
        for checkpoint in candidates:
            by_rank = self.get_checkpoint_objects_by_rank(checkpoint)
            planner_rank = next(
                (r for r in sorted(by_rank) if any(os.path.basename(o.data) == md_name for o in by_rank[r])), None
            )
            if planner_rank is None:
                _LOGGER.warning("Rank %s: No metadata found for '%s'", rank, checkpoint)
                continue
            box = [self._compute_retrieval_plan(checkpoint, by_rank) if rank == planner_rank else None]
            self._broadcast_object_list_func(box, src=planner_rank)
            plan = box[0]
            if plan is None:
                _LOGGER.warning("Rank %s: retrieval plan is None for '%s'. Not viable.", rank, checkpoint)
                continue
            if not plan:
                return checkpoint
            if self.retrieve_checkpoint(plan):
                return checkpoint
            _LOGGER.warning("Failed to retrieve all necessary objects for checkpoint '%s'.", checkpoint)
        _LOGGER.warning("Rank %s: No complete checkpoint found.", rank)
        return None

    def _compute_retrieval_plan(
        self,
        checkpoint: CheckpointContainerId,
        available_objects_by_rank: dict[int, List[CheckpointObjectId]],
    ) -> Optional[dict[int, List[Tuple[int, str]]]]:
        """``{rank: [(source rank, object path)]}`` of what each rank must fetch; ``{}`` if nothing;
        None if some needed object exists nowhere.

        A rank needs the objects whose name carries its ``src<rank>`` tag; each node's first rank
        also needs ``common.pt``, ``.metadata`` and whatever ``_get_extra_needed_objects`` adds.
        """
        try:
            metadata = self.read_metadata(checkpoint)
        except Exception:
            _LOGGER.warning("Failed to read metadata for '%s'", checkpoint)
            return None
        if metadata.storage_data is None:
            return None

        needed: dict[int, set[str]] = defaultdict(set)
        for info in metadata.storage_data.values():
            tagged = GLOBAL_RANK_PATTERN.search(info.relative_path)
            if tagged:
                needed[int(tagged.group(1))].add(str(CheckpointObjectId.from_container(checkpoint, info.relative_path)))

        per_node = {
            str(CheckpointObjectId.from_container(checkpoint, COMMON_STATE_FNAME)),
            str(CheckpointObjectId.from_container(checkpoint, default_metadata_object_name())),
        }
        per_node.update(self._get_extra_needed_objects(checkpoint, available_objects_by_rank))
        world = self._world_size_getter()
        ranks_per_node = world // get_num_of_nodes()
        for r in range(0, world, ranks_per_node):
            needed[r].update(per_node)

        holders = defaultdict(list)
        for r, objs in available_objects_by_rank.items():
            for o in objs:
                holders[str(o)].append(r)

        plan: dict[int, List[Tuple[int, str]]] = {}
        for r, wanted in needed.items():
            have = {str(o) for o in available_objects_by_rank.get(r, [])}
            missing = wanted - have
            if not missing:
                continue
            plan[r] = []
            for obj in missing:
                if not holders.get(obj):
                    _LOGGER.warning("Object '%s' is missing globally (needed by rank %s)", obj, r)
                    return None
                plan[r].append((holders[obj][0], obj))
        return plan

    @log_execution_time(logger=_LOGGER, name="get_candidate_checkpoints")
    def get_candidate_checkpoints(
        self, checkpoint_base_container: CheckpointContainerId
    ) -> List[CheckpointContainerId]:
        """Containers without an unfinished marker that every reporting rank sees, newest first."""
        base = Path(checkpoint_base_container.data)
        local: List[str] = []
        if base.is_dir():
            step_dir = re.compile(r"(step-\d+_ckpt)")
            seen, dirty = set(), set()
            for entry in os.listdir(base):
                hit = step_dir.match(entry)
                if not hit:
                    continue
                if entry.endswith(DIRTY_MARKER_SUFFIX):
                    dirty.add(hit.group(1))
                else:
                    seen.add(entry)
            local = [str(base / name) for name in seen - dirty]
        gathered = [None] * self._world_size_getter()
        self._all_gather_object_func(gathered, local)
        reported = [set(paths) for paths in gathered if paths]
        if not reported:
            return []
        common = set.intersection(*reported)
        return sorted(
            (CheckpointContainerId(p) for p in common),
            key=lambda cid: CheckpointContainerId.parse_version_container_step(os.path.basename(cid.data)) or -1,
            reverse=True,
        )

    @log_execution_time(logger=_LOGGER, name="get_checkpoint_objects_by_rank")
    def get_checkpoint_objects_by_rank(
        self, checkpoint_container_id: CheckpointContainerId
    ) -> dict[int, List[CheckpointObjectId]]:
        """Directory listing of the container on every rank; also refreshes the location cache."""
        here = Path(checkpoint_container_id.data)
        local: List[CheckpointObjectId] = []
        if here.is_dir():
            local = [CheckpointObjectId.from_container(checkpoint_container_id, e) for e in os.listdir(here)]
            local.extend(self._get_extra_local_objects(here))
        gathered = [None] * self._world_size_getter()
        self._all_gather_object_func(gathered, local)
        result: dict[int, List[CheckpointObjectId]] = {}
        locations = defaultdict(list)
        for r, objs in enumerate(gathered or []):
            result[r] = objs or []
            for o in result[r]:
                locations[o.data].append(r)
        self._available_objects_cache[checkpoint_container_id] = locations
        return result

    @log_execution_time(logger=_LOGGER, name="retrieve_checkpoint")
    def retrieve_checkpoint(self, retrieval_plan: dict[int, List[Tuple[int, str]]]) -> bool:
        """Fetches this rank's share of ``retrieval_plan``; True only if every rank succeeded."""
        rank = self._global_rank_getter()
        ok = True
        by_source: dict[int, List[CheckpointObjectId]] = defaultdict(list)
        for source, path in (retrieval_plan or {}).get(rank, []) or []:
            by_source[source].append(CheckpointObjectId(path))
        for source, objects in by_source.items():
            if not self._replication_manager.sync_bulk_retrieve(
                source_global_rank=source, object_ids_to_retrieve=objects, container_ids_to_retrieve=[]
            ):
                _LOGGER.error("Failed to retrieve objects from rank %s", source)
                ok = False
        verdicts = [None] * self._world_size_getter()
        self._all_gather_object_func(verdicts, ok)
        return all(verdicts)

    def _get_extra_local_objects(self, container_path: Path) -> List[CheckpointObjectId]:
        """Hook: further objects this rank can serve (e.g. framework context files). Here: the replicas
        it holds for other ranks, under their original paths, when a replica namespace is configured."""
        namespace = getattr(self, "_replica_namespace", None)
        if namespace is None:
            return []
        return [CheckpointObjectId(path) for path in namespace.held_objects(str(container_path))]

    def _get_extra_needed_objects(
        self,
        checkpoint: CheckpointContainerId,
        available_objects_by_rank: dict[int, List[CheckpointObjectId]],
    ) -> Set[str]:
        """Hook: further objects each node's first rank needs. Pair with ``_get_extra_local_objects``."""
        return set()
