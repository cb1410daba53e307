"""Checkpoint save pipeline.

Public surface and semantics follow the reference's core/checkpoint_saver.py (``ObjectWriteBucket``
:50-63, ``WriteItemResolver`` :66-103, ``MLFlashpointCheckpointSaver`` :106-286,
``DefaultMLFlashpointCheckpointSaver`` :289-800): dirty marker, bucketing through torch's
``_split_by_size_and_type``, one object per bucket named ``{prefix}_{n}_src{rank}.distcp``, atomic
``.metadata``, finalize with barrier and removal of older steps.

What differs is who moves the bytes. The reference copies tensor by tensor on the host
(``dest.copy_(tensor)``, :797-800) after staging every tensor to pageable CPU memory. Here a
bucket's whole data section is planned up front (``gpu_engine.plan_object_layout``) and written by
ONE gather-pack kernel launch reading the tensors where they live in HBM
(``gpu_engine.CudaCopyEngine``); the resulting object files are byte-identical.
"""

import abc
import concurrent.futures
import dataclasses
import io
import logging
import os
import pickle
import queue
import subprocess
import threading
from typing import Callable, Optional, Protocol, Union

import torch
from torch.distributed.checkpoint import metadata as torchdistmeta
from torch.distributed.checkpoint.filesystem import _split_by_size_and_type, _StorageInfo
from torch.distributed.checkpoint.planner import WriteItem, WriteItemType
from torch.distributed.checkpoint.storage import WriteResult

from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core import gpu_engine
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.defaults import DIRTY_MARKER_SUFFIX, CheckpointFormat, default_metadata_object_name
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import get_accelerator_count, log_execution_time  # noqa: F401  (patch point kept)
from ml_flashpoint.replication.replication_manager import ReplicationManager

DEFAULT_INITIAL_BUFFER_SIZE_BYTES = 16 * 1024 * 1024 * 1024
"""Size of a standalone (non-pooled) object file before it is trimmed on close: 16 GiB."""

_DEFAULT_OBJ_NAME_SUFFIX = ".distcp"

_LOGGER = get_logger(__name__)


@dataclasses.dataclass
class ObjectWriteBucket:
    """Everything that goes into one object (one file): resolved tensors and byte items."""

    object_id: CheckpointObjectId
    object_name: str
    bytesio_data: list[tuple[WriteItem, io.BytesIO]]
    tensor_data: list[tuple[WriteItem, torch.Tensor]]


class PendingSave:
    """A save whose bytes are still moving (returned by ``write_data_async``).

    ``wait_safe_to_mutate`` returns once every source tensor has been read: the training loop may
    then overwrite parameters and optimizer state while the host transfer continues.
    ``safe_to_mutate_event`` is the CUDA event for the same moment, for
    ``stream.wait_event`` without blocking the host. ``result`` blocks until every object is
    complete in its buffer, closes the buffers and returns the write results.

    With ``replicate_after_write`` the push of an object to its replication partners is queued as
    soon as its pack kernel is, when the object's file already has its final size (pool buffers):
    the copy over NVLink reads the finished HBM image while the copy engine still drains the same
    image to the host. Objects in standalone files are replicated from ``result``, after the close
    that trims them. ``replication_futures`` collects the transfer futures either way.
    """

    def __init__(self, saver: "DefaultMLFlashpointCheckpointSaver", replicate_after_write: bool):
        self._saver = saver
        self._replicate = replicate_after_write
        self._parts: list = []  # (bucket, writer, records, ticket)
        self._results: Optional[list[WriteResult]] = None
        self._replicated_early: set = set()  # object names whose replication started with the pack kernel
        self.replication_futures: list = []  # transfer futures of replications started so far

    def _add(self, bucket, writer, records, ticket) -> None:
        self._parts.append((bucket, writer, records, ticket))

    def _note_early_replication(self, bucket, futures) -> None:
        self._replicated_early.add(bucket.object_name)
        self.replication_futures.extend(futures or [])

    @property
    def safe_to_mutate_event(self):
        return self._parts[-1][3].mutate_event if self._parts else None

    def wait_safe_to_mutate(self) -> None:
        for _, _, _, ticket in self._parts:
            ticket.mutate_event.synchronize()

    def done(self) -> bool:
        return all(ticket.done_event.query() for _, _, _, ticket in self._parts)

    def result(self) -> list[WriteResult]:
        if self._results is not None:
            return self._results
        results: list[WriteResult] = []
        first_error: Optional[BaseException] = None
        for bucket, writer, records, ticket in self._parts:
            try:
                ticket.wait()
                results.extend(self._saver._to_write_results(bucket.object_name, records))
            except BaseException as e:  # keep closing the remaining buffers
                first_error = first_error or e
            finally:
                writer.close()
        if first_error is not None:
            raise first_error
        if self._replicate:
            for bucket, _, _, _ in self._parts:
                if bucket.object_name not in self._replicated_early:
                    self.replication_futures.extend(self._saver.async_replicate_object(bucket.object_id) or [])
        self._results = results
        return results


class WriteItemResolver(Protocol):
    """Anything with ``resolve_data(write_item) -> Tensor | BytesIO``; a DCP ``SavePlanner`` qualifies."""

    @abc.abstractmethod
    def resolve_data(self, write_item: WriteItem) -> Union[torch.Tensor, io.BytesIO]:
        pass


class MLFlashpointCheckpointSaver(abc.ABC):
    """Stages of a save, in call order: ``initialize_checkpoint``, (``prepare_write_data``,)
    ``stage_data``, ``write_data``, ``async_replicate_object`` per object unless ``write_data``
    replicated already, ``write_metadata``, ``finalize_checkpoint``."""

    @abc.abstractmethod
    def initialize_checkpoint(self, checkpoint_id: CheckpointContainerId) -> None:
        """Marks ``checkpoint_id`` as in progress. Must precede every other step."""

    @abc.abstractmethod
    def stage_data(self, checkpoint_id: CheckpointContainerId, state_dict: dict, non_blocking: bool = True) -> dict:
        """Returns a state dict that is safe to write from; blocking."""

    @abc.abstractmethod
    def prepare_write_data(
        self,
        checkpoint_id: CheckpointContainerId,
        write_items: list[WriteItem],
        write_item_resolver: WriteItemResolver,
        object_name_prefix: str,
        bucket_count: int,
    ) -> list[ObjectWriteBucket]:
        """Resolves the items and groups them into one bucket per object."""

    @abc.abstractmethod
    def write_data(
        self,
        checkpoint_id: CheckpointContainerId,
        write_buckets: list[ObjectWriteBucket],
        thread_count: int,
        replicate_after_write: bool,
    ) -> list[WriteResult]:
        """Writes every bucket to its object; synchronous."""

    def async_replicate_object(self, object_id: CheckpointObjectId) -> list[concurrent.futures.Future]:
        """Starts replicating one written object; returns the transfer futures."""

    @abc.abstractmethod
    def write_metadata(
        self,
        checkpoint_id: CheckpointContainerId,
        metadata: torchdistmeta.Metadata,
        md_object_name: str = default_metadata_object_name(),
    ):
        """Atomically writes ``metadata`` as ``{checkpoint_id}/{md_object_name}``."""

    @abc.abstractmethod
    def finalize_checkpoint(self, checkpoint_id: CheckpointContainerId) -> Union[subprocess.Popen, None]:
        """Removes the in-progress marker, waits for all ranks, and on local rank 0 starts deleting older steps."""


class DefaultMLFlashpointCheckpointSaver(MLFlashpointCheckpointSaver):
    def __init__(
        self,
        global_rank_getter: Callable[[], int],
        local_rank_getter: Callable[[], int],
        global_barrier_func: Callable[[], None],
        ckpt_obj_manager: CheckpointObjectManager,
        replication_manager: ReplicationManager,
        initial_buffer_size_bytes: int = DEFAULT_INITIAL_BUFFER_SIZE_BYTES,
        use_optimized_save: bool = True,
        copy_engine: Optional["gpu_engine.CudaCopyEngine"] = None,
    ):
        """``copy_engine`` moves the bytes; by default the process-wide CUDA engine is created on
        first use. The other arguments are as in the reference (:290-321)."""
        self._global_rank_getter = global_rank_getter
        self._local_rank_getter = local_rank_getter
        self._barrier_func = global_barrier_func
        self._chkpt_obj_manager = ckpt_obj_manager
        self._replication_manager = replication_manager
        self._initial_buffer_size_bytes = initial_buffer_size_bytes
        self._use_optimized_save = use_optimized_save
        self._copy_engine = copy_engine
        self._layouts: dict = {}  # id(bucket) -> (bucket, layout) planned by _announce_save, consumed by _write_bucket

    # Worker processes get a saver without the replication manager and without CUDA state.
    def __getstate__(self):
        state = self.__dict__.copy()
        state.pop("_replication_manager", None)
        state["_copy_engine"] = None
        state["_layouts"] = {}
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._replication_manager = None

    def _engine(self) -> "gpu_engine.CudaCopyEngine":
        if self._copy_engine is None:
            self._copy_engine = gpu_engine.default_engine()
        return self._copy_engine

    # ------------------------------------------------------------------ init / stage / prepare
    @log_execution_time(logger=_LOGGER, name="initialize_checkpoint")
    def initialize_checkpoint(self, checkpoint_id: CheckpointContainerId) -> None:
        self._create_dirty_checkpoint_marker(checkpoint_id)
        os.makedirs(checkpoint_id.data, exist_ok=True)
        _LOGGER.info("Created checkpoint directory: '%s'", checkpoint_id.data)

    @log_execution_time(logger=_LOGGER, name="stage_data", level=logging.INFO)
    def stage_data(self, checkpoint_id: CheckpointContainerId, state_dict: dict, non_blocking: bool = True) -> dict:
        """Tensors stay where they are: the pack kernel reads them from HBM in ``write_data``.

        Only pending work on the current stream is flushed so that the values are final.
        """
        staged = dict(state_dict)
        if torch.cuda.is_available() and any(isinstance(v, torch.Tensor) and v.is_cuda for v in staged.values()):
            torch.cuda.current_stream().synchronize()
        return staged

    @log_execution_time(logger=_LOGGER, name="prepare_write_data")
    def prepare_write_data(
        self,
        checkpoint_id: CheckpointContainerId,
        write_items: list[WriteItem],
        write_item_resolver: WriteItemResolver,
        object_name_prefix: str,
        bucket_count: int,
    ) -> list[ObjectWriteBucket]:
        bucket_count = max(bucket_count, 1)
        rank = self._global_rank_getter()
        write_buckets: list[ObjectWriteBucket] = []
        for items in _split_by_size_and_type(bucket_count, write_items):
            if not items:
                continue
            blobs = [(wi, write_item_resolver.resolve_data(wi)) for wi in items if wi.type == WriteItemType.BYTE_IO]
            tensors = [
                (wi, write_item_resolver.resolve_data(wi).detach()) for wi in items if wi.type != WriteItemType.BYTE_IO
            ]
            if not blobs and not tensors:
                continue
            # same naming scheme as torch's FileSystemWriter; the index counts non-empty buckets only
            name = f"{object_name_prefix}_{len(write_buckets)}_src{rank}{_DEFAULT_OBJ_NAME_SUFFIX}"
            write_buckets.append(
                ObjectWriteBucket(
                    object_id=CheckpointObjectId.from_container(checkpoint_id, name),
                    object_name=name,
                    bytesio_data=blobs,
                    tensor_data=tensors,
                )
            )
        return write_buckets

    # ------------------------------------------------------------------ write
    @log_execution_time(logger=_LOGGER, name="write_data", level=logging.INFO)
    def write_data(
        self,
        checkpoint_id: CheckpointContainerId,
        write_buckets: list[ObjectWriteBucket],
        replicate_after_write: bool,
        thread_count: int = 1,
    ) -> list[WriteResult]:
        thread_count = max(thread_count, 1)
        self._announce_save(write_buckets)
        pending: queue.Queue = queue.Queue()
        for bucket in write_buckets:
            pending.put(bucket)
        outcomes: queue.Queue = queue.Queue()  # (results | None, exception | None)
        args = (pending, outcomes, replicate_after_write, self._use_optimized_save)
        helpers = [
            threading.Thread(
                target=self._write_to_buffer_from_queue_worker, args=args, name=f"{self.__class__.__name__}-Thread-{i}"
            )
            for i in range(1, thread_count)
        ]
        for t in helpers:
            t.start()
        self._write_to_buffer_from_queue_worker(*args)
        for t in helpers:
            t.join()

        results: list[WriteResult] = []
        errors: list[Exception] = []
        while True:
            try:
                done, err = outcomes.get_nowait()
            except queue.Empty:
                break
            if err:
                errors.append(err)
            elif done:
                results.extend(done)
        if errors:
            _LOGGER.error(
                "'%s' encountered %d error(s) during multi-threaded write (will propagate the first one):\n%s.",
                self.__class__.__name__,
                len(errors),
                errors,
            )
            raise errors[0]
        return results

    @log_execution_time(logger=_LOGGER, name="write_data_async", level=logging.INFO)
    def write_data_async(
        self,
        checkpoint_id: CheckpointContainerId,
        write_buckets: list[ObjectWriteBucket],
        replicate_after_write: bool = False,
    ) -> PendingSave:
        """Starts writing every bucket and returns without waiting for the bytes to land.

        This is the overlapped form of ``write_data``: one pack kernel per bucket is queued on the
        engine's side stream (ordered after the caller's current stream), followed by the transfer
        into the bucket's buffer. The call returns after the launches; see ``PendingSave`` for the
        two completion points. Buffers are acquired here and closed by ``PendingSave.result``.
        """
        pending = PendingSave(self, replicate_after_write)
        self._announce_save(write_buckets)
        for bucket in write_buckets:
            writer = self._chkpt_obj_manager.acquire_buffer(bucket.object_id, self._initial_buffer_size_bytes)
            try:
                records, ticket = self._write_bucket(bucket, writer, self._use_optimized_save, wait=False)
            except BaseException:
                writer.close()
                for _, open_writer, _, open_ticket in pending._parts:
                    try:
                        open_ticket.wait()
                    finally:
                        open_writer.close()
                raise
            pending._add(bucket, writer, records, ticket)
            if replicate_after_write and self._can_replicate_early(writer):
                try:
                    pending._note_early_replication(bucket, self.async_replicate_object(bucket.object_id))
                except Exception:
                    _LOGGER.exception("Could not start replication of '%s' early; it will follow the write", bucket.object_id)
        return pending

    def _can_replicate_early(self, writer) -> bool:
        """True when replication of the object behind ``writer`` may start before its bytes have
        reached the host mapping: the file must already have its final size (a pool buffer sized by
        ``ensure_total_size``), because the receiver is told the object's size up front; a
        replication manager must be present; and this saver's engine must be the process-wide one,
        because that is where the transfer service looks the object up: it then either sends the
        finished HBM image or waits for the drain itself (``wait_object_on_host``). A saver with an
        engine of its own replicates after the write, as before."""
        if self._replication_manager is None or not hasattr(writer, "ensure_total_size"):
            return False
        engine = self._engine()
        return hasattr(engine, "wait_object_on_host") and engine is gpu_engine.peek_default_engine()

    @log_execution_time(logger=_LOGGER, name="_write_to_buffer_from_queue_worker")
    def _write_to_buffer_from_queue_worker(
        self,
        object_write_bucket_queue: queue.Queue,
        results_from_threads: queue.Queue,
        replicate_after_write: bool,
        use_optimized_write: bool,
    ):
        """Drains buckets from the queue; each becomes one object written by one kernel launch."""
        while True:
            try:
                bucket: ObjectWriteBucket = object_write_bucket_queue.get_nowait()
            except queue.Empty:
                return
            try:
                # existing objects are overwritten: a restarted job may rewrite steps it abandoned
                with self._chkpt_obj_manager.acquire_buffer(bucket.object_id, self._initial_buffer_size_bytes) as writer:
                    records, ticket = self._write_bucket(bucket, writer, use_optimized_write, wait=False)
                    early = False
                    if replicate_after_write and self._can_replicate_early(writer):
                        # the NVLink hop reads the HBM image while the copy engine drains it to the host
                        try:
                            self.async_replicate_object(bucket.object_id)
                            early = True
                        except Exception:
                            _LOGGER.exception("Could not start replication of '%s' early", bucket.object_id)
                    results = self._to_write_results(bucket.object_name, records)  # while the bytes move
                    ticket.wait()
                results_from_threads.put((results, None))
                if replicate_after_write and not early:
                    self.async_replicate_object(bucket.object_id)
            except Exception as e:
                _LOGGER.exception("Error in writer thread for object '%s'", bucket.object_id)
                results_from_threads.put((None, e))
            finally:
                object_write_bucket_queue.task_done()

    def _announce_save(self, write_buckets: list[ObjectWriteBucket]) -> None:
        """Plans every bucket's layout once and tells the engine how much HBM the images of this save
        take together, so that no bucket's pack kernel has to wait for another bucket's transfer."""
        self._layouts.clear()  # entries of a save that failed before consuming them would pin its tensors
        if not write_buckets:
            return
        total = 0
        for bucket in write_buckets:
            layout = self._plan_layout(bucket, self._use_optimized_save)
            self._layouts[id(bucket)] = (bucket, layout)
            total += layout.total_bytes
        announce = getattr(self._engine(), "begin_save", None)
        if announce is not None:
            announce(total)

    @staticmethod
    def _plan_layout(bucket: ObjectWriteBucket, use_optimized_write: bool):
        if use_optimized_write:
            return gpu_engine.plan_object_layout(bucket.tensor_data, bucket.bytesio_data, start_offset=0)
        # legacy format: every tensor is a torch.save stream; the streams travel as byte items
        streams = []
        for item, tensor in bucket.tensor_data:
            sink = io.BytesIO()
            torch.save(tensor, sink)
            streams.append((item, sink))
        return gpu_engine.plan_object_layout([], streams + list(bucket.bytesio_data), start_offset=0)

    def _write_bucket(self, bucket: ObjectWriteBucket, writer, use_optimized_write: bool, wait: bool = True):
        writer.set_format_signature(CheckpointFormat.MLF_FORMAT if use_optimized_write else CheckpointFormat.TORCH_SAVE)
        planned = self._layouts.pop(id(bucket), None)
        if planned is not None and planned[0] is bucket and use_optimized_write == self._use_optimized_save:
            layout = planned[1]
        else:
            layout = self._plan_layout(bucket, use_optimized_write)
        start = writer.tell()
        if hasattr(writer, "ensure_total_size"):
            # pooled file: one remap to the exact final size instead of grow-then-trim
            from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE

            writer.ensure_total_size(METADATA_SIZE + start + layout.total_bytes)
        writer.next_buffer_slice(layout.total_bytes)  # claims the bytes; raises if they do not fit
        records = [(r.item, start + r.offset, r.length) for r in layout.records]
        if wait:
            self._engine().pack(layout, writer, start, object_id=str(bucket.object_id))
            return records
        return records, self._engine().pack_async(layout, writer, start, object_id=str(bucket.object_id))

    @staticmethod
    def _to_write_results(object_name: str, records) -> list[WriteResult]:
        return [
            WriteResult(
                index=item.index,
                size_in_bytes=length,
                storage_data=_StorageInfo(relative_path=object_name, offset=offset, length=length),
            )
            for item, offset, length in records
        ]

    def _save_tensor_optimized(self, tensor: torch.Tensor, buffer_io_writer):
        """Appends one tensor (header + C-order bytes, whatever its strides) at the writer's cursor."""
        layout = gpu_engine.plan_object_layout([(None, tensor)], [], start_offset=0)
        start = buffer_io_writer.tell()
        buffer_io_writer.next_buffer_slice(layout.total_bytes)
        self._engine().pack(layout, buffer_io_writer, start)

    # ------------------------------------------------------------------ replicate / metadata / finalize
    @log_execution_time(logger=_LOGGER, name="async_replicate_object")
    def async_replicate_object(self, object_id: CheckpointObjectId) -> list[concurrent.futures.Future]:
        if self._replication_manager is None:
            # savers unpickled in worker processes carry no replication manager
            raise RuntimeError("ReplicationManager is not available (None). Cannot replicate object.")
        return self._replication_manager.async_replicate(self._chkpt_obj_manager.get_buffer(object_id))

    @log_execution_time(logger=_LOGGER, name="write_metadata")
    def write_metadata(
        self,
        checkpoint_id: CheckpointContainerId,
        metadata: torchdistmeta.Metadata,
        md_object_name: str = default_metadata_object_name(),
    ):
        _LOGGER.info("Writing metadata for checkpoint ID: '%s', with object name: '%s'", checkpoint_id, md_object_name)
        final_path = os.path.join(checkpoint_id.data, md_object_name)
        os.makedirs(os.path.dirname(final_path), exist_ok=True)
        scratch = final_path + ".tmp"
        with open(scratch, "wb") as f:
            pickle.dump(metadata, f)
        os.rename(scratch, final_path)  # readers see the whole file or none of it

    @log_execution_time(logger=_LOGGER, name="finalize_checkpoint")
    def finalize_checkpoint(self, checkpoint_id: CheckpointContainerId) -> Union[subprocess.Popen, None]:
        self._remove_dirty_checkpoint_marker(checkpoint_id)
        with log_execution_time(logger=_LOGGER, name="finalize_checkpoint__barrier_func", level=logging.DEBUG):
            self._barrier_func()
        if self._local_rank_getter() == 0:
            return self._remove_older_checkpoints(older_than=checkpoint_id)
        return None

    def _get_dirty_marker_file_path(self, checkpoint_id: CheckpointContainerId):
        if str(checkpoint_id) == "/":
            raise ValueError("CheckpointContainerId cannot be the root path '/'")
        return f"{str(checkpoint_id).rstrip('/')}__{self._local_rank_getter()}__{DIRTY_MARKER_SUFFIX}"

    def _create_dirty_checkpoint_marker(self, checkpoint_id: CheckpointContainerId) -> None:
        marker = self._get_dirty_marker_file_path(checkpoint_id)
        os.makedirs(os.path.dirname(marker), exist_ok=True)
        open(marker, "w").close()
        _LOGGER.info(
            "Created dirty marker file for checkpoint_id '%s' on local rank '%d': '%s'",
            checkpoint_id,
            self._local_rank_getter(),
            marker,
        )

    def _remove_dirty_checkpoint_marker(self, checkpoint_id: CheckpointContainerId) -> None:
        marker = self._get_dirty_marker_file_path(checkpoint_id)
        if not os.path.exists(marker):
            _LOGGER.warning("Dirty marker file path: '%s' does not exist, skipping removal.", marker)
            return
        os.remove(marker)
        _LOGGER.info(
            "Removed dirty marker file for checkpoint_id '%s' on local rank '%d': '%s'",
            checkpoint_id,
            self._local_rank_getter(),
            marker,
        )

    @log_execution_time(logger=_LOGGER, name="_remove_older_checkpoints")
    def _remove_older_checkpoints(self, older_than: CheckpointContainerId) -> Optional[subprocess.Popen]:
        """Starts ``rm -rf`` on every sibling ``step-<N>_ckpt`` directory with a smaller N.

        Runs detached in its own session so that neither the GIL nor a Ctrl-C sent to the job
        interferes with a large deletion. Call once per node.
        """
        parent = os.path.dirname(older_than.data)
        this_step = CheckpointContainerId.parse_version_container_step(os.path.basename(older_than.data))
        if this_step is None:
            _LOGGER.warning(
                "Could not parse step from 'older_than' checkpoint container: '%s'. "
                "Skipping removal of older checkpoints.",
                older_than,
            )
            return None
        doomed = []
        for name in os.listdir(parent):
            step = CheckpointContainerId.parse_version_container_step(name)
            path = os.path.join(parent, name)
            if step is not None and step < this_step and os.path.isdir(path):
                doomed.append(path)
        if not doomed:
            return None
        try:
            return subprocess.Popen(
                ["rm", "-rf"] + doomed, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, start_new_session=True
            )
        except Exception as e:
            _LOGGER.exception("Background deletion of old checkpoints failed: %s", e)
            return None
