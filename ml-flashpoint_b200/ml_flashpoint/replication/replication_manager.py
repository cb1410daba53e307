"""Replication of written checkpoint objects to peer ranks, and retrieval from them.

Same surface as the reference's replication/replication_manager.py (``ReplicationStrategy`` :44-77,
``PairwiseReplicationStrategy`` :80-145, ``ReplicationRetryConfig`` :148-160, ``ReplicationManager``
:175-545): a strategy maps a rank to the service addresses of its replica holders, the manager
issues one ``async_put`` per destination and closes the object's buffer when all have finished,
``sync_bulk_retrieve`` pulls objects back during recovery.

Added: ``RingReplicationStrategy`` for ranks that share one NVLink domain (a single 8-GPU box, or
several trays behind NVSwitch): rank ``r`` replicates to ``(r + 1) mod world``. The pairwise strategy
pairs *nodes* and switches itself off on a single node, which leaves nothing to replicate to there.
"""

import abc
import concurrent.futures
import logging
import socket
import threading
import time
from pathlib import Path
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from ml_flashpoint.checkpoint_object_manager.buffer_io import BufferIO
from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core import utils
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time
from ml_flashpoint.replication.transfer_service import transfer_service_ext

_LOGGER = get_logger(__name__)


class ReplicationStrategy:
    """Decides where a rank's objects are replicated to."""

    def __init__(self, replication_service_addresses: List[str]):
        # service address of every rank, indexed by global rank
        self._replication_service_addresses = replication_service_addresses

    @abc.abstractmethod
    def get_destination_addresses(self, global_rank: int) -> List[str]:
        """Service addresses ("<host>:<port>") that receive ``global_rank``'s objects."""
        raise NotImplementedError()

    def get_replication_service_addresses(self) -> List[str]:
        return self._replication_service_addresses


class PairwiseReplicationStrategy(ReplicationStrategy):
    """Nodes are paired (0<>1, 2<>3, ...); a rank replicates to the same local rank on the paired node.

    Needs an even node count, except that a single node is accepted and simply replicates nothing.
    """

    def __init__(self, replication_service_addresses: List[str], processes_per_node: int) -> None:
        super().__init__(replication_service_addresses)
        if not self._replication_service_addresses:
            raise ValueError("The replication_service_addresses cannot be empty.")
        self._processes_per_node = processes_per_node
        self._world_size = len(self._replication_service_addresses)
        if self._world_size % self._processes_per_node != 0:
            raise ValueError(
                f"World size ({self._world_size}) must be divisible by processes per node ({self._processes_per_node})."
            )
        self._num_nodes = utils.get_num_of_nodes()
        if self._num_nodes > 1 and self._num_nodes % 2 != 0:
            raise ValueError(f"The total number of nodes ({self._num_nodes}) must be even for pairwise replication.")
        self._disable_replication = self._num_nodes == 1
        if self._num_nodes != self._world_size // self._processes_per_node:
            raise ValueError(
                f"The total number of nodes ({self._num_nodes}) must be equal to the world size "
                f"({self._world_size}) divided by the processes per node ({self._processes_per_node})."
            )

    def get_destination_addresses(self, global_rank: int) -> List[str]:
        if self._disable_replication:
            return []
        if not 0 <= global_rank < self._world_size:
            raise ValueError(f"global_rank {global_rank} is out of valid range [0, {self._world_size - 1}].")
        node, local = divmod(global_rank, self._processes_per_node)
        partner = (node ^ 1) * self._processes_per_node + local
        return [self._replication_service_addresses[partner]]


class RingReplicationStrategy(ReplicationStrategy):
    """Rank ``r`` replicates to ``(r + offset) mod world``. Every rank sends one stream and receives one,
    which NVSwitch carries at full per-GPU bandwidth whatever the permutation."""

    def __init__(self, replication_service_addresses: List[str], offset: int = 1) -> None:
        super().__init__(replication_service_addresses)
        if not self._replication_service_addresses:
            raise ValueError("The replication_service_addresses cannot be empty.")
        self._world_size = len(self._replication_service_addresses)
        self._offset = offset % self._world_size if self._world_size else 0

    def get_destination_addresses(self, global_rank: int) -> List[str]:
        if not 0 <= global_rank < self._world_size:
            raise ValueError(f"global_rank {global_rank} is out of valid range [0, {self._world_size - 1}].")
        if self._offset == 0:
            return []  # a ring of one has no partner
        return [self._replication_service_addresses[(global_rank + self._offset) % self._world_size]]


class ReplicationRetryConfig:
    def __init__(self, max_retries: int = 3, timeout_seconds: float = 30.0):
        self._max_retries = max_retries
        self._timeout_seconds = timeout_seconds

    def get_timeout(self) -> float:
        return self._timeout_seconds

    def get_retries(self) -> int:
        return self._max_retries


def get_default_retry_config() -> ReplicationRetryConfig:
    return ReplicationRetryConfig()


class ReplicationManager:
    """Owns the transfer service and turns "replicate this buffer" into transfers."""

    @log_execution_time(_LOGGER, "ReplicationManager.initialize")
    def initialize(
        self,
        checkpoint_object_manager: CheckpointObjectManager,
        listen_port: int = 0,
        retry_config: ReplicationRetryConfig = get_default_retry_config(),
        replication_transfer_service: Optional[transfer_service_ext.TransferService] = None,
        repl_strategy: Optional[ReplicationStrategy] = None,
    ) -> None:
        """Collective: starts (or adopts) the transfer service, all-gathers the service addresses
        unless a strategy that already knows them is supplied."""
        self._checkpoint_object_manager = checkpoint_object_manager
        self._listen_port = listen_port
        self._retry_config = retry_config
        self._repl_strategy = repl_strategy
        self._transfer_service = replication_transfer_service
        self._initialize_address()

        if self._transfer_service is None:
            self._transfer_service = transfer_service_ext.TransferService()
            bound = self._transfer_service.initialize(listen_port, global_rank=dist.get_rank())
            if bound <= 0:
                raise RuntimeError("Failed to initialize TransferService")
            self._listen_port = bound

        if self._repl_strategy is None:
            self._gather_replication_service_addresses()
            self._repl_strategy = PairwiseReplicationStrategy(
                self._replication_service_addr_global_view, torch.cuda.device_count()
            )
        elif hasattr(self._repl_strategy, "get_replication_service_addresses"):
            self._replication_service_addr_global_view = self._repl_strategy.get_replication_service_addresses()

    @log_execution_time(_LOGGER, "ReplicationManager.async_replicate")
    def async_replicate(self, buffer_io: BufferIO) -> list[concurrent.futures.Future]:
        """Sends the whole object (metadata block included) to every destination of this rank.

        Non-blocking. The buffer is closed once all transfers have ended, or at once if there is
        no destination.
        """
        if self._repl_strategy is None:
            _LOGGER.error("No replication strategy set. Cannot replicate.")
            return []
        if self._transfer_service is None:
            _LOGGER.error("TransferService is not initialized. Cannot replicate.")
            return []
        obj_id = str(buffer_io.buffer_obj.get_id())
        destinations = self._repl_strategy.get_destination_addresses(dist.get_rank())
        if not destinations:
            _LOGGER.warning("No destinations found for '%s'. Replication skipped.", obj_id)
            try:
                self._checkpoint_object_manager.close_buffer(buffer_io, skip_close_if_symlink=True)
            except Exception:
                _LOGGER.exception("Failed to close buffer '%s'", obj_id)
            return []
        started = time.perf_counter()
        futures = [
            self._transfer_service.async_put(
                buffer_io.buffer_obj.get_data_ptr(), buffer_io.buffer_obj.get_capacity(), address, obj_id
            )
            for address in destinations
        ]
        self._add_aggregate_callback(futures, lambda done: self._final_replication_callback(buffer_io, done, started))
        return futures

    @staticmethod
    @log_execution_time(_LOGGER, "ReplicationManager._add_aggregate_callback")
    def _add_aggregate_callback(
        futures: List[concurrent.futures.Future],
        final_callback: Callable[[List[concurrent.futures.Future]], None],
    ) -> None:
        """Calls ``final_callback(futures)`` exactly once, after the last of ``futures`` completes."""
        if not futures:
            final_callback([])
            return
        lock = threading.Lock()
        outstanding = [len(futures)]

        def _one_done(_future: concurrent.futures.Future) -> None:
            with lock:
                outstanding[0] -= 1
                if outstanding[0] == 0:
                    final_callback(futures)

        for f in futures:
            f.add_done_callback(_one_done)

    @log_execution_time(_LOGGER, "ReplicationManager._final_replication_callback")
    def _final_replication_callback(
        self, buffer_io: BufferIO, completed_futures: List[concurrent.futures.Future], repl_start_time: float
    ) -> None:
        name = buffer_io.buffer_obj.get_id()
        errors = []
        for f in completed_futures:
            exc = f.exception()
            if exc:
                errors.append(exc)
                _LOGGER.error("Buffer object '%s' replication failed with exception: '%s'", name, exc)
                continue
            result = f.result()
            if not result.success:
                errors.append(RuntimeError(f"Buffer object {name} replication failed: {result.error_message}"))
                _LOGGER.error("%s", errors[-1])
        _LOGGER.info("Replication of '%s' took %.4fs", Path(name).name, time.perf_counter() - repl_start_time)
        with log_execution_time(_LOGGER, "_final_replication_callback__close_buffer", level=logging.DEBUG):
            self._checkpoint_object_manager.close_buffer(buffer_io, skip_close_if_symlink=True)
        if errors:
            _LOGGER.error("%d replications failed: '%s'", len(errors), errors)
        else:
            _LOGGER.info("All replications completed successfully.")

    def _async_retrieve(
        self,
        source_address: str,
        object_id_to_retrieve: CheckpointObjectId,
        retrieved_object_id: CheckpointObjectId,
    ) -> concurrent.futures.Future:
        if self._transfer_service is None:
            failed: concurrent.futures.Future = concurrent.futures.Future()
            failed.set_exception(RuntimeError("TransferService is not initialized."))
            return failed
        return self._transfer_service.async_get(str(object_id_to_retrieve), source_address, str(retrieved_object_id))

    @log_execution_time(_LOGGER, "ReplicationManager.sync_bulk_retrieve")
    def sync_bulk_retrieve(
        self,
        source_global_rank: int,
        object_ids_to_retrieve: List[CheckpointObjectId],
        container_ids_to_retrieve: List[CheckpointContainerId],
        retrieved_object_ids: List[CheckpointObjectId] | None = None,
        retrieved_container_ids: List[CheckpointContainerId] | None = None,
    ) -> bool:
        """Blocking fetch of objects held by ``source_global_rank``; True if every one arrived
        within the retry config's timeout. Containers are accepted but not fetched (as upstream)."""
        if getattr(self, "_retry_config", None) is None:
            _LOGGER.error("ReplicationManager is not initialized. Cannot retrieve.")
            return False
        if retrieved_object_ids and len(retrieved_object_ids) != len(object_ids_to_retrieve):
            _LOGGER.error("Retrieved_object_ids must be empty or the same length as object_ids_to_retrieve.")
            return False
        if retrieved_container_ids and len(retrieved_container_ids) != len(container_ids_to_retrieve):
            _LOGGER.error("Retrieved_container_ids must be empty or the same length as container_ids_to_retrieve.")
        addresses = self._replication_service_addr_global_view
        if not 0 <= source_global_rank < len(addresses):
            _LOGGER.error("Invalid source_global_rank: %d", source_global_rank)
            return False
        local_names = retrieved_object_ids if retrieved_object_ids else object_ids_to_retrieve
        futures = [
            self._async_retrieve(addresses[source_global_rank], remote, local_names[i])
            for i, remote in enumerate(object_ids_to_retrieve)
        ]
        done, pending = concurrent.futures.wait(futures, timeout=self._retry_config.get_timeout())
        if pending:
            _LOGGER.error("Timed out waiting for %d retrievals.", len(pending))
            return False
        ok = True
        for f in done:
            try:
                result = f.result()
                if not result.success:
                    _LOGGER.error("Retrieval failed: %s", result.error_message)
                    ok = False
            except Exception:
                _LOGGER.exception("Retrieval failed with exception")
                ok = False
        return ok

    @log_execution_time(_LOGGER, "ReplicationManager.shutdown")
    def shutdown(self):
        if getattr(self, "_transfer_service", None):
            self._transfer_service.shutdown()

    def _initialize_address(self):
        try:
            self._hostname = socket.gethostbyname(socket.gethostname())
        except Exception:
            _LOGGER.exception("Failed to initialize replication address")
            self._hostname = "Error"

    @log_execution_time(_LOGGER, "ReplicationManager._gather_replication_service_addresses")
    def _gather_replication_service_addresses(self):
        mine = f"{self._hostname}:{self._listen_port}"
        self._replication_service_addr_global_view = [None] * dist.get_world_size()
        try:
            dist.all_gather_object(self._replication_service_addr_global_view, mine)
        except Exception as e:
            self._replication_service_addr_global_view = []
            raise RuntimeError(f"Failed to gather replication service addresses from all ranks. Error: {e}")
