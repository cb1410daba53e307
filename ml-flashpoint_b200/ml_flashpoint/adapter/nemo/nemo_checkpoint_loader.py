"""Loader that also recovers NeMo's ``context/`` directory from peers.

Same class as the reference's adapter/nemo/nemo_checkpoint_loader.py:30-101: with
``recover_context`` every file under ``<checkpoint>/context`` is advertised as an extra local object
and counted as needed by each node's first rank, so that the retrieval plan fetches it.
"""

import os
from pathlib import Path
from typing import Callable, List, Set

from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId, CheckpointObjectId
from ml_flashpoint.core.checkpoint_loader import DefaultMLFlashpointCheckpointLoader
from ml_flashpoint.replication.replication_manager import ReplicationManager


class NeMoMLFlashpointCheckpointLoader(DefaultMLFlashpointCheckpointLoader):
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
        recover_context: bool = False,
        copy_engine=None,
    ):
        super().__init__(
            checkpoint_object_manager,
            replication_manager,
            global_rank_getter=global_rank_getter,
            local_rank_getter=local_rank_getter,
            broadcast_object_list_func=broadcast_object_list_func,
            all_gather_object_func=all_gather_object_func,
            world_size_getter=world_size_getter,
            copy_engine=copy_engine,
        )
        self._recover_context = recover_context

    def _get_extra_local_objects(self, container_path: Path) -> List[CheckpointObjectId]:
        if not self._recover_context:
            return []
        context = container_path / "context"
        if not context.is_dir():
            return []
        return [CheckpointObjectId(str(Path(root) / name)) for root, _, names in os.walk(context) for name in names]

    def _get_extra_needed_objects(
        self,
        checkpoint: CheckpointContainerId,
        available_objects_by_rank: dict[int, List[CheckpointObjectId]],
    ) -> Set[str]:
        if not self._recover_context:
            return set()
        context = Path(checkpoint.data) / "context"
        wanted = set()
        for objects in available_objects_by_rank.values():
            for obj in objects:
                if Path(str(obj.data)).is_relative_to(context):
                    wanted.add(str(obj.data))
        return wanted
