"""``AutoResume`` that prefers the newest complete ML Flashpoint checkpoint.

Same class as the reference's adapter/nemo/auto_resume.py:35-93: the first lookup asks the
checkpoint loader for the latest checkpoint every rank can load (fetching missing objects from
peers on the way); if there is none, NeMo's own resume logic runs. Megatron's stub
``metadata.json`` is recreated when it was lost with a node.
"""

import json
import logging
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import torch.distributed as dist
from nemo.lightning import AutoResume
from nemo.lightning import io as nemo_lightning_io

from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
from ml_flashpoint.core.checkpoint_loader import MLFlashpointCheckpointLoader
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.core.utils import log_execution_time

_LOGGER = get_logger(__name__)


@dataclass(kw_only=True)
class MLFlashpointAutoResume(AutoResume):
    """``checkpoint_base_container`` and ``checkpoint_loader`` are required; every ``AutoResume``
    field (``resume_if_exists=True`` and ``resume_ignore_no_checkpoint=True`` are advisable) may be
    given as well."""

    checkpoint_base_container: CheckpointContainerId
    checkpoint_loader: MLFlashpointCheckpointLoader
    _checkpoint_path_cache: Optional[Path] = field(default=None, init=False)
    _flashpoint_resolved: bool = field(default=False, init=False)

    @log_execution_time(logger=_LOGGER, name="MLFlashpointAutoResume._find_trainer_ckpt_path", level=logging.INFO)
    def _find_trainer_ckpt_path(self) -> Optional[Path]:
        if self._checkpoint_path_cache is not None:
            return self._checkpoint_path_cache
        if not self._flashpoint_resolved:
            self._flashpoint_resolved = True  # the search is collective: run it once
            found = self.checkpoint_loader.get_latest_complete_checkpoint(self.checkpoint_base_container)
            _LOGGER.info("Latest complete checkpoint: '%s'", found)
            if found is not None:
                if dist.get_node_local_rank() == 0:
                    stub = os.path.join(found.data, "metadata.json")
                    if not os.path.exists(stub):
                        with open(stub, "w") as f:
                            json.dump({"sharded_backend": ""}, f)
                self._checkpoint_path_cache = Path(found.data)
                return self._checkpoint_path_cache
        return super()._find_trainer_ckpt_path()

    def get_trainer_ckpt_path(self, model: Optional[nemo_lightning_io.ConnectorMixin] = None) -> Optional[Path]:
        return self._find_trainer_ckpt_path()
