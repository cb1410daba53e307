"""Constants of the on-disk checkpoint layout (names mirror the reference's core/defaults.py:18-36)."""

import enum
import re

# `<container>__<local_rank>__unfinished` marks a checkpoint that is still being written.
DIRTY_MARKER_SUFFIX = "unfinished"
# Object names carry the global rank that wrote them: `..._src<rank>.distcp`.
GLOBAL_RANK_PATTERN = re.compile(r"src(\d+)")
# Per-node file with the state shared by all ranks (written by the Megatron path).
COMMON_STATE_FNAME = "common.pt"


class CheckpointFormat(bytes, enum.Enum):
    """8-byte signature at bytes [8, 16) of every object, naming how tensors are serialised."""

    TORCH_SAVE = b"TORCH___"  # one torch.save stream per tensor
    MLF_FORMAT = b"MLF_TENS"  # length-prefixed pickled TensorHeader followed by raw bytes


def default_metadata_object_name() -> str:
    """File name of the pickled DCP ``Metadata`` inside a checkpoint container."""
    return ".metadata"
