"""Per-tensor header of the ``MLF_TENS`` object format.

Wire form (reference: core/tensor_header.py:30-56): a little-endian ``u32`` length followed by the
pickle of a ``TensorHeader`` instance. The pickle embeds this module's import path and the class
name, and the attribute order ``dtype``, ``shape``; all three are therefore part of the format and
must not change, or stored objects stop being byte-identical (and readable) across builds.
"""

import pickle
import struct
from typing import Tuple

import torch

_LENGTH = struct.Struct("<I")


class TensorHeader:
    """dtype and shape of a stored tensor; the payload that follows is its C-order bytes."""

    def __init__(self, dtype: torch.dtype, shape: torch.Size):
        # attribute insertion order is the pickled order
        self.dtype = dtype
        self.shape = shape

    def __eq__(self, other) -> bool:
        return isinstance(other, TensorHeader) and self.dtype == other.dtype and self.shape == other.shape

    def __repr__(self) -> str:
        return f"TensorHeader(dtype={self.dtype!r}, shape={self.shape!r})"

    def to_bytes(self) -> bytes:
        body = pickle.dumps(self)
        return _LENGTH.pack(len(body)) + body

    @classmethod
    def from_bytes(cls, buffer: bytes) -> Tuple["TensorHeader", int]:
        """Parses a header at the start of ``buffer``; returns it with the byte count consumed."""
        (body_len,) = _LENGTH.unpack_from(buffer, 0)
        end = _LENGTH.size + body_len
        return pickle.loads(bytes(buffer[_LENGTH.size : end])), end
