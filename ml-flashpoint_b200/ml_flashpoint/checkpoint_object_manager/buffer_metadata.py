"""The 4096-byte metadata block at the start of every checkpoint object.

Layout (reference: checkpoint_object_manager/buffer_metadata.py:18-37), little-endian, packed:
  [0, 8)     u64  number of valid data bytes that follow the block
  [8, 16)    8 bytes format signature (see ``CheckpointFormat``)
  [16, 4096) reserved, zero
Stream positions and storage offsets everywhere else are relative to the end of this block.
"""

import ctypes

METADATA_SIZE = 4096
_SIGNATURE_BYTES = 8


class BufferMetadataType(ctypes.LittleEndianStructure):
    _pack_ = 1
    _fields_ = [
        ("len_written_data", ctypes.c_uint64),
        ("format_signature", ctypes.c_char * _SIGNATURE_BYTES),
        ("reserved", ctypes.c_uint8 * (METADATA_SIZE - ctypes.sizeof(ctypes.c_uint64) - _SIGNATURE_BYTES)),
    ]


assert ctypes.sizeof(BufferMetadataType) == METADATA_SIZE, (
    f"BufferMetadataType size mismatch: Actual {ctypes.sizeof(BufferMetadataType)} != Expected {METADATA_SIZE}"
)


def get_metadata_str(metadata: "BufferMetadataType | None") -> str:
    if metadata is None:
        return "[Metadata: None]"
    return f"Metadata(len_written_data={metadata.len_written_data})"
