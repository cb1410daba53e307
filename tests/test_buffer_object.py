"""BufferObject / BufferIO semantics on the host (no GPU needed): same contract as the reference's
buffer tests (create / overwrite / read-only open / resize / truncating close / cursor arithmetic)."""

import io
import os
import struct

import pytest

from ml_flashpoint.checkpoint_object_manager.buffer_io import BufferIO
from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE, BufferMetadataType
from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject


def test_create_maps_a_zero_filled_file_and_creates_parents(tmp_path):
    path = str(tmp_path / "a" / "b" / "obj.distcp")
    buf = BufferObject(path, 8192)
    assert os.path.getsize(path) == 8192
    assert buf.get_id() == path and buf.get_capacity() == 8192
    assert not buf.closed and not buf.is_readonly and buf.get_data_ptr() != 0
    view = memoryview(buf)
    assert view.format == "B" and view.ndim == 1 and len(view) == 8192 and not view.readonly
    assert bytes(view[:64]) == bytes(64)
    view[10:14] = b"abcd"
    buf.close()
    assert buf.closed and buf.get_capacity() == 0
    with open(path, "rb") as f:
        assert f.read()[10:14] == b"abcd"
    buf.close()  # idempotent
    with pytest.raises(RuntimeError):
        buf.get_data_ptr()
    with pytest.raises(BufferError) as closed_view:  # as the reference's binding: BufferError caused by a RuntimeError
        memoryview(buf)
    assert isinstance(closed_view.value.__cause__, RuntimeError)


def test_create_refuses_existing_file_unless_overwrite(tmp_path):
    path = str(tmp_path / "obj")
    BufferObject(path, 4096).close()
    with pytest.raises(RuntimeError, match="exists"):
        BufferObject(path, 4096)
    again = BufferObject(path, 100, overwrite=True)  # truncates and resizes
    assert again.get_capacity() == 100
    again.close()
    with pytest.raises(RuntimeError):
        BufferObject(str(tmp_path / "zero"), 0)


def test_read_only_open(tmp_path):
    path = str(tmp_path / "obj")
    w = BufferObject(path, 5000)
    memoryview(w)[0:3] = b"xyz"
    w.close(truncate_size=4500)
    assert os.path.getsize(path) == 4500
    r = BufferObject(path)
    assert r.is_readonly and r.get_capacity() == 4500
    view = memoryview(r)
    assert view.readonly and bytes(view[:3]) == b"xyz"
    with pytest.raises(TypeError):
        view[0] = 1
    with pytest.raises(RuntimeError):
        r.resize(8000)
    r.close(truncate_size=10)  # ignored for read-only mappings
    assert os.path.getsize(path) == 4500
    with pytest.raises(RuntimeError):
        BufferObject(str(tmp_path / "missing"))
    open(tmp_path / "empty", "wb").close()
    with pytest.raises(RuntimeError):
        BufferObject(str(tmp_path / "empty"))
    with pytest.raises(RuntimeError):
        BufferObject(str(tmp_path))  # a directory


def test_resize_keeps_contents(tmp_path):
    path = str(tmp_path / "obj")
    buf = BufferObject(path, 4096)
    memoryview(buf)[0:5] = b"hello"
    buf.resize(1 << 20)
    assert buf.get_capacity() == 1 << 20 and os.path.getsize(path) == 1 << 20
    assert bytes(memoryview(buf)[:5]) == b"hello"
    buf.resize(4100)
    assert bytes(memoryview(buf)[:5]) == b"hello" and os.path.getsize(path) == 4100
    buf.close()
    with pytest.raises(RuntimeError):
        buf.resize(8192)


def _writer(tmp_path, capacity=METADATA_SIZE + 1000, name="obj"):
    return BufferIO(BufferObject(str(tmp_path / name), capacity, overwrite=True))


def test_bufferio_needs_room_for_the_metadata_block(tmp_path):
    with pytest.raises(ValueError):
        BufferIO(BufferObject(str(tmp_path / "small"), 100))
    closed = BufferObject(str(tmp_path / "c"), METADATA_SIZE)
    closed.close()
    with pytest.raises(ValueError):
        BufferIO(closed)


def test_bufferio_cursor_write_read_seek(tmp_path):
    bio = _writer(tmp_path)
    assert bio.tell() == 0 and bio.write(b"") == 0
    assert bio.write(b"0123456789") == 10 and bio.tell() == 10
    assert bio.read() == b""  # cursor sits at the high-water mark
    assert bio.seek(2) == 2 and bio.read(3) == b"234" and bio.tell() == 5
    assert bio.seek(-2, io.SEEK_END) == 8 and bio.read(100) == b"89"
    assert bio.seek(-4, io.SEEK_CUR) == 6
    target = bytearray(3)
    assert bio.readinto(target) == 3 and bytes(target) == b"678"
    with pytest.raises(TypeError):
        bio.readinto(b"abc")
    with pytest.raises(ValueError):
        bio.seek(-1)
    with pytest.raises(ValueError):
        bio.seek(0, 9)
    # overwriting earlier bytes does not move the high-water mark back
    bio.seek(0)
    bio.write(b"AB")
    assert bio._metadata.len_written_data == 10
    bio.seek(0)
    assert bio.read() == b"AB23456789"
    bio.flush()


def test_bufferio_capacity_and_slices(tmp_path):
    bio = _writer(tmp_path, METADATA_SIZE + 16)
    piece = bio.next_buffer_slice(8)
    assert len(piece) == 8 and not piece.readonly and bio.tell() == 8
    piece[:] = b"abcdefgh"
    with pytest.raises(ValueError):
        bio.next_buffer_slice(-1)
    with pytest.raises(ValueError, match="exceeds buffer capacity"):
        bio.next_buffer_slice(9)
    with pytest.raises(ValueError, match="exceeds buffer capacity"):
        bio.write(b"x" * 9)
    bio.write(b"12345678")
    assert bio.host_address(3) == bio.buffer_obj.get_data_ptr() + METADATA_SIZE + 3
    assert bio.capacity == METADATA_SIZE + 16


def test_bufferio_close_truncates_and_metadata_block_is_the_documented_layout(tmp_path):
    path = tmp_path / "obj"
    bio = _writer(tmp_path, METADATA_SIZE + 1000)
    bio.set_format_signature(b"MLF_TENS")
    with pytest.raises(ValueError):
        bio.set_format_signature(b"123456789")
    bio.write(b"payload!")
    with bio:
        pass
    assert bio.closed
    with pytest.raises(ValueError):
        bio.tell()
    raw = path.read_bytes()
    assert len(raw) == METADATA_SIZE + 8
    assert raw[:16] == struct.pack("<Q", 8) + b"MLF_TENS"
    assert raw[16:METADATA_SIZE] == bytes(METADATA_SIZE - 16)
    assert raw[METADATA_SIZE:] == b"payload!"

    ro = BufferIO(BufferObject(str(path)))
    assert ro.is_readonly and ro.format_signature == b"MLF_TENS" and ro.read() == b"payload!"
    for op in (lambda: ro.write(b"x"), lambda: ro.next_buffer_slice(1), lambda: ro.set_format_signature(b"x"), lambda: ro.resize(8192)):
        with pytest.raises(TypeError):
            op()
    ro.close()
    assert os.path.getsize(path) == METADATA_SIZE + 8

    keep = _writer(tmp_path, METADATA_SIZE + 100, name="keep")
    keep.write(b"abc")
    keep.close(truncate=False)
    assert os.path.getsize(tmp_path / "keep") == METADATA_SIZE + 100


def test_bufferio_resize_preserves_cursor_and_data(tmp_path):
    bio = _writer(tmp_path, METADATA_SIZE + 10)
    bio.write(b"0123456789")
    bio.resize(METADATA_SIZE + 100)
    assert bio.tell() == 10 and bio._metadata.len_written_data == 10
    bio.write(b"x" * 90)
    with pytest.raises(ValueError):
        bio.resize(100)
    bio.seek(0)
    assert bio.read(12) == b"0123456789xx"
    bio.close()


def test_metadata_struct_size():
    import ctypes

    assert ctypes.sizeof(BufferMetadataType) == METADATA_SIZE
    assert BufferMetadataType.format_signature.offset == 8
