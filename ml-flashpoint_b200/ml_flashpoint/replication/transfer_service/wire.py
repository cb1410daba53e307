"""The reference transfer service's TCP wire format.

Every message of the reference's service starts with one fixed-size packed header
(replication/transfer_service/protocol.h:32-72): a one-byte message type, four NUL-terminated
strings in fixed fields and a signed 64-bit object size in host (little-endian) byte order, 2 249
bytes in all. A put is ``header(kPutObj, dest_obj_id, obj_size)`` followed by the object's bytes and
answered by ``header(kAck)`` or ``header(kError)`` on the same connection
(transfer_service.cpp:628-690, 702-780). A get is ``header(kGetObj, task_id, source_obj_id,
dest_obj_id, source_address, dest_address)``, answered at once by an ack or an error; the holder
then opens a connection of its own to ``dest_address`` and pushes the object as
``header(kRespondToGetObj, task_id, ...)`` + bytes, which the requester acknowledges and matches to
its pending get by ``task_id`` (transfer_service.cpp:782-915, 975-1035).

Speaking this format on the TCP path lets ranks running this package replicate to and retrieve from
ranks running the reference's service. ``NATIVE`` is a message type the reference does not define:
it opens this package's own negotiation (NVLink transport between ranks of one host), and a peer
that does not answer it is treated as a reference peer.
"""

from __future__ import annotations

import socket
import struct
from typing import NamedTuple

PUT_OBJ = 1
GET_OBJ = 2
RESPOND_TO_GET_OBJ = 3
ACK = 4
ERROR = 5
NATIVE = 0x42  # outside the reference's enum: its dispatcher ignores the message

_HEADER = struct.Struct("<B1024s1024s64s64s64sq")
HEADER_SIZE = _HEADER.size  # 2249
assert HEADER_SIZE == 1 + 1024 + 1024 + 64 + 64 + 64 + 8

_FIELD_BYTES = {"source_obj_id": 1024, "dest_obj_id": 1024, "source_address": 64, "dest_address": 64, "task_id": 64}


class Header(NamedTuple):
    type: int
    source_obj_id: str = ""
    dest_obj_id: str = ""
    source_address: str = ""
    dest_address: str = ""
    task_id: str = ""
    obj_size: int = 0


def _field(name: str, value: str) -> bytes:
    raw = value.encode()
    if len(raw) >= _FIELD_BYTES[name]:  # the reference's snprintf would cut it short silently
        raise ValueError(f"{name} of {len(raw)} bytes does not fit the {_FIELD_BYTES[name]}-byte wire field")
    return raw  # struct pads with NULs


def pack_header(type: int, *, source_obj_id: str = "", dest_obj_id: str = "", source_address: str = "", dest_address: str = "",
                task_id: str = "", obj_size: int = 0) -> bytes:
    return _HEADER.pack(
        type, _field("source_obj_id", source_obj_id), _field("dest_obj_id", dest_obj_id), _field("source_address", source_address),
        _field("dest_address", dest_address), _field("task_id", task_id), int(obj_size),
    )


def _text(raw: bytes) -> str:
    # up to the first NUL; the last byte counts as one whatever it holds (protocol.h:62-68)
    return raw[:-1].split(b"\0", 1)[0].decode(errors="replace")


def unpack_header(raw: bytes) -> Header:
    type_, src_obj, dst_obj, src_addr, dst_addr, task, size = _HEADER.unpack(raw)
    return Header(type_, _text(src_obj), _text(dst_obj), _text(src_addr), _text(dst_addr), _text(task), size)


def recv_header(sock: socket.socket, allow_eof: bool = False):
    """The next header on the connection; ``None`` when ``allow_eof`` and the peer closed it between
    messages."""
    buf = bytearray()
    while len(buf) < HEADER_SIZE:
        chunk = sock.recv(HEADER_SIZE - len(buf))
        if not chunk:
            if allow_eof and not buf:
                return None
            raise ConnectionError("peer closed the connection in the middle of a header")
        buf += chunk
    return unpack_header(bytes(buf))
