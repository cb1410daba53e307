"""The TCP path of the transfer service speaks the reference service's wire format.

The reference's C++ service cannot be built here (abseil, pybind11, cmake), so its side of each
exchange is played by a few lines of socket code written from the format's definition
(replication/transfer_service/protocol.h:32-72: a packed header of one type byte, char fields of
1024, 1024, 64, 64 and 64 bytes and a signed 64-bit size) and from the message flows in
transfer_service.cpp (put :628-690 / :702-780, get :782-836 / :975-1035, the push that answers a get
:838-915). The header is built here with ``struct`` independently of ``wire.py``, so the two must
agree byte for byte."""

import os
import random
import socket
import struct
import threading
import uuid

import pytest

from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

HEADER_SIZE = 2249
PUT, GET, RESPOND, ACK, ERROR = 1, 2, 3, 4, 5


def ref_header(type_, source_obj_id="", dest_obj_id="", source_address="", dest_address="", task_id="", obj_size=0):
    """The reference's ``ObjInfoHeader`` as its compiler lays it out (packed, little-endian)."""
    raw = bytes([type_])
    for text, width in ((source_obj_id, 1024), (dest_obj_id, 1024), (source_address, 64), (dest_address, 64), (task_id, 64)):
        raw += text.encode().ljust(width, b"\0")
    raw += struct.pack("<q", obj_size)
    assert len(raw) == HEADER_SIZE
    return raw


def ref_parse(raw):
    assert len(raw) == HEADER_SIZE
    fields, at = [], 1
    for width in (1024, 1024, 64, 64, 64):
        fields.append(raw[at : at + width].split(b"\0", 1)[0].decode())
        at += width
    return {
        "type": raw[0], "source_obj_id": fields[0], "dest_obj_id": fields[1], "source_address": fields[2],
        "dest_address": fields[3], "task_id": fields[4], "obj_size": struct.unpack("<q", raw[at:])[0],
    }


def recv_exact(sock, n):
    out = b""
    while len(out) < n:
        chunk = sock.recv(n - len(out))
        if not chunk:
            raise ConnectionError("closed")
        out += chunk
    return out


@pytest.fixture
def service(tmp_path, monkeypatch):
    monkeypatch.setenv("MLFLASHPOINT_REPL_TRANSPORT", "tcp")
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    replicas = str(tmp_path / "replicas")
    svc = TransferService(replica_path_mapper=lambda obj, src: os.path.join(replicas, f"src{src}", obj.lstrip("/")))
    assert svc.initialize(0, threads=4, global_rank=3) > 0
    yield svc, replicas
    svc.shutdown()


def connect(address):
    host, port = address.split(":")
    return socket.create_connection((host, int(port)), timeout=30)


def test_header_layout_matches_the_reference_struct():
    from ml_flashpoint.replication.transfer_service import wire

    assert wire.HEADER_SIZE == HEADER_SIZE
    ours = wire.pack_header(wire.GET_OBJ, source_obj_id="/a/b", dest_obj_id="/c/d", source_address="10.0.0.1:5", dest_address="10.0.0.2:6",
                            task_id="0123-abc", obj_size=-7)
    assert ours == ref_header(GET, "/a/b", "/c/d", "10.0.0.1:5", "10.0.0.2:6", "0123-abc", -7)
    assert (wire.PUT_OBJ, wire.GET_OBJ, wire.RESPOND_TO_GET_OBJ, wire.ACK, wire.ERROR) == (PUT, GET, RESPOND, ACK, ERROR)
    back = wire.unpack_header(ref_header(RESPOND, "s", "d", "x:1", "y:2", "t", 1 << 40))
    assert back == wire.Header(RESPOND, "s", "d", "x:1", "y:2", "t", 1 << 40)
    # a field that is not NUL-terminated reads up to its last byte, never beyond (protocol.h:62-68)
    unterminated = bytes([ACK]) + b"s" * 1024 + b"\0" * (HEADER_SIZE - 1025)
    assert wire.unpack_header(unterminated).source_obj_id == "s" * 1023
    with pytest.raises(ValueError):
        wire.pack_header(wire.PUT_OBJ, dest_obj_id="x" * 1024)
    with pytest.raises(ValueError):
        wire.pack_header(wire.PUT_OBJ, task_id="t" * 64)


def test_a_reference_sender_can_put_here_on_a_connection_it_keeps_open(service, tmp_path):
    svc, replicas = service
    first, second = random.Random(1).randbytes(70001), random.Random(2).randbytes(4096)
    with connect(svc.address) as s:
        for name, data in (("/ckpt/step-1/o_a.distcp", first), ("/ckpt/step-1/o_b.distcp", second)):
            s.sendall(ref_header(PUT, dest_obj_id=name, obj_size=len(data)) + data)
            answer = ref_parse(recv_exact(s, HEADER_SIZE))
            assert answer["type"] == ACK and answer["obj_size"] == 0
            landed = os.path.join(replicas, "src-1", name.lstrip("/"))  # no rank on a reference task id
            assert open(landed, "rb").read() == data and not os.path.exists(landed + ".tmp")
        # a size that is not positive is refused with an error header, as the reference refuses it
        s.sendall(ref_header(PUT, dest_obj_id="/ckpt/step-1/o_c.distcp", obj_size=0, task_id="abc"))
        answer = ref_parse(recv_exact(s, HEADER_SIZE))
        assert answer["type"] == ERROR and answer["task_id"] == "abc"
        # and the connection still works afterwards
        s.sendall(ref_header(PUT, dest_obj_id="/ckpt/step-1/o_d.distcp", obj_size=3) + b"xyz")
        assert ref_parse(recv_exact(s, HEADER_SIZE))["type"] == ACK


def test_a_reference_requester_can_get_from_here(service, tmp_path):
    svc, _ = service
    held = tmp_path / "held" / "o_src3.distcp"
    os.makedirs(held.parent)
    data = random.Random(3).randbytes(123457)
    buf = BufferObject(str(held), len(data), overwrite=True)
    memoryview(buf)[:] = data
    buf.close()
    listener = socket.socket()
    listener.bind(("127.0.0.1", 0))
    listener.listen(4)
    listener.settimeout(30)
    mine = f"127.0.0.1:{listener.getsockname()[1]}"
    task = str(uuid.uuid4())
    want = str(tmp_path / "fetched.distcp")
    with connect(svc.address) as s:
        s.sendall(ref_header(GET, source_obj_id=str(held), dest_obj_id=want, source_address=svc.address, dest_address=mine, task_id=task))
        answer = ref_parse(recv_exact(s, HEADER_SIZE))
        assert answer["type"] == ACK and answer["task_id"] == task
        push, _ = listener.accept()
        with push:
            header = ref_parse(recv_exact(push, HEADER_SIZE))
            assert header["type"] == RESPOND and header["task_id"] == task and header["dest_obj_id"] == want
            assert header["obj_size"] == len(data)
            assert recv_exact(push, header["obj_size"]) == data
            push.sendall(ref_header(ACK))
        # an object that is not there: an error header on the request's connection, no push
        s.sendall(ref_header(GET, source_obj_id="/no/such/object", dest_obj_id=want, source_address=svc.address, dest_address=mine, task_id="t2"))
        answer = ref_parse(recv_exact(s, HEADER_SIZE))
        assert answer["type"] == ERROR and answer["task_id"] == "t2"
    listener.close()


class _ReferencePeer:
    """The receiving half of the reference's service, in memory: stores puts, serves gets by pushing
    to the requester's listener, keeps every header it saw."""

    def __init__(self):
        self.objects, self.headers = {}, []
        self.listener = socket.socket()
        self.listener.bind(("127.0.0.1", 0))
        self.listener.listen(8)
        self.address = f"127.0.0.1:{self.listener.getsockname()[1]}"
        self.thread = threading.Thread(target=self._accept, daemon=True)
        self.thread.start()

    def _accept(self):
        while True:
            try:
                conn, _ = self.listener.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn):
        with conn:
            while True:
                try:
                    header = ref_parse(recv_exact(conn, HEADER_SIZE))
                except (ConnectionError, OSError):
                    return
                self.headers.append(header)
                if header["type"] == PUT:
                    self.objects[header["dest_obj_id"]] = recv_exact(conn, header["obj_size"])
                    conn.sendall(ref_header(ACK))
                elif header["type"] == GET:
                    data = self.objects.get(header["source_obj_id"])
                    if data is None:
                        conn.sendall(ref_header(ERROR, task_id=header["task_id"]))
                        continue
                    conn.sendall(ref_header(ACK, task_id=header["task_id"]))
                    with connect(header["dest_address"]) as push:
                        push.sendall(ref_header(RESPOND, source_obj_id=header["source_obj_id"], dest_obj_id=header["dest_obj_id"],
                                                task_id=header["task_id"], obj_size=len(data)) + data)
                        assert ref_parse(recv_exact(push, HEADER_SIZE))["type"] == ACK
                # unknown types are ignored, as the reference's dispatcher ignores them

    def close(self):
        self.listener.close()


def test_put_to_and_get_from_a_reference_peer(service, tmp_path):
    svc, _ = service
    peer = _ReferencePeer()
    try:
        src = tmp_path / "primary" / "o_src3.distcp"
        os.makedirs(src.parent)
        data = random.Random(5).randbytes(300001)
        buf = BufferObject(str(src), len(data), overwrite=True)
        memoryview(buf)[:] = data
        buf.close()
        ro = BufferObject(str(src))
        assert svc.async_put(ro.get_data_ptr(), ro.get_capacity(), peer.address, str(src)).result(timeout=60).success
        ro.close()
        assert peer.objects[str(src)] == data
        put = next(h for h in peer.headers if h["type"] == PUT)
        assert put["obj_size"] == len(data) and put["dest_obj_id"] == str(src) and put["task_id"].endswith("~3")
        back = str(tmp_path / "back" / "o.distcp")
        assert svc.async_get(str(src), peer.address, back).result(timeout=60).success
        assert open(back, "rb").read() == data and not os.path.exists(back + ".tmp")
        get = next(h for h in peer.headers if h["type"] == GET)
        assert get["dest_address"] == svc.address and get["source_address"] == peer.address and get["dest_obj_id"] == back
        with pytest.raises(RuntimeError, match="not held here"):
            svc.async_get("/not/there", peer.address, back + "2").result(timeout=60)
    finally:
        peer.close()


def test_a_peer_that_ignores_the_native_opening_is_remembered_as_a_reference_peer(service, tmp_path, monkeypatch):
    from ml_flashpoint.replication.transfer_service import transfer_service_ext as mod

    svc, _ = service
    monkeypatch.setattr(mod, "_HELLO_TIMEOUT_S", 0.3)
    peer = _ReferencePeer()
    try:
        src = tmp_path / "o.distcp"
        buf = BufferObject(str(src), 4096, overwrite=True)
        buf.close()
        ro = BufferObject(str(src))
        assert svc._put_native("task", ro.get_data_ptr(), ro.get_capacity(), peer.address, str(src), False) is False
        ro.close()
        assert peer.address in svc._wire_only
        assert any(h["type"] == 0x42 for h in peer.headers) and str(src) not in peer.objects
        # a CUDA rank would now use the wire format for this peer, and ask again once the mark has aged
        monkeypatch.setattr(svc, "_cuda", True)
        monkeypatch.setattr(svc, "_transport", "auto")
        assert not svc._native_first(peer.address)
        svc._wire_only[peer.address] -= mod._WIRE_ONLY_S + 1
        assert svc._native_first(peer.address)
    finally:
        peer.close()


def test_an_error_message_from_the_holder_fails_the_pending_get(service, tmp_path):
    """A holder that acknowledged a get and then cannot push the object sends an error header with
    the task id to the requester's listener (the reference fails the task on it,
    transfer_service.cpp:608-611); the get must fail then, not wait for its timeout."""
    svc, _ = service
    listener = socket.socket()
    listener.bind(("127.0.0.1", 0))
    listener.listen(4)
    holder = f"127.0.0.1:{listener.getsockname()[1]}"

    def play_holder():
        conn, _ = listener.accept()
        with conn:
            request = ref_parse(recv_exact(conn, HEADER_SIZE))
            conn.sendall(ref_header(ACK, task_id=request["task_id"]))
            with connect(request["dest_address"]) as back:
                back.sendall(ref_header(ERROR, task_id=request["task_id"]))

    thread = threading.Thread(target=play_holder, daemon=True)
    thread.start()
    with pytest.raises(RuntimeError, match="Received error message"):
        svc.async_get("/held/elsewhere", holder, str(tmp_path / "never")).result(timeout=30)
    thread.join(timeout=10)
    listener.close()
    assert not os.path.exists(tmp_path / "never")


def test_a_message_of_unknown_type_ends_the_connection(service):
    svc, _ = service
    with connect(svc.address) as s:
        s.sendall(bytes([99]) + b"\0" * (HEADER_SIZE - 1))
        s.settimeout(10)
        assert s.recv(1) == b""  # closed by the service, nothing sent
    # the service itself keeps working
    with connect(svc.address) as s:
        s.sendall(ref_header(PUT, dest_obj_id="/after/unknown.distcp", obj_size=2) + b"ok")
        assert ref_parse(recv_exact(s, HEADER_SIZE))["type"] == ACK


def test_replication_manager_replicates_to_and_recovers_from_a_reference_peer(service, tmp_path, monkeypatch):
    """The manager-level flow of a mixed fleet: rank 0 runs this package, its ring partner rank 1 the
    reference's service. ``async_replicate`` leaves the whole object with the partner;
    after the local copy is lost ``sync_bulk_retrieve`` brings it back, byte for byte."""
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.checkpoint_id_types import CheckpointObjectId
    from ml_flashpoint.replication import replication_manager as rm

    svc, _ = service
    peer = _ReferencePeer()
    try:
        monkeypatch.setattr(rm.dist, "get_rank", lambda: 0)
        manager = rm.ReplicationManager()
        manager.initialize(CheckpointObjectManager(), replication_transfer_service=svc,
                           repl_strategy=rm.RingReplicationStrategy([svc.address, peer.address]))
        com = CheckpointObjectManager()
        oid = CheckpointObjectId(str(tmp_path / "step-7_ckpt" / "o_src0.distcp"))
        payload = random.Random(11).randbytes(200003)
        with com.acquire_buffer(oid, len(payload) + 8192) as w:
            w.write(payload)
        on_disk = open(str(oid), "rb").read()
        futures = manager.async_replicate(com.get_buffer(oid))
        assert len(futures) == 1 and futures[0].result(timeout=60).success
        assert peer.objects[str(oid)] == on_disk
        os.remove(str(oid))
        assert manager.sync_bulk_retrieve(1, [oid], []) is True
        assert open(str(oid), "rb").read() == on_disk
    finally:
        peer.close()
