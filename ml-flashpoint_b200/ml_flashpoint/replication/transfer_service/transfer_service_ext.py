"""``TransferService``: moves whole checkpoint objects between ranks of one NVLink domain.

Same four-call surface as the reference's compiled service of this name and module path
(replication/transfer_service/bindings.cpp:23-80, transfer_service.h:57-186): ``initialize`` returns
the bound control port (or -1), ``async_put`` / ``async_get`` return ``concurrent.futures.Future``s
that resolve to a ``TransferResult`` or carry an exception, ``shutdown`` fails what is pending. The
receiver writes ``<object>.tmp`` and renames it once complete, as the reference does
(transfer_service.cpp:702-780).

The reference streams the object through TCP sockets in 1 MiB ``send()`` calls. Here only a few
small JSON control messages travel over a socket; the object itself goes GPU to GPU:

  sender HBM image --(copy kernel, 16-byte stores to the peer's HBM over NVLink)--> receiver HBM
  receiver HBM --(copy engine, PCIe)--> receiver's object mapping --rename--> done

The sender reuses the HBM image the save just produced when it is still resident (see
``gpu_engine.resident_image``); otherwise the object is first brought into HBM from the host
pointer that was passed in. The receiving buffer is exported with CUDA IPC and opened by the
sender; peers inside one process exchange the raw device pointer instead.

CUDA IPC works between processes of one host only. Peers on different hosts (or without a CUDA
device) stream the object over TCP, straight from the sender's mapping into the receiver's
``<object>.tmp`` mapping, which is what the reference does for every transfer, and in the
reference's own wire format (``wire.py``; protocol.h:32-72): a rank running this service can
replicate to, and retrieve from, a rank running the reference's service and the other way round.
Gets always travel in that format (request, ack, and the holder pushing the object back to the
requester's listener); the push itself, like every put, goes over NVLink when the destination is a
CUDA rank of this host that answers this package's own opening message (``wire.NATIVE``, a message
type the reference ignores). A peer that does not answer it within ``_HELLO_TIMEOUT_S`` is
taken for a reference peer for the next ``_WIRE_ONLY_S`` seconds. ``MLFLASHPOINT_REPL_TRANSPORT`` = ``auto`` (default) | ``nvlink`` |
``tcp`` (``tcp``: the reference's wire format for everything, no opening message).
"""

from __future__ import annotations

import concurrent.futures
import contextlib
import ctypes
import json
import os
import socket
import struct
import threading
import time
import uuid
from typing import Callable, Dict, Optional, Tuple

from ml_flashpoint import _native
from ml_flashpoint.core.mlf_logging import get_logger
from ml_flashpoint.replication.transfer_service import wire

_LOGGER = get_logger(__name__)

METADATA_SIZE = 4096
_LEN = struct.Struct("<I")
_MAX_MESSAGE = 1 << 20
_HELLO_TIMEOUT_S = 3.0  # how long a peer may take to answer the native opening message
_GET_TIMEOUT_S = 300.0  # how long a get waits for the holder's push after its request was acknowledged
_WIRE_ONLY_S = 60.0  # how long a peer that ignored the opening message is spoken to in the wire format before it is asked again


def _task_key_and_rank(wire_task_id: str) -> Tuple[str, int]:
    """Task ids this service puts on the wire are ``<id>~<global rank>``; the reference's are bare
    UUIDs. Returns the id and the rank (-1 for a reference peer)."""
    key, sep, rank = wire_task_id.partition("~")
    if sep and rank.lstrip("-").isdigit():
        return key, int(rank)
    return wire_task_id, -1


class TransferResult:
    """Outcome of one transfer (reference: ``TransferResult`` in transfer_service.h:50-54)."""

    def __init__(self, task_id: str = "", success: bool = False, error_message: str = ""):
        self.task_id = task_id
        self.success = success
        self.error_message = error_message

    def __repr__(self) -> str:
        return f"TransferResult(task_id={self.task_id!r}, success={self.success}, error_message={self.error_message!r})"


def _send_msg(sock: socket.socket, payload: dict) -> None:
    raw = json.dumps(payload).encode()
    sock.sendall(_LEN.pack(len(raw)) + raw)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    parts = []
    while n:
        chunk = sock.recv(n)
        if not chunk:
            raise ConnectionError("peer closed the control connection")
        parts.append(chunk)
        n -= len(chunk)
    return b"".join(parts)


def _recv_msg(sock: socket.socket) -> dict:
    (n,) = _LEN.unpack(_recv_exact(sock, _LEN.size))
    if n > _MAX_MESSAGE:
        raise ValueError(f"control message of {n} bytes exceeds the limit")
    return json.loads(_recv_exact(sock, n))


def _split_address(address: str) -> Tuple[str, int]:
    host, _, port = address.rpartition(":")
    if not host or not port.isdigit():
        raise ValueError(f"address must look like '<host>:<port>', got '{address}'")
    return host, int(port)


def _host_identity() -> str:
    """Identifies this machine boot: CUDA IPC handles are only meaningful between equal identities."""
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            boot = f.read().strip()
    except OSError:
        boot = ""
    return f"{socket.gethostname()}/{boot}"


def _cuda_usable() -> bool:
    try:
        import torch

        return bool(torch.cuda.is_available())
    except Exception:
        return False


def _recv_into(sock: socket.socket, view: memoryview) -> None:
    got = 0
    while got < len(view):
        n = sock.recv_into(view[got:], min(len(view) - got, 4 << 20))
        if n == 0:
            raise ConnectionError("peer closed the connection in the middle of an object")
        got += n


class ReplicaNamespace:
    """Where replicas live when replication partners share one filesystem (the ranks of one box).

    The reference stores a replica under the sender's own path on another host
    (transfer_service.cpp:702-780). On one box that path is the primary itself, so replicas go to
    ``<root>/src<sender rank>/<object path>`` instead. An instance is callable as the
    ``replica_path_mapper`` of ``TransferService``; ``held_objects`` is the reverse view a loader
    needs during recovery: which objects of a container this rank can serve from its replicas."""

    def __init__(self, root: str):
        self.root = str(root)

    def __call__(self, object_id: str, source_rank: int) -> str:
        return os.path.join(self.root, f"src{source_rank}", str(object_id).lstrip("/"))

    def held_objects(self, container_path: str) -> list:
        """Original object paths of the replicas held here for ``container_path`` (any sender)."""
        found = []
        try:
            senders = sorted(os.listdir(self.root))
        except OSError:
            return found
        for sender in senders:
            if not sender.startswith("src"):
                continue
            mirrored = os.path.join(self.root, sender, str(container_path).lstrip("/"))
            try:
                names = os.listdir(mirrored)
            except OSError:
                continue
            found.extend(os.path.join(str(container_path), n) for n in names if not n.endswith(".tmp"))
        return found


class _DeviceBuffer:
    """Device memory from plain ``cudaMalloc`` (so that an IPC handle can be exported for it)."""

    def __init__(self, nbytes: int):
        ptr = ctypes.c_void_p()
        _native.check(_native.lib().mlf_dev_alloc(nbytes, ctypes.byref(ptr)))
        self.ptr = int(ptr.value)
        self.nbytes = nbytes
        handle = (ctypes.c_uint8 * _native.MLF_IPC_HANDLE_BYTES)()
        _native.check(_native.lib().mlf_ipc_export(ctypes.c_void_p(self.ptr), handle))
        self.ipc_hex = bytes(handle).hex()

    def free(self) -> None:
        if self.ptr:
            _native.lib().mlf_dev_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0


class TransferService:
    def __init__(self, replica_path_mapper: Optional[Callable[[str, int], str]] = None, landing_pool=None,
                 landing_chunk_bytes: Optional[int] = None):
        """``replica_path_mapper(object_id, source_rank) -> path`` decides where a received object is
        stored. The default keeps the sender's path, which is right when peers have separate
        filesystems; ranks that share one must map replicas elsewhere or they would overwrite the
        primary copy.

        ``landing_pool`` is an optional ``BufferPool`` of page-locked files: received objects are then
        drained into a pool file by one copy-engine transfer (and appear as a symlink to it, like
        objects saved through the pool) instead of into a fresh pageable file.

        ``landing_chunk_bytes`` (default: ``MLFLASHPOINT_REPL_LANDING_CHUNK_BYTES``, 0 = off) bounds
        the HBM a transfer holds: instead of a landing buffer the size of the object, the receiver keeps
        two slots of that many bytes per sender and drains one to its file while the sender's copy
        kernel fills the other; the sender's own bounce buffer shrinks to one slot as well. The NVLink
        hop then runs at the pace of the receiver's drain to host memory."""
        self._map_path = replica_path_mapper or (lambda object_id, source_rank: object_id)
        self._landing_pool = landing_pool
        if landing_chunk_bytes is None:
            landing_chunk_bytes = int(os.environ.get("MLFLASHPOINT_REPL_LANDING_CHUNK_BYTES", "0") or 0)
        self._landing_chunk = max(0, int(landing_chunk_bytes)) // 256 * 256
        self._listener: Optional[socket.socket] = None
        self._accept_thread: Optional[threading.Thread] = None
        self._workers: Optional[concurrent.futures.ThreadPoolExecutor] = None
        self._running = False
        self._rank = -1
        self._device = 0
        self._host = "127.0.0.1"
        self._port = -1
        self._lock = threading.Lock()
        self._pending: Dict[str, concurrent.futures.Future] = {}
        self._gets: Dict[str, dict] = {}  # acknowledged gets waiting for the holder's push, by task id
        self._wire_only: Dict[str, float] = {}  # addresses that did not answer the native opening message, and when
        self._local_hosts: Dict[str, bool] = {}
        self._connections: set = set()  # accepted connections being served
        self._inbound: Dict[int, _DeviceBuffer] = {}  # per source rank
        self._inbound_locks: Dict[int, threading.Lock] = {}
        self._retired: list = []  # outgrown landing buffers, kept until shutdown
        self._opened_ipc: Dict[str, int] = {}
        self._bounce: Optional[_DeviceBuffer] = None
        self._stream = ctypes.c_void_p()
        self._task_marks = threading.local()  # phase timestamps of the transfer a worker thread is running
        self._transport = os.environ.get("MLFLASHPOINT_REPL_TRANSPORT", "auto").lower()
        self._cuda = False
        # device timing of the most recent outgoing transfer: {"bytes", "hop_ms", "from_hbm_image"}
        self.last_put_stats: Optional[dict] = None

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, listen_port: int = 0, threads: int = 16, conn_pool_per_peer: int = 16, global_rank: int = -1) -> int:
        """Binds the control socket and starts the workers. Returns the port, or -1 on failure.

        The CUDA device current on the calling thread becomes the service's device.
        ``conn_pool_per_peer`` is accepted for signature compatibility; outgoing connections are
        opened per transfer and not pooled (incoming ones may stay open between messages, as the
        reference's pooled connections do).
        """
        try:
            if self._transport not in ("auto", "nvlink", "tcp"):
                raise ValueError(f"unknown MLFLASHPOINT_REPL_TRANSPORT '{self._transport}'")
            self._cuda = self._transport != "tcp" and _cuda_usable()
            if self._transport == "nvlink" and not self._cuda:
                raise RuntimeError("the nvlink transport needs a CUDA device")
            if self._cuda:
                dev = ctypes.c_int32()
                _native.check(_native.lib().mlf_get_device(ctypes.byref(dev)))
                self._device = dev.value
                _native.check(_native.lib().mlf_stream_create(ctypes.byref(self._stream)))
            self._rank = global_rank
            self._host = os.environ.get("MLFLASHPOINT_REPL_HOST", "127.0.0.1")
            listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            listener.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            listener.bind((self._host, listen_port))
            listener.listen(128)
            listener.settimeout(0.2)
            self._listener = listener
            self._port = listener.getsockname()[1]
            self._workers = concurrent.futures.ThreadPoolExecutor(max_workers=max(2, threads), thread_name_prefix="mlf-xfer")
            self._running = True
            self._accept_thread = threading.Thread(target=self._accept_loop, name="mlf-xfer-accept", daemon=True)
            self._accept_thread.start()
            return self._port
        except Exception:
            _LOGGER.exception("TransferService failed to initialize")
            return -1

    @property
    def address(self) -> str:
        return f"{self._host}:{self._port}"

    def held_device_bytes(self) -> int:
        """HBM this service holds right now: landing buffers (one per source rank), outgrown ones kept
        until shutdown, and the sender-side bounce buffer."""
        with self._lock:
            buffers = list(self._inbound.values()) + list(self._retired) + ([self._bounce] if self._bounce else [])
        return sum(b.nbytes for b in buffers if b.ptr)

    def release_peers(self) -> None:
        """Closes the landing buffers of other processes that this service has opened.

        An exporter may free a buffer only after every importer has closed it, so ranks that shut
        down together call this first, synchronise, and then ``shutdown``."""
        if self._cuda:
            _native.lib().mlf_set_device(self._device)
        with self._lock:
            opened, self._opened_ipc = self._opened_ipc, {}
        for ptr in opened.values():
            _native.lib().mlf_ipc_close(ctypes.c_void_p(ptr))

    def shutdown(self) -> None:
        """Stops accepting, fails every pending future, releases device buffers."""
        with self._lock:
            if not self._running:
                return
            self._running = False
            pending = list(self._pending.values())
            self._pending.clear()
            waiting_gets = list(self._gets.values())
            connections = list(self._connections)
        for f in pending:
            if not f.done():
                f.set_exception(RuntimeError("TransferService is shutting down"))
        for entry in waiting_gets:
            entry["error"] = RuntimeError("TransferService is shutting down")
            entry["event"].set()
        for conn in connections:  # wakes the threads serving them
            try:
                conn.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass
        if self._accept_thread:
            self._accept_thread.join(timeout=2.0)
        if self._listener:
            self._listener.close()
        if self._workers:
            self._workers.shutdown(wait=True, cancel_futures=True)
        if self._cuda:
            _native.lib().mlf_set_device(self._device)
        for ptr in self._opened_ipc.values():
            _native.lib().mlf_ipc_close(ctypes.c_void_p(ptr))
        self._opened_ipc.clear()
        for buf in list(self._inbound.values()) + self._retired + ([self._bounce] if self._bounce else []):
            buf.free()
        self._inbound.clear()
        self._retired = []
        self._bounce = None
        if self._stream:
            _native.lib().mlf_stream_destroy(self._stream)
            self._stream = ctypes.c_void_p()

    # ------------------------------------------------------------------ public transfers
    def async_put(self, data_ptr: int, data_size: int, dest_address: str, dest_object_id: str) -> concurrent.futures.Future:
        """Copies ``data_size`` bytes at host address ``data_ptr`` to the peer as ``dest_object_id``.

        The memory is borrowed until the future completes.
        """
        return self._submit(self._run_put, "PUT", int(data_size), int(data_ptr), int(data_size), dest_address, dest_object_id)

    def async_get(self, remote_object_id_to_get_obj_from: str, source_address: str, local_object_id_to_save_received_obj: str) -> concurrent.futures.Future:
        """Asks the peer at ``source_address`` to send one of its objects here."""
        return self._submit(self._run_get, "GET", 0, remote_object_id_to_get_obj_from, source_address, local_object_id_to_save_received_obj)

    def _submit(self, fn, task_type: str, data_size: int, *args) -> concurrent.futures.Future:
        future: concurrent.futures.Future = concurrent.futures.Future()
        task_id = uuid.uuid4().hex
        submitted = time.perf_counter()
        with self._lock:
            if not self._running:
                future.set_exception(RuntimeError("TransferService is not running"))
                return future
            self._pending[task_id] = future

        def _run():
            marks = {"start": time.perf_counter()}
            self._task_marks.marks = marks
            try:
                fn(task_id, *args)
                outcome, error = TransferResult(task_id, True, ""), None
            except Exception as e:  # surfaces on the future, as the reference's service does
                _LOGGER.exception("transfer task %s failed", task_id)
                outcome, error = None, e
            finally:
                self._task_marks.marks = None
            self._report_result(task_id, task_type, data_size, error, submitted, marks)
            with self._lock:
                self._pending.pop(task_id, None)
            if future.done():
                return
            if error is None:
                future.set_result(outcome)
            else:
                future.set_exception(RuntimeError(str(error)))

        self._workers.submit(_run)
        return future

    def _mark(self, name: str) -> None:
        """Timestamps a phase of the transfer running on this worker thread."""
        marks = getattr(self._task_marks, "marks", None)
        if marks is not None:
            marks.setdefault(name, time.perf_counter())

    @staticmethod
    def _report_result(task_id: str, task_type: str, data_size: int, error, submitted: float, marks: dict) -> None:
        """One line per finished transfer in the shape the reference's service logs
        (transfer_service.cpp:489-492 with the fields of task.cpp:39-111), which its log
        summariser reads. ``data_sent`` covers the GPU-to-GPU hop for the NVLink transport."""
        finished = time.perf_counter()

        def span(a, b):
            if a is None or b is None:
                return 0.0
            return (b - a) * 1e3

        start = marks.get("start")
        connected = marks.get("connection_acquired")
        header = marks.get("header_sent")
        moved = marks.get("data_sent") or marks.get("data_received")
        label = "data_received" if task_type == "GET" else "data_sent"
        timing = (
            f"wait_to_be_executed={span(submitted, start):.3f}ms, connection_acquired={span(start, connected):.3f}ms, "
            f"header_sent={span(connected, header):.3f}ms, {label}={span(header, moved):.3f}ms, total={span(submitted, finished):.3f}ms"
        )
        _LOGGER.info(
            "TransferService::report_result: task_id=%s, task_type=%s, data_size=%d, success=%d, message=%s, timing=%s",
            task_id, task_type, data_size, 0 if error else 1, "" if error is None else str(error), timing,
        )

    # ------------------------------------------------------------------ sender side
    def _connect(self, address: str) -> socket.socket:
        host, port = _split_address(address)
        last = None
        for _ in range(5):  # the reference retries connects 5 times, 100 ms apart
            try:
                conn = socket.create_connection((host, port), timeout=30.0)
                conn.settimeout(300.0)  # the peer answers only after draining the whole object to its file
                return conn
            except OSError as e:
                last = e
                threading.Event().wait(0.1)
        raise ConnectionError(f"cannot reach transfer service at {address}: {last}")

    def _peer_pointer(self, reply: dict) -> int:
        if reply["pid"] == os.getpid():
            if reply["device"] != self._device:
                _native.check(_native.lib().mlf_enable_peer_access(reply["device"]))
            return int(reply["ptr"])
        key = reply["ipc"]
        with self._lock:  # several transfers to one peer may run at once; the handle is opened once
            if key not in self._opened_ipc:
                out = ctypes.c_void_p()
                handle = (ctypes.c_uint8 * _native.MLF_IPC_HANDLE_BYTES).from_buffer_copy(bytes.fromhex(key))
                _native.check(_native.lib().mlf_ipc_open(handle, ctypes.byref(out)))
                self._opened_ipc[key] = int(out.value)
            return self._opened_ipc[key]

    def _is_local(self, host: str) -> bool:
        """Whether ``host`` names this machine: only an address of a local interface can be bound."""
        known = self._local_hosts.get(host)
        if known is None:
            try:
                with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as probe:
                    probe.bind((socket.gethostbyname(host), 0))
                known = True
            except OSError:
                known = False
            self._local_hosts[host] = known
        return known

    def _native_first(self, dest_address: str) -> bool:
        """Puts open with this package's own negotiation when it can end in the NVLink transport: a
        CUDA rank sending to a peer on this host that has not ignored the opening message before."""
        if self._transport == "nvlink":
            return True
        if self._transport == "tcp" or not self._cuda:
            return False
        ignored_at = self._wire_only.get(dest_address)
        if ignored_at is not None and time.monotonic() - ignored_at < _WIRE_ONLY_S:
            return False  # a busy peer of this package may have missed the greeting: it is asked again later
        return self._is_local(_split_address(dest_address)[0])

    def _run_put(self, task_id: str, data_ptr: int, data_size: int, dest_address: str, dest_object_id: str, exact_path: bool = False) -> None:
        if data_size <= 0 or not data_ptr:
            raise RuntimeError("Empty buffer or null data_ptr: async_put needs a non-empty source")
        if self._native_first(dest_address):
            if self._put_native(task_id, data_ptr, data_size, dest_address, dest_object_id, exact_path):
                return
            if self._transport == "nvlink":
                raise RuntimeError(f"the peer at {dest_address} does not answer the NVLink negotiation")
        self._put_wire(f"{task_id}~{self._rank}", data_ptr, data_size, dest_address, dest_object_id, respond=exact_path)

    def _put_wire(self, wire_task_id: str, data_ptr: int, data_size: int, dest_address: str, dest_object_id: str, respond: bool) -> None:
        """The reference's put (transfer_service.cpp:628-690), or with ``respond`` its answer to a get
        (:838-915): header, the object's bytes from the host mapping, then the peer's ack."""
        from ml_flashpoint.core import gpu_engine

        with self._connect(dest_address) as sock:
            self._mark("connection_acquired")
            gpu_engine.wait_object_on_host(dest_object_id)  # a save of it may still be draining
            sock.sendall(
                wire.pack_header(
                    wire.RESPOND_TO_GET_OBJ if respond else wire.PUT_OBJ, dest_obj_id=dest_object_id, obj_size=data_size,
                    task_id=wire_task_id, source_address=self.address,
                )
            )
            self._mark("header_sent")
            source = (ctypes.c_ubyte * data_size).from_address(data_ptr)
            sock.sendall(memoryview(source).cast("B"))
            self._mark("data_sent")
            self.last_put_stats = {"bytes": data_size, "hop_ms": None, "from_hbm_image": False, "transport": "tcp"}
            answer = wire.recv_header(sock)
        if answer.type == wire.ERROR:
            raise RuntimeError(f"Received error from destination for '{dest_object_id}'")
        if answer.type != wire.ACK:
            raise RuntimeError(f"Received unexpected ACK (message type {answer.type}) for '{dest_object_id}'")

    def _put_native(self, task_id: str, data_ptr: int, data_size: int, dest_address: str, dest_object_id: str, exact_path: bool) -> bool:
        """This package's own put: negotiated over the connection, carried by NVLink when both ends are
        CUDA ranks of one host. Returns False when the peer does not answer the opening message."""
        from ml_flashpoint.core import gpu_engine

        lib = _native.lib()
        if self._cuda:
            _native.check(lib.mlf_set_device(self._device))
        with self._connect(dest_address) as sock:
            self._mark("connection_acquired")
            sock.sendall(wire.pack_header(wire.NATIVE, task_id=f"{task_id}~{self._rank}", source_address=self.address))
            sock.settimeout(_HELLO_TIMEOUT_S)
            try:
                hello = _recv_msg(sock)
                if hello.get("hello") != "mlf-b200":
                    raise ValueError("not this package's greeting")
            except (socket.timeout, ConnectionError, ValueError, AttributeError):
                _LOGGER.info("peer %s does not answer the native opening message: using the reference's wire format for it", dest_address)
                self._wire_only[dest_address] = time.monotonic()
                return False
            sock.settimeout(300.0)  # the peer answers only after draining the whole object to its file
            _send_msg(
                sock,
                {
                    "op": "put_begin", "obj": dest_object_id, "size": data_size, "src_rank": self._rank, "task": task_id,
                    "exact_path": exact_path, "host": _host_identity(), "gpu": self._cuda,
                },
            )
            reply = _recv_msg(sock)
            self._mark("header_sent")
            if not reply.get("ok"):
                raise RuntimeError(f"peer refused put of '{dest_object_id}': {reply.get('error')}")
            if reply.get("transport") == "tcp":
                gpu_engine.wait_object_on_host(dest_object_id)  # a save of it may still be draining
                source = (ctypes.c_ubyte * data_size).from_address(data_ptr)
                sock.sendall(memoryview(source).cast("B"))
                self._mark("data_sent")
                self.last_put_stats = {"bytes": data_size, "hop_ms": None, "from_hbm_image": False, "transport": "tcp"}
                final = _recv_msg(sock)
                if not final.get("ok"):
                    raise RuntimeError(f"peer failed to store '{dest_object_id}': {final.get('error')}")
                return True
            peer = self._peer_pointer(reply)
            stream = self._stream
            twin = None if exact_path else gpu_engine.resident_image(dest_object_id, data_size - METADATA_SIZE)
            if reply.get("chunked"):
                self._put_in_chunks(sock, reply, peer, twin, data_ptr, data_size, dest_object_id)
                return True
            t0, t1 = ctypes.c_void_p(), ctypes.c_void_p()
            _native.check(lib.mlf_event_create(ctypes.byref(t0)))
            _native.check(lib.mlf_event_create(ctypes.byref(t1)))
            try:
                with contextlib.ExitStack() as lease:
                    image_ptr = None
                    if twin is not None:
                        try:
                            # waits for the pack kernel only: the hop overlaps the drain to the host
                            image_ptr = lease.enter_context(twin)
                        except RuntimeError:
                            # a newer save or a restore took the arena between lookup and lease: the
                            # object itself is complete in the host mapping, send it from there
                            twin = None
                    since_save_ms = None
                    if image_ptr is not None:
                        # metadata block from the host mapping (final since the bytes were claimed),
                        # data section from the HBM image of the save
                        _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(peer), ctypes.c_void_p(data_ptr), METADATA_SIZE, _native.MLF_COPY_H2D, stream))
                        _native.check(lib.mlf_event_record(t0, stream))
                        _native.check(lib.mlf_copy_kernel_launch(ctypes.c_void_p(peer + METADATA_SIZE), ctypes.c_void_p(image_ptr), data_size - METADATA_SIZE, stream, 0))
                        _native.check(lib.mlf_event_record(t1, stream))
                        _native.check(lib.mlf_stream_sync(stream))
                        began = twin.start_event
                        if began is not None:
                            ms = ctypes.c_float()
                            if lib.mlf_event_elapsed_ms(ctypes.c_void_p(began.cuda_event), t1, ctypes.byref(ms)) == 0:
                                since_save_ms = float(ms.value)
                    else:
                        gpu_engine.wait_object_on_host(dest_object_id)
                        with self._lock:
                            if self._bounce is None or self._bounce.nbytes < data_size:
                                if self._bounce:
                                    self._bounce.free()
                                self._bounce = _DeviceBuffer(data_size)
                            bounce = self._bounce
                        _native.check(lib.mlf_bounce_copy(ctypes.c_void_p(bounce.ptr), ctypes.c_void_p(data_ptr), data_size, 1, 0))
                        _native.check(lib.mlf_event_record(t0, stream))
                        _native.check(lib.mlf_copy_kernel_launch(ctypes.c_void_p(peer), ctypes.c_void_p(bounce.ptr), data_size, stream, 0))
                        _native.check(lib.mlf_event_record(t1, stream))
                        _native.check(lib.mlf_stream_sync(stream))
                self._mark("data_sent")
                ms = ctypes.c_float()
                _native.check(lib.mlf_event_elapsed_ms(t0, t1, ctypes.byref(ms)))
                self.last_put_stats = {
                    "bytes": data_size,
                    "hop_ms": float(ms.value),
                    "from_hbm_image": image_ptr is not None,
                    # device time from the start of the save's pack kernel to the last byte in the peer's HBM
                    "since_save_start_ms": since_save_ms,
                    "in_peer_hbm_at": time.perf_counter(),
                }
            finally:
                lib.mlf_event_destroy(t0)
                lib.mlf_event_destroy(t1)
            _send_msg(sock, {"op": "put_commit", "token": reply["token"]})
            final = _recv_msg(sock)
            if not final.get("ok"):
                raise RuntimeError(f"peer failed to store '{dest_object_id}': {final.get('error')}")
        return True

    def _put_in_chunks(self, sock, reply: dict, peer: int, twin, data_ptr: int, data_size: int, dest_object_id: str) -> None:
        """Sender side of a transfer whose receiver keeps a two-slot landing ring: chunk k goes into
        slot k mod 2 once the receiver has reported the chunk before last drained."""
        from ml_flashpoint.core import gpu_engine

        lib = _native.lib()
        stream = self._stream
        slot_bytes = int(reply["slot_bytes"])
        nchunks = (data_size + slot_bytes - 1) // slot_bytes
        t0, t1 = ctypes.c_void_p(), ctypes.c_void_p()
        _native.check(lib.mlf_event_create(ctypes.byref(t0)))
        _native.check(lib.mlf_event_create(ctypes.byref(t1)))
        hop_ms, freed = 0.0, 0

        def await_freed(upto: int) -> None:
            nonlocal freed
            while freed < upto:
                note = _recv_msg(sock)
                if note.get("op") != "slot_free":
                    raise RuntimeError(f"peer failed while receiving '{dest_object_id}': {note.get('error', note)}")
                freed += 1

        try:
            with contextlib.ExitStack() as lease:
                image_ptr = None
                if twin is not None:
                    try:
                        image_ptr = lease.enter_context(twin)
                    except RuntimeError:
                        image_ptr = None
                bounce = None
                if image_ptr is None:
                    gpu_engine.wait_object_on_host(dest_object_id)
                    with self._lock:
                        if self._bounce is None or self._bounce.nbytes < slot_bytes:
                            if self._bounce:
                                self._bounce.free()
                            self._bounce = _DeviceBuffer(slot_bytes)
                        bounce = self._bounce
                for k in range(nchunks):
                    off = k * slot_bytes
                    n = min(slot_bytes, data_size - off)
                    await_freed(k - 1)  # chunk k - 2 has left the slot this chunk goes into
                    slot = peer + (k % 2) * slot_bytes
                    if image_ptr is not None:
                        # object byte b < 4096 is the metadata block (host mapping), b >= 4096 is image[b - 4096]
                        skip = 0
                        if off < METADATA_SIZE:
                            skip = min(n, METADATA_SIZE - off)
                            _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(slot), ctypes.c_void_p(data_ptr + off), skip, _native.MLF_COPY_H2D, stream))
                        _native.check(lib.mlf_event_record(t0, stream))
                        if n > skip:
                            _native.check(lib.mlf_copy_kernel_launch(ctypes.c_void_p(slot + skip), ctypes.c_void_p(image_ptr + off + skip - METADATA_SIZE), n - skip, stream, 0))
                    else:
                        _native.check(lib.mlf_bounce_copy(ctypes.c_void_p(bounce.ptr), ctypes.c_void_p(data_ptr + off), n, 1, 0))
                        _native.check(lib.mlf_event_record(t0, stream))
                        _native.check(lib.mlf_copy_kernel_launch(ctypes.c_void_p(slot), ctypes.c_void_p(bounce.ptr), n, stream, 0))
                    _native.check(lib.mlf_event_record(t1, stream))
                    _native.check(lib.mlf_stream_sync(stream))
                    ms = ctypes.c_float()
                    _native.check(lib.mlf_event_elapsed_ms(t0, t1, ctypes.byref(ms)))
                    hop_ms += float(ms.value)
                    _send_msg(sock, {"op": "chunk", "k": k, "off": off, "len": n})
                self._mark("data_sent")
                await_freed(nchunks)
            self.last_put_stats = {
                "bytes": data_size, "hop_ms": hop_ms, "from_hbm_image": image_ptr is not None, "since_save_start_ms": None,
                "in_peer_hbm_at": time.perf_counter(), "chunks": nchunks, "chunk_bytes": slot_bytes,
            }
        finally:
            lib.mlf_event_destroy(t0)
            lib.mlf_event_destroy(t1)
        _send_msg(sock, {"op": "put_commit", "token": reply["token"]})
        final = _recv_msg(sock)
        if not final.get("ok"):
            raise RuntimeError(f"peer failed to store '{dest_object_id}': {final.get('error')}")

    def _run_get(self, task_id: str, remote_object_id: str, source_address: str, local_object_id: str) -> None:
        """The reference's get (transfer_service.cpp:782-836): the request names this service's own
        listener as destination; the holder acknowledges and then pushes the object there, which
        completes the get (``_finish_get``)."""
        entry = {"event": threading.Event(), "error": None}
        with self._lock:
            self._gets[task_id] = entry
        try:
            with self._connect(source_address) as sock:
                self._mark("connection_acquired")
                sock.sendall(
                    wire.pack_header(
                        wire.GET_OBJ, task_id=f"{task_id}~{self._rank}", source_obj_id=remote_object_id, dest_obj_id=local_object_id,
                        source_address=source_address, dest_address=self.address,
                    )
                )
                self._mark("header_sent")
                answer = wire.recv_header(sock)
            if answer.type == wire.ERROR:
                raise RuntimeError(f"Received error message from peer: object '{remote_object_id}' is not held here")
            if answer.type != wire.ACK:
                raise RuntimeError(f"Received unexpected response (message type {answer.type}) for GET request")
            deadline = time.monotonic() + _GET_TIMEOUT_S
            while not entry["event"].wait(0.2):
                if not self._running:
                    raise RuntimeError("TransferService is shutting down")
                if time.monotonic() > deadline:
                    raise TimeoutError(f"the holder of '{remote_object_id}' acknowledged the get but sent nothing")
            if entry["error"] is not None:
                raise RuntimeError(f"get of '{remote_object_id}' failed while it was being received: {entry['error']}")
            self._mark("data_received")
        finally:
            with self._lock:
                self._gets.pop(task_id, None)

    def _finish_get(self, task_key: str, error) -> None:
        with self._lock:
            entry = self._gets.get(task_key)
        if entry is not None:
            entry["error"] = error
            entry["event"].set()

    # ------------------------------------------------------------------ receiver side
    def _accept_loop(self) -> None:
        while self._running:
            try:
                conn, _ = self._listener.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            conn.settimeout(300.0)
            # a thread per connection, not a pool worker: the reference's service keeps its pooled
            # connections open between messages, and each would pin a worker for as long
            with self._lock:
                self._connections.add(conn)
            threading.Thread(target=self._serve, args=(conn,), name="mlf-xfer-serve", daemon=True).start()

    def _serve(self, conn: socket.socket) -> None:
        """Messages of one connection, one after the other, until the peer closes it."""
        try:
            with conn:
                while self._running:
                    try:
                        header = wire.recv_header(conn, allow_eof=True)
                    except socket.timeout:
                        continue  # an idle pooled connection
                    if header is None or not self._serve_message(conn, header):
                        return
        except (ConnectionError, OSError):
            if self._running:
                _LOGGER.warning("transfer service connection ended unexpectedly", exc_info=True)
        finally:
            with self._lock:
                self._connections.discard(conn)

    def _serve_message(self, conn: socket.socket, header: "wire.Header") -> bool:
        """Handles one message; False when the connection cannot carry another one."""
        if header.type in (wire.PUT_OBJ, wire.RESPOND_TO_GET_OBJ):
            return self._serve_wire_receive(conn, header, respond=header.type == wire.RESPOND_TO_GET_OBJ)
        if header.type == wire.GET_OBJ:
            self._serve_wire_get(conn, header)
            return True
        if header.type == wire.ERROR:  # a holder that could not push what it had acknowledged
            _LOGGER.error("error message received for task %s", header.task_id)
            self._finish_get(_task_key_and_rank(header.task_id)[0], RuntimeError("Received error message"))
            return True
        if header.type == wire.ACK:
            _LOGGER.error("unexpected ACK message received for task %s", header.task_id)
            return True
        if header.type != wire.NATIVE:
            _LOGGER.error("message of unknown type %d: closing the connection", header.type)
            return False
        # this package's own negotiation: greet, then one JSON request and its exchange
        request: dict = {}
        try:
            _send_msg(conn, {"hello": "mlf-b200"})
            request = _recv_msg(conn)
            if request.get("op") != "put_begin":
                raise ValueError(f"unknown op {request.get('op')}")
            self._serve_put(conn, request)
            if request.get("exact_path") and request.get("task"):
                self._finish_get(request["task"], None)  # the push a pending get of ours was waiting for
        except Exception as e:
            _LOGGER.exception("transfer service request failed")
            if request.get("exact_path") and request.get("task"):
                self._finish_get(request["task"], e)
            try:
                _send_msg(conn, {"ok": False, "error": str(e)})
            except OSError:
                pass
        return False  # native connections carry one transfer

    def _serve_wire_receive(self, conn: socket.socket, header: "wire.Header", respond: bool) -> bool:
        """Receiver of the reference's put, or of the push that answers a get of ours
        (transfer_service.cpp:702-780): ``<object>.tmp``, rename, ack."""
        from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

        task_key, source = _task_key_and_rank(header.task_id)

        def refuse(error) -> None:
            _LOGGER.error("receiving '%s' failed: %s", header.dest_obj_id, error)
            if respond:
                self._finish_get(task_key, error)
            try:
                conn.sendall(wire.pack_header(wire.ERROR, task_id=header.task_id))
            except OSError:
                pass

        if header.obj_size <= 0 or not header.dest_obj_id:
            refuse(ValueError(f"Invalid obj_size received: {header.obj_size}" if header.dest_obj_id else "empty dest_obj_id"))
            return True  # no bytes follow such a header
        final_path = header.dest_obj_id if respond else self._map_path(header.dest_obj_id, source)
        tmp_path = final_path + ".tmp"
        target = None
        try:
            os.makedirs(os.path.dirname(final_path) or ".", exist_ok=True)
            target = BufferObject(tmp_path, header.obj_size, overwrite=True)
            _recv_into(conn, memoryview(target))
            target.close()
            target = None
            os.rename(tmp_path, final_path)
        except BaseException as e:
            if target is not None:
                target.close()
            try:
                os.remove(tmp_path)  # never leave a partial object behind
            except OSError:
                pass
            refuse(e)
            if not isinstance(e, Exception):
                raise
            return False  # the rest of the object may still be in the connection
        conn.sendall(wire.pack_header(wire.ACK, task_id=header.task_id))
        if respond:
            self._finish_get(task_key, None)
        return True

    def _serve_wire_get(self, conn: socket.socket, header: "wire.Header") -> None:
        """Holder side of a get (transfer_service.cpp:975-1035): error when the object is not here,
        else an ack at once and the push to the requester's listener from a thread of its own."""
        _, requester = _task_key_and_rank(header.task_id)
        # the object itself, or the replica this service keeps on behalf of the asking rank
        candidates = [header.source_obj_id, self._map_path(header.source_obj_id, requester)]
        path = next((c for c in candidates if c and os.path.exists(c)), None)
        if path is None or not header.dest_address or not header.dest_obj_id:
            _LOGGER.error("get of '%s': object is not held here", header.source_obj_id)
            conn.sendall(wire.pack_header(wire.ERROR, task_id=header.task_id))
            return
        conn.sendall(wire.pack_header(wire.ACK, task_id=header.task_id))
        # a thread of its own, not a pool worker: the workers of two services that get from each other
        # may all be waiting for exactly these pushes
        threading.Thread(target=self._respond_to_get, args=(header, path), name="mlf-xfer-respond", daemon=True).start()

    def _respond_to_get(self, header: "wire.Header", path: str) -> None:
        from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

        task_key, requester = _task_key_and_rank(header.task_id)
        try:
            source = BufferObject(path)
            try:
                if requester >= 0 or "~" in header.task_id:
                    # a requester running this package: a put to its exact path, over NVLink when it can be
                    self._run_put(task_key, source.get_data_ptr(), source.get_capacity(), header.dest_address, header.dest_obj_id, exact_path=True)
                else:
                    self._put_wire(header.task_id, source.get_data_ptr(), source.get_capacity(), header.dest_address, header.dest_obj_id, respond=True)
            finally:
                source.close()
        except Exception:
            _LOGGER.exception("pushing '%s' to %s for get %s failed", path, header.dest_address, header.task_id)
            try:  # let the requester fail its get instead of waiting for the push
                with self._connect(header.dest_address) as sock:
                    sock.sendall(wire.pack_header(wire.ERROR, task_id=header.task_id))
            except Exception:
                pass

    def _serve_put(self, conn: socket.socket, request: dict) -> None:
        from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

        lib = _native.lib()
        size = int(request["size"])
        source = int(request.get("src_rank", -1))
        same_host = request.get("host") == _host_identity()
        if not (self._cuda and request.get("gpu") and same_host):
            if self._transport == "nvlink":
                raise RuntimeError("the nvlink transport needs both peers on one host with CUDA devices")
            self._serve_put_tcp(conn, request, size, source)
            return
        _native.check(lib.mlf_set_device(self._device))
        with self._lock:
            gate = self._inbound_locks.setdefault(source, threading.Lock())
        with gate:  # one inbound object per source at a time: they share the landing buffer
            if self._landing_chunk and size > 2 * self._landing_chunk:
                self._receive_in_chunks(conn, request, size, source)
                return
            landing = self._inbound.get(source)
            if landing is None or landing.nbytes < size:
                if landing:
                    # senders may still hold the old buffer open through its IPC handle: it is
                    # freed at shutdown, after they have released it
                    self._retired.append(landing)
                landing = _DeviceBuffer(size)
                self._inbound[source] = landing
            token = uuid.uuid4().hex
            _send_msg(conn, {"ok": True, "transport": "nvlink", "token": token, "ipc": landing.ipc_hex, "ptr": landing.ptr, "pid": os.getpid(), "device": self._device})
            commit = _recv_msg(conn)
            if commit.get("op") != "put_commit" or commit.get("token") != token:
                raise RuntimeError("put was not committed by the sender")
            final_path = request["obj"] if request.get("exact_path") else self._map_path(request["obj"], source)
            tmp_path = final_path + ".tmp"
            os.makedirs(os.path.dirname(final_path), exist_ok=True)
            for stale in (tmp_path, final_path):
                if os.path.lexists(stale):
                    os.remove(stale)
            pooled = None
            if self._landing_pool is not None:
                try:
                    pooled = self._landing_pool.acquire(associated_symlink=tmp_path)
                except RuntimeError:
                    pooled = None  # pool exhausted: fall back to a plain file
            if pooled is not None:
                pooled.ensure_total_size(size)
                inner = pooled._buffer_io
                stream = ctypes.c_void_p()
                _native.check(lib.mlf_stream_create(ctypes.byref(stream)))
                try:
                    host = inner.buffer_obj.get_data_ptr()
                    if inner.buffer_obj.is_cuda_registered:
                        _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(host), ctypes.c_void_p(landing.ptr), size, _native.MLF_COPY_D2H, stream))
                        _native.check(lib.mlf_stream_sync(stream))
                    else:
                        _native.check(lib.mlf_bounce_copy(ctypes.c_void_p(landing.ptr), ctypes.c_void_p(host), size, 0, 0))
                finally:
                    lib.mlf_stream_destroy(stream)
                self._landing_pool.relink(pooled, tmp_path, final_path)
            else:
                target = BufferObject(tmp_path, size, overwrite=True)
                try:
                    # the fresh file is pageable: drain through the bounce ring, whose CPU threads also
                    # fault the new tmpfs pages in parallel
                    _native.check(lib.mlf_bounce_copy(ctypes.c_void_p(landing.ptr), ctypes.c_void_p(target.get_data_ptr()), size, 0, 0))
                finally:
                    target.close()
                os.rename(tmp_path, final_path)
        _send_msg(conn, {"ok": True})

    def _receive_in_chunks(self, conn: socket.socket, request: dict, size: int, source: int) -> None:
        """Receiver side of a transfer through a two-slot landing ring (see ``landing_chunk_bytes``):
        every announced chunk is drained from its slot into the object's file at once, then the slot
        is reported free. The file is opened up front, under its temporary name."""
        from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

        lib = _native.lib()
        chunk = self._landing_chunk
        landing = self._inbound.get(source)
        if landing is None or landing.nbytes < 2 * chunk:
            if landing:
                self._retired.append(landing)
            landing = _DeviceBuffer(2 * chunk)
            self._inbound[source] = landing
        final_path = request["obj"] if request.get("exact_path") else self._map_path(request["obj"], source)
        tmp_path = final_path + ".tmp"
        os.makedirs(os.path.dirname(final_path), exist_ok=True)
        for stale in (tmp_path, final_path):
            if os.path.lexists(stale):
                os.remove(stale)
        pooled = None
        if self._landing_pool is not None:
            try:
                pooled = self._landing_pool.acquire(associated_symlink=tmp_path)
            except RuntimeError:
                pooled = None
        target = None
        stream = ctypes.c_void_p()
        _native.check(lib.mlf_stream_create(ctypes.byref(stream)))
        try:
            if pooled is not None:
                pooled.ensure_total_size(size)
                file_obj = pooled._buffer_io.buffer_obj
            else:
                target = BufferObject(tmp_path, size, overwrite=True)
                file_obj = target
            host = file_obj.get_data_ptr()
            locked = bool(getattr(file_obj, "is_cuda_registered", False))
            token = uuid.uuid4().hex
            _send_msg(conn, {"ok": True, "transport": "nvlink", "token": token, "ipc": landing.ipc_hex, "ptr": landing.ptr,
                             "pid": os.getpid(), "device": self._device, "chunked": True, "slot_bytes": chunk})
            while True:
                note = _recv_msg(conn)
                if note.get("op") == "put_commit":
                    if note.get("token") != token:
                        raise RuntimeError("put was not committed by the sender")
                    break
                if note.get("op") != "chunk":
                    raise RuntimeError(f"unexpected message during a chunked put: {note.get('op')}")
                k, off, n = int(note["k"]), int(note["off"]), int(note["len"])
                if off < 0 or n < 0 or n > chunk or off + n > size:
                    raise RuntimeError("chunk outside the announced object")
                slot = landing.ptr + (k % 2) * chunk
                if locked:
                    _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(host + off), ctypes.c_void_p(slot), n, _native.MLF_COPY_D2H, stream))
                    _native.check(lib.mlf_stream_sync(stream))
                else:
                    _native.check(lib.mlf_bounce_copy(ctypes.c_void_p(slot), ctypes.c_void_p(host + off), n, 0, 0))
                _send_msg(conn, {"op": "slot_free", "k": k})
        except BaseException:
            if target is not None:
                target.close()
                try:
                    os.remove(tmp_path)
                except OSError:
                    pass
            raise
        finally:
            lib.mlf_stream_destroy(stream)
        if pooled is not None:
            self._landing_pool.relink(pooled, tmp_path, final_path)
        else:
            target.close()
            os.rename(tmp_path, final_path)
        _send_msg(conn, {"ok": True})

    def _serve_put_tcp(self, conn: socket.socket, request: dict, size: int, source: int) -> None:
        """Receives the object's bytes from the connection into ``<object>.tmp`` and renames it."""
        from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

        final_path = request["obj"] if request.get("exact_path") else self._map_path(request["obj"], source)
        tmp_path = final_path + ".tmp"
        target = BufferObject(tmp_path, size, overwrite=True)
        try:
            _send_msg(conn, {"ok": True, "transport": "tcp"})
            _recv_into(conn, memoryview(target))
        except BaseException:
            target.close()
            try:
                os.remove(tmp_path)  # never leave a partial object behind
            except OSError:
                pass
            raise
        target.close()
        os.rename(tmp_path, final_path)
        _send_msg(conn, {"ok": True})
