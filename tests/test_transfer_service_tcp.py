"""The transfer service's TCP transport (peers on different hosts, or no GPU), on the CPU.
(``test_transfer_wire_format.py`` checks the bytes on the wire against the reference's format.)

Mirrors the reference's point-to-point service tests: two services on 127.0.0.1, put / get round
trips, temporary file + rename on the receiver, failures surfacing on the future, shutdown failing
what is pending. Failures are made on the host: a dead address, a missing object, a peer that
closes the connection in the middle of an object."""

import os
import socket
import threading

import pytest

from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject


@pytest.fixture
def pair(tmp_path, monkeypatch):
    monkeypatch.setenv("MLFLASHPOINT_REPL_TRANSPORT", "tcp")
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    replicas = str(tmp_path / "replicas")
    a = TransferService()
    b = TransferService(replica_path_mapper=lambda obj, src: os.path.join(replicas, f"src{src}", obj.lstrip("/")))
    assert a.initialize(0, threads=4, global_rank=0) > 0 and b.initialize(0, threads=4, global_rank=1) > 0
    yield a, b, replicas
    a.shutdown()
    b.shutdown()


def _object(path, nbytes, seed):
    import random

    data = random.Random(seed).randbytes(nbytes)
    buf = BufferObject(str(path), nbytes, overwrite=True)
    memoryview(buf)[:] = data
    buf.close()
    return data


@pytest.mark.parametrize("nbytes", [4096, 4096 + 1, 9 << 20])
def test_put_and_get_round_trip_over_tcp(pair, tmp_path, nbytes):
    a, b, replicas = pair
    src = tmp_path / "primary" / "step-1_ckpt" / "o_src0.distcp"
    data = _object(src, nbytes, nbytes)
    ro = BufferObject(str(src))
    result = a.async_put(ro.get_data_ptr(), ro.get_capacity(), b.address, str(src)).result(timeout=60)
    ro.close()
    assert result.success and a.last_put_stats["transport"] == "tcp"
    landed = os.path.join(replicas, "src0", str(src).lstrip("/"))
    assert open(landed, "rb").read() == data and not os.path.exists(landed + ".tmp")
    back = str(tmp_path / "restored.distcp")
    assert a.async_get(str(src), b.address, back).result(timeout=60).success
    assert open(back, "rb").read() == data


def test_failures_and_shutdown(pair, tmp_path):
    a, b, replicas = pair
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        dead = f"127.0.0.1:{s.getsockname()[1]}"
    src = tmp_path / "o.distcp"
    _object(src, 8192, 1)
    ro = BufferObject(str(src))
    with pytest.raises(RuntimeError, match="cannot reach"):
        a.async_put(ro.get_data_ptr(), ro.get_capacity(), dead, str(src)).result(timeout=60)
    with pytest.raises(RuntimeError, match="not held here"):
        a.async_get("/no/such/object", b.address, str(tmp_path / "x")).result(timeout=60)
    with pytest.raises(RuntimeError):
        a.async_put(ro.get_data_ptr(), ro.get_capacity(), "not-an-address", str(src)).result(timeout=60)
    a.shutdown()
    a.shutdown()  # idempotent
    with pytest.raises(RuntimeError, match="not running"):
        a.async_put(ro.get_data_ptr(), ro.get_capacity(), b.address, str(src)).result(timeout=5)
    ro.close()


def test_receiver_discards_a_partial_object(pair, tmp_path):
    """A sender that dies in the middle of an object must not leave a file (or a .tmp) behind."""
    from ml_flashpoint.replication.transfer_service import wire

    _, b, replicas = pair
    host, port = b.address.split(":")
    with socket.create_connection((host, int(port))) as s:
        s.sendall(wire.pack_header(wire.PUT_OBJ, dest_obj_id="/c/step-1_ckpt/o_src5.distcp", obj_size=1 << 20, task_id="t~5"))
        s.sendall(b"x" * 1000)  # then the "host" goes away
    target = os.path.join(replicas, "src5", "c/step-1_ckpt/o_src5.distcp")
    deadline = threading.Event()
    for _ in range(100):
        if os.path.exists(os.path.dirname(target)) and not os.path.exists(target + ".tmp"):
            break
        deadline.wait(0.05)
    assert not os.path.exists(target) and not os.path.exists(target + ".tmp")


def test_every_transfer_logs_the_result_line_the_reference_logs(pair, tmp_path):
    """``TransferService::report_result: task_id=…, task_type=…, data_size=…, success=…, message=…,
    timing=…`` once per finished task, with the reference's phase names, so that log summarisers
    written for the reference service keep working."""
    import logging
    import re

    from ml_flashpoint.replication.transfer_service import transfer_service_ext as mod

    lines = []

    class _Collect(logging.Handler):
        def emit(self, record):
            lines.append(record.getMessage())

    handler = _Collect(level=logging.INFO)
    before = mod._LOGGER.level
    mod._LOGGER.addHandler(handler)
    mod._LOGGER.setLevel(logging.INFO)
    try:
        a, b, replicas = pair
        src = tmp_path / "primary" / "step-1_ckpt" / "o_src0.distcp"
        _object(src, 70000, 3)
        ro = BufferObject(str(src))
        put = a.async_put(ro.get_data_ptr(), ro.get_capacity(), b.address, str(src)).result(timeout=60)
        ro.close()
        got = a.async_get(str(src), b.address, str(tmp_path / "back.distcp")).result(timeout=60)
        with pytest.raises(RuntimeError):
            a.async_get("/no/such/object", b.address, str(tmp_path / "nothing")).result(timeout=60)
    finally:
        mod._LOGGER.removeHandler(handler)
        mod._LOGGER.setLevel(before)
    reports = [l for l in lines if l.startswith("TransferService::report_result:")]
    shape = re.compile(
        r"task_id=(\w+), task_type=(PUT|GET), data_size=(\d+), success=([01]), message=(.*), "
        r"timing=wait_to_be_executed=[\d.]+ms, connection_acquired=[\d.]+ms, header_sent=[\d.]+ms, "
        r"(data_sent|data_received)=[\d.]+ms, total=[\d.]+ms$"
    )
    parsed = [shape.search(l) for l in reports]
    assert all(parsed) and len(parsed) == 3
    by_task = {m.group(1): m for m in parsed}
    assert by_task[put.task_id].group(2, 3, 4) == ("PUT", "70000", "1")
    assert by_task[got.task_id].group(2, 4) == ("GET", "1")
    failed = [m for m in parsed if m.group(4) == "0"]
    assert len(failed) == 1 and "not held here" in failed[0].group(5)


def test_services_that_get_from_each_other_with_every_worker_busy(tmp_path, monkeypatch):
    """Two services with two workers each ask each other for four objects at once: every worker is a
    get waiting for the other side's push. The pushes must not queue behind those workers."""
    monkeypatch.setenv("MLFLASHPOINT_REPL_TRANSPORT", "tcp")
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    a, b = TransferService(), TransferService()
    assert a.initialize(0, threads=2, global_rank=0) > 0 and b.initialize(0, threads=2, global_rank=1) > 0
    try:
        held = {}
        for owner in ("a", "b"):
            for k in range(4):
                path = tmp_path / owner / f"o{k}.distcp"
                os.makedirs(path.parent, exist_ok=True)
                held[(owner, k)] = (str(path), _object(path, 50000 + k, k))
        futures = []
        for k in range(4):
            futures.append((("b", k), a.async_get(held[("b", k)][0], b.address, str(tmp_path / "a_got" / f"o{k}"))))
            futures.append((("a", k), b.async_get(held[("a", k)][0], a.address, str(tmp_path / "b_got" / f"o{k}"))))
        for key, f in futures:
            assert f.result(timeout=60).success
        for k in range(4):
            assert open(tmp_path / "a_got" / f"o{k}", "rb").read() == held[("b", k)][1]
            assert open(tmp_path / "b_got" / f"o{k}", "rb").read() == held[("a", k)][1]
    finally:
        a.shutdown()
        b.shutdown()
