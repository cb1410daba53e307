"""Times the reference's own CPU save / restore path from ``oracle/_ref`` (TEST INFRASTRUCTURE).

Only the benchmark's reference arm, its CPU-baseline leg and the tests may import this module.
``oracle/_ref`` holds the reference package byte-compiled by ``build_ref.py`` (one zip archive of
sourceless ``.pyc`` files); this module makes it importable (two stand-in extension modules, see below) and drives, per emulated rank, exactly what
the reference does for one save of GPU-resident state:

  stage    ``MemoryStorageWriter.stage_write_data_buckets`` (adapter/pytorch/memory_storage_writer.py:211-233):
           ``tensor.to("cpu", non_blocking=True)`` per tensor, one ``torch.cuda.synchronize()``
  write    ``DefaultMLFlashpointCheckpointSaver.prepare_write_data`` -> ``write_data``
           (core/checkpoint_saver.py:362-431, 433-519) with ``thread_count=1`` and the torch thread
           count the reference sets itself (``cpus // 2 // accelerators``), into a
           ``CheckpointObjectManager(BufferPoolConfig(num_buffers=2, buffer_size=16 GiB))`` on tmpfs
           (adapter/nemo/wrapper_util.py:47, 92-97; core/buffer_pool.py:205-247, 297-342), so pages are
           warm from each pool buffer's second use on
  restore  ``DefaultMLFlashpointCheckpointLoader.read_data`` (core/checkpoint_loader.py:298-336) into
           tensors on the device the state came from

Several ranks per host are emulated the way the reference runs them: one process per rank, all
saving at once, each with its own pool and its own device. Every rank is a freshly spawned
interpreter, so the reference's ``ml_flashpoint`` never meets the product package of the same name.

Stand-ins (the compiled extensions need abseil, which is fetched at configure time and is absent):
``BufferObject`` = ``open`` + ``ftruncate`` + ``mmap(MAP_SHARED)`` exactly as
checkpoint_object_manager/buffer_object/buffer_helper.cpp:43-120, 273-314 does it, and an inert
``TransferService`` (replication is not part of this arm).
"""

from __future__ import annotations

import importlib.util
import json
import mmap
import os
import shutil
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_ARCHIVE = os.path.join(REF_DIR, "reference_bytecode.zip")  # sourceless .pyc files, imported by zipimport
POOL_BUFFERS = 2  # NUM_OF_BUFFERS_PER_OBJECT x write_thread_count (adapter/nemo/wrapper_util.py:47, 95)
POOL_BUFFER_BYTES = 16 * 1024**3  # DEFAULT_INITIAL_BUFFER_SIZE_BYTES (core/checkpoint_saver.py)


def unavailable_reason() -> str | None:
    """None when ``oracle/_ref`` can be imported by this interpreter, else why not (one line)."""
    try:
        with open(os.path.join(REF_DIR, "manifest.json")) as f:
            manifest = json.load(f)
    except (OSError, ValueError):
        return "oracle/_ref is not built (run oracle/build_ref.py against a reference checkout)"
    if manifest.get("magic") != importlib.util.MAGIC_NUMBER.hex():
        return f"oracle/_ref was compiled by Python {manifest.get('python')}, not by this interpreter"
    if not os.path.isfile(REF_ARCHIVE):
        return "oracle/_ref holds a manifest but no bytecode archive (rebuild it with oracle/build_ref.py)"
    return None


class _MmapBufferObject:
    """File-backed stand-in for the reference's compiled ``BufferObject`` (same constructor forms,
    methods, properties and error type; 1-D byte buffer protocol)."""

    def __init__(self, object_id, capacity=None, overwrite=False):
        self._id = str(object_id)
        try:
            if capacity is None:
                self._fd = os.open(self._id, os.O_RDONLY)
                size = os.fstat(self._fd).st_size
                if size == 0:
                    os.close(self._fd)
                    raise RuntimeError(f"cannot map zero-sized file {self._id}")
                self._map = mmap.mmap(self._fd, size, flags=mmap.MAP_SHARED, prot=mmap.PROT_READ)
                self._readonly = True
            else:
                if capacity <= 0:
                    raise RuntimeError("capacity must be greater than 0")
                os.makedirs(os.path.dirname(self._id) or ".", exist_ok=True)
                how = os.O_TRUNC if overwrite else os.O_EXCL
                self._fd = os.open(self._id, os.O_CREAT | os.O_RDWR | how, 0o666)
                os.ftruncate(self._fd, capacity)
                self._map = mmap.mmap(self._fd, capacity, flags=mmap.MAP_SHARED, prot=mmap.PROT_READ | mmap.PROT_WRITE)
                self._readonly = False
        except OSError as e:
            raise RuntimeError(f"{type(e).__name__}: {e}") from e
        self._closed = False

    def __buffer__(self, flags):
        view = memoryview(self._map)
        return view.toreadonly() if self._readonly else view

    closed = property(lambda self: self._closed)
    is_readonly = property(lambda self: self._readonly)

    def get_id(self):
        return self._id

    def get_capacity(self):
        return 0 if self._closed else len(self._map)

    def get_data_ptr(self):
        return 0

    def resize(self, new_capacity):
        # unmap, ftruncate, map again (buffer_helper.cpp:273-314); views still exported keep the old mapping alive
        os.ftruncate(self._fd, new_capacity)
        self._map = mmap.mmap(self._fd, new_capacity, flags=mmap.MAP_SHARED, prot=mmap.PROT_READ | mmap.PROT_WRITE)

    def close(self, truncate_size=None):
        if self._closed:
            return
        if truncate_size is not None and not self._readonly:
            os.ftruncate(self._fd, truncate_size)
        os.close(self._fd)
        self._closed = True


def install() -> None:
    """Makes ``import ml_flashpoint`` resolve to the reference build in this process."""
    why = unavailable_reason()
    if why:
        raise RuntimeError(why)
    loaded = sys.modules.get("ml_flashpoint")
    if loaded is not None:
        origin = os.path.dirname(getattr(loaded, "__file__", "") or "")
        if not origin.startswith(REF_ARCHIVE):
            raise RuntimeError(f"another ml_flashpoint package is already imported from {origin}")
        return
    buf = types.ModuleType("ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext")
    buf.BufferObject = _MmapBufferObject
    sys.modules[buf.__name__] = buf
    xfer = types.ModuleType("ml_flashpoint.replication.transfer_service.transfer_service_ext")
    xfer.TransferService = type("TransferService", (), {})
    xfer.TransferResult = type("TransferResult", (), {})
    sys.modules[xfer.__name__] = xfer
    sys.path.insert(0, REF_ARCHIVE)
    os.environ.setdefault("MLFLASHPOINT_LOG_LEVEL", "ERROR")
    import ml_flashpoint

    origin = os.path.dirname(ml_flashpoint.__file__)
    if not origin.startswith(REF_ARCHIVE):
        raise RuntimeError(f"ml_flashpoint resolved to {origin}, not to the reference build")


class RefRank:
    """One rank of a job that checkpoints with the reference implementation."""

    def __init__(self, rank: int, workdir: str, world_size: int = 1):
        install()
        from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter
        from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
        from ml_flashpoint.core.buffer_pool import BufferPoolConfig
        from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
        from ml_flashpoint.core.checkpoint_loader import DefaultMLFlashpointCheckpointLoader
        from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver

        self.rank = rank
        self._container = CheckpointContainerId
        self._stage = MemoryStorageWriter.stage_write_data_buckets
        self.base = os.path.join(workdir, "ref_ckpt")
        self.com = CheckpointObjectManager(
            BufferPoolConfig(
                pool_dir_path=os.path.join(self.base, "buffer_pool"),
                rank=rank,
                num_buffers=POOL_BUFFERS,
                buffer_size=POOL_BUFFER_BYTES,
            )
        )
        self.saver = DefaultMLFlashpointCheckpointSaver(
            global_rank_getter=lambda: rank,
            local_rank_getter=lambda: rank,
            global_barrier_func=lambda: None,
            ckpt_obj_manager=self.com,
            replication_manager=None,
        )
        self.loader = DefaultMLFlashpointCheckpointLoader(
            self.com,
            None,
            global_rank_getter=lambda: rank,
            local_rank_getter=lambda: rank,
            broadcast_object_list_func=lambda *a, **k: None,
            all_gather_object_func=lambda *a, **k: None,
            world_size_getter=lambda: world_size,
        )
        self._step = 0
        self._previous = None
        self.last = None

    def save(self, items, resolver) -> dict:
        """One save: stage to host, then write into a pool buffer. The previous checkpoint is
        deleted afterwards (its pool buffer becomes free), as a retention of one would."""
        ckpt = self._container(os.path.join(self.base, f"step-{self._step}_ckpt"))
        self._step += 1
        t0 = time.perf_counter()
        self.saver.initialize_checkpoint(ckpt)
        buckets = self.saver.prepare_write_data(ckpt, items, resolver, f"__{self.rank}_", bucket_count=1)
        t1 = time.perf_counter()
        staged = self._stage(ckpt, buckets, non_blocking=True)
        t2 = time.perf_counter()
        results = self.saver.write_data(ckpt, staged, replicate_after_write=False, thread_count=1)
        t3 = time.perf_counter()
        del staged
        if self._previous is not None:
            self.com.delete_container(self._previous)
        self._previous = ckpt
        self.last = (ckpt, buckets, results)
        return {"plan_s": t1 - t0, "stage_s": t2 - t1, "write_s": t3 - t2, "total_s": t3 - t0}

    def restore(self, targets: dict) -> float:
        """Reads the last saved object back into ``targets`` (index -> tensor); returns seconds."""
        import torch
        from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

        _, buckets, results = self.last
        storage = {r.index: r.storage_data for r in results}
        reqs = [
            ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * t.dim()), idx, torch.Size([0] * t.dim()), t.shape)
            for idx, t in targets.items()
        ]

        class _Planner:
            def resolve_tensor(self, req):
                return targets[req.dest_index]

            def commit_tensor(self, req, tensor):
                pass

        t0 = time.perf_counter()
        self.loader.read_data(buckets[0].object_id, reqs, _Planner(), storage)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return time.perf_counter() - t0

    def object_path(self) -> str:
        return str(self.last[1][0].object_id)

    def close(self) -> None:
        try:
            self.com.teardown_pool()
        except Exception:
            pass
        shutil.rmtree(self.base, ignore_errors=True)


def _take(shard, budget_bytes: int):
    picked, total = [], 0
    for entry in shard:
        n = entry[1].numel() * entry[1].element_size()
        if total + n > budget_bytes and picked:
            break
        picked.append(entry)
        total += n
    return picked, total


class _Link:
    """Child side of the line-JSON protocol with the coordinating parent (stdin / a dup of stdout)."""

    def __init__(self):
        self._out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)  # whatever else prints goes to stderr; the protocol pipe stays clean
        self._in = sys.stdin

    def send(self, kind: str, **payload) -> None:
        self._out.write(json.dumps({"kind": kind, **payload}) + "\n")
        self._out.flush()

    def recv(self) -> dict:
        line = self._in.readline()
        if not line:
            raise RuntimeError("the coordinating process went away")
        return json.loads(line)

    def barrier(self) -> None:
        self.send("barrier")
        self.recv()


def _rank_main(rank: int, world: int, cfg: dict) -> None:
    """Body of one emulated rank (a process of its own, started by ``run``)."""
    link = _Link()
    try:
        import torch

        root = os.path.dirname(HERE)
        if root not in sys.path:
            sys.path.insert(0, root)
        import bench  # workload definition only; the product package is never imported here

        use_cuda = torch.cuda.is_available() and not cfg.get("force_cpu")
        device = torch.device("cuda", rank % torch.cuda.device_count()) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(device)
        shard = bench.build_shard(rank, device, layers=cfg["layers"])
        full = sum(t.numel() * t.element_size() for _, t, _, _ in shard)
        me = RefRank(rank, cfg["workdir"], world)

        # calibration: a small sample saved until every pool buffer has been used once (warm pages);
        # the last save gives this rank's rate while all ranks save at once
        calib, calib_bytes = _take(shard, min(full, cfg["calib_bytes"]))
        items, resolver = bench.write_items_for(calib)
        rate = 0.0
        for _ in range(POOL_BUFFERS + 1):
            link.barrier()
            rate = calib_bytes / me.save(items, resolver)["total_s"]
        link.send("calib", rate=rate, full=full)
        sample_bytes = link.recv()["sample_bytes"]

        sample, nbytes = _take(shard, sample_bytes)
        items, resolver = bench.write_items_for(sample)
        for _ in range(cfg["warmup"]):
            me.save(items, resolver)
        if use_cuda:
            torch.cuda.synchronize()
        link.barrier()
        t0 = time.perf_counter()
        phases = [me.save(items, resolver) for _ in range(cfg["steps"])]
        if use_cuda:
            torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        link.barrier()

        def median(key):
            return sorted(p[key] * 1e3 for p in phases)[len(phases) // 2]

        accelerators = torch.cuda.device_count() if torch.cuda.is_available() else 0
        out = {
            "rank": rank,
            "bytes_per_step": nbytes,
            "tensors": len(sample),
            "full_bytes": full,
            "elapsed_s": elapsed,
            "stage_ms": median("stage_s"),
            "write_ms": median("write_s"),
            "plan_ms": median("plan_s"),
            # what write_data sets for itself (core/checkpoint_saver.py:443-450)
            "torch_threads": max(1, (os.cpu_count() or 1) // 2 // max(accelerators, 1)),
            "device": str(device),
        }
        if cfg.get("restore", True):
            sources = {wi.index: resolver.resolve_data(wi) for wi in items}
            targets = {idx: torch.empty_like(t) for idx, t in sources.items()}
            me.restore(targets)  # first pass faults the read-only mapping in
            link.barrier()
            out["restore_s"] = me.restore(targets)
            link.barrier()
            out["restore_verified"] = all(torch.equal(targets[i], sources[i]) for i in targets)
        if cfg.get("digest"):
            import hashlib

            h = hashlib.sha256()
            with open(me.object_path(), "rb") as f:
                for block in iter(lambda: f.read(1 << 24), b""):
                    h.update(block)
            out["object_sha256"] = h.hexdigest()
            out["object_size"] = os.path.getsize(me.object_path())
        me.close()
        link.send("result", **out)
    except BaseException as e:  # the parent must hear about it instead of waiting for ever
        import traceback

        link.send("error", text=f"rank {rank}: {type(e).__name__}: {e}\n{traceback.format_exc()}")


def _mem_available_bytes() -> int:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 64 << 30


def run(world: int, steps: int, warmup: int, workdir: str, layers: int = 32, budget_s: float = 150.0,
        max_sample_bytes: int | None = None, restore: bool = True, digest: bool = False, force_cpu: bool = False) -> dict:
    """Runs ``world`` reference ranks at once on this host and returns the aggregate.

    Every rank saves the same number of bytes per step: its whole shard, unless the time budget
    (``budget_s`` for all ``warmup + steps`` saves, judged from a calibration save) or the host's
    memory (two pool buffers on tmpfs plus the pageable staging copy per rank) asks for a prefix.
    """
    import queue
    import subprocess
    import threading

    why = unavailable_reason()
    if why:
        raise RuntimeError(why)
    os.makedirs(workdir, exist_ok=True)
    stat = os.statvfs(workdir)
    host_cap = int(0.6 * min(_mem_available_bytes(), stat.f_bavail * stat.f_frsize) / (world * (POOL_BUFFERS + 1)))
    cfg = {"layers": layers, "steps": steps, "warmup": warmup, "calib_bytes": 1 << 30, "restore": restore,
           "digest": digest, "force_cpu": force_cpu}
    inbox: "queue.Queue" = queue.Queue()
    procs = []

    def pump(r, proc):
        for line in proc.stdout:
            try:
                inbox.put((r, json.loads(line)))
            except ValueError:
                pass
        inbox.put((r, {"kind": "eof"}))

    for r in range(world):
        rank_cfg = dict(cfg, workdir=os.path.join(workdir, f"ref_rank{r}"))
        proc = subprocess.Popen(
            [sys.executable, os.path.abspath(__file__), "--rank", str(r), "--world", str(world), "--cfg", json.dumps(rank_cfg)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1,
        )
        procs.append(proc)
        threading.Thread(target=pump, args=(r, proc), daemon=True).start()

    def tell_all(obj):
        for proc in procs:
            proc.stdin.write(json.dumps(obj) + "\n")
            proc.stdin.flush()

    results, waiting, calib = {}, set(), {}
    by_time = 0
    full = 0
    try:
        while len(results) < world:
            r, msg = inbox.get(timeout=1800)
            kind = msg.get("kind")
            if kind == "error":
                raise RuntimeError(msg["text"])
            if kind == "eof":
                if r not in results:
                    raise RuntimeError(f"reference rank {r} exited early (code {procs[r].poll()})")
            elif kind == "barrier":
                waiting.add(r)
                if len(waiting) == world:
                    waiting.clear()
                    tell_all({"go": True})
            elif kind == "calib":
                calib[r] = msg
                if len(calib) == world:
                    rate = min(m["rate"] for m in calib.values())
                    full = min(m["full"] for m in calib.values())
                    by_time = int(rate * budget_s / max(steps + warmup, 1))
                    tell_all({"sample_bytes": min(full, by_time, host_cap, max_sample_bytes or full)})
            elif kind == "result":
                results[r] = msg
    finally:
        for proc in procs:
            try:
                proc.stdin.close()
            except OSError:
                pass
            try:
                proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                proc.kill()
        shutil.rmtree(workdir, ignore_errors=True)
    results = [results[r] for r in range(world)]

    total_per_step = sum(r["bytes_per_step"] for r in results)
    slowest = max(r["elapsed_s"] for r in results)
    per_rank = results[0]["bytes_per_step"]
    limit = "whole shard" if per_rank >= full else (
        "prefix: time budget" if by_time <= min(host_cap, max_sample_bytes or full) else
        "prefix: host memory" if host_cap <= (max_sample_bytes or full) else "prefix: requested size")
    out = {
        "value": total_per_step * steps / 1e9 / slowest,
        "ms_per_step": slowest / steps * 1e3,
        "bytes_per_step_per_rank": per_rank,
        "full_bytes_per_rank": full,
        "ranks": world,
        "torch_threads_per_rank": results[0]["torch_threads"],
        "cores": results[0]["torch_threads"] * world,
        "host_cpus": os.cpu_count(),
        "blocking_stage_ms": max(r["stage_ms"] for r in results),
        "write_ms": max(r["write_ms"] for r in results),
        "plan_ms": max(r["plan_ms"] for r in results),
        "device": results[0]["device"],
        "sample": (
            f"{limit}: first {results[0]['tensors']} tensors of each rank's shard, {per_rank / 1e9:.2f} of {full / 1e9:.2f} GB per rank per step, "
            f"{world} rank(s) saving at once; reference saver with its buffer pool ({POOL_BUFFERS} x 16 GiB files on tmpfs), "
            f"staged from {results[0]['device']}, thread_count=1, {results[0]['torch_threads']} torch thread(s) per rank"
        ),
    }
    if restore:
        out["restore_value"] = total_per_step / 1e9 / max(r["restore_s"] for r in results)
        out["restore_verified"] = all(r["restore_verified"] for r in results)
    if digest:
        out["objects"] = [{"rank": r["rank"], "sha256": r["object_sha256"], "size": r["object_size"]} for r in results]
    return out


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="one emulated reference rank (started by ref_arm.run)")
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--cfg", required=True)
    a = ap.parse_args()
    _rank_main(a.rank, a.world, json.loads(a.cfg))
