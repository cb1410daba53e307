"""Benchmark of the checkpoint save / restore data path on B200.

One "step" is one full save of a rank's shard of a Llama-3-8B training state (bf16 weights, fp32
master copy, fp32 Adam moments: 2 + 4 + 4 + 4 = 14 bytes per parameter, FSDP-sharded 8 ways on
dimension 0, 14.05 GB per rank) into a memory-backed checkpoint object, followed (outside the save
timing) by a restore of the same object. Every rank saves its own shard with no data-path
collective, so the job scales weakly: ``value`` is the bytes all ranks saved divided by the slowest
rank's time.

    python bench.py --gpus 1 --steps 3 --warmup 3            # this implementation
    python bench.py --impl reference --steps 2 --warmup 1     # the reference's own CPU path (oracle/_ref)
    python bench.py --probe host-link                          # plain pinned copies, fresh process per rank

Prints ONE JSON line on rank 0. Synthetic data only: random-initialised tensors with the shapes,
dtypes and value distributions of the named configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "ml-flashpoint_b200"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

os.environ.setdefault("MLFLASHPOINT_LOG_LEVEL", "WARNING")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "checkpoint_save_throughput"
UNIT = "GB/s"
FSDP_WORLD = 8  # the named configuration shards the model 8 ways whatever --gpus is
# DRAM bytes (read + write) per payload byte of the pack kernel, from an ncu capture of the 2-layer
# variant of this workload (dram__bytes_read.sum + dram__bytes_write.sum = 5.154 GB for 2.602 GB of
# payload); traffic grows in proportion to the payload, so a full launch is this ratio times its payload.
NCU_DRAM_BYTES_PER_PAYLOAD_BYTE = 1.982


# --------------------------------------------------------------------------------------
# Workload: Llama-3-8B training state, one FSDP shard
# --------------------------------------------------------------------------------------
def llama3_8b_params(layers: int = 32):
    d, kv, ff, vocab = 4096, 1024, 14336, 128256
    yield "model.embed_tokens.weight", (vocab, d)
    for i in range(layers):
        p = f"model.layers.{i}."
        yield p + "self_attn.q_proj.weight", (d, d)
        yield p + "self_attn.k_proj.weight", (kv, d)
        yield p + "self_attn.v_proj.weight", (kv, d)
        yield p + "self_attn.o_proj.weight", (d, d)
        yield p + "mlp.gate_proj.weight", (ff, d)
        yield p + "mlp.up_proj.weight", (ff, d)
        yield p + "mlp.down_proj.weight", (d, ff)
        yield p + "input_layernorm.weight", (d,)
        yield p + "post_attention_layernorm.weight", (d,)
    yield "model.norm.weight", (d,)
    yield "lm_head.weight", (vocab, d)


def build_shard(rank: int, device, layers: int = 32, seed: int = 2):
    """This rank's dim-0 shard of every tensor of the training state, as ``(fqn, tensor, offsets, global_shape)``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000 + rank)
    out = []
    for name, shape in llama3_8b_params(layers):
        rows = shape[0] // FSDP_WORLD
        local = (rows,) + tuple(shape[1:])
        offsets = (rank % FSDP_WORLD * rows,) + (0,) * (len(shape) - 1)
        w32 = torch.randn(local, generator=gen, device=device, dtype=torch.float32) * 0.02
        if name.endswith("norm.weight"):
            w32.fill_(1.0)
        out.append((name, w32.to(torch.bfloat16), offsets, shape))
        out.append(("optim.master." + name, w32, offsets, shape))
        m = torch.randn(local, generator=gen, device=device, dtype=torch.float32) * 1e-3
        out.append(("optim.exp_avg." + name, m, offsets, shape))
        v = (torch.randn(local, generator=gen, device=device, dtype=torch.float32) * 1e-3) ** 2
        out.append(("optim.exp_avg_sq." + name, v, offsets, shape))
    return out


def write_items_for(shard):
    from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
    from torch.distributed.checkpoint.planner import TensorWriteData, WriteItem, WriteItemType

    items, lookup = [], {}
    for fqn, tensor, offsets, global_shape in shard:
        idx = MetadataIndex(fqn, torch.Size(offsets))
        items.append(
            WriteItem(
                index=idx,
                type=WriteItemType.SHARD,
                tensor_data=TensorWriteData(
                    chunk=ChunkStorageMetadata(offsets=torch.Size(offsets), sizes=tensor.shape),
                    properties=TensorProperties.create_from_tensor(tensor),
                    size=torch.Size(global_shape),
                ),
            )
        )
        lookup[idx] = tensor

    class _Resolver:
        def resolve_data(self, write_item):
            return lookup[write_item.index]

    return items, _Resolver()


# --------------------------------------------------------------------------------------
# Clock sampling during the timed region
# --------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.rows = []
        self._proc = None
        self._gpu = gpu_index

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self._gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL,
                text=True,
            )
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self._proc = None

    def _pump(self):
        for line in self._proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 7:
                continue
            try:
                sm.append(float(row[0]))
                smax = float(row[1])
            except ValueError:
                continue
            for name, cell in zip(names, row[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": smax,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)"


# --------------------------------------------------------------------------------------
# Distributed helpers
# --------------------------------------------------------------------------------------
def world():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def _collective_device(device):
    return torch.device("cpu") if dist.get_backend() == "gloo" else device


def all_max(value: float, device) -> float:
    if not dist.is_initialized():
        return value
    t = torch.tensor([value], dtype=torch.float64, device=_collective_device(device))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_sum(value: float, device) -> float:
    if not dist.is_initialized():
        return value
    t = torch.tensor([value], dtype=torch.float64, device=_collective_device(device))
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def barrier():
    if dist.is_initialized():
        dist.barrier()


# --------------------------------------------------------------------------------------
# Host-link calibration: what a plain pinned copy reaches while all ranks copy at once
# --------------------------------------------------------------------------------------
def calibrate_host_link(device, nbytes: int = 2 << 30) -> dict:
    """Copy-engine D2H and H2D between HBM and driver-allocated pinned memory, all ranks at the
    same time: the denominator for the save's drain and the restore's feed at this GPU count."""
    dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
    host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    out = {}
    for name, dst, src in (("d2h", host, dev), ("h2d", dev, host)):
        best = 0.0
        for _ in range(3):
            barrier()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            dst.copy_(src, non_blocking=True)
            t1.record()
            torch.cuda.synchronize()
            best = max(best, nbytes / 1e9 / (t0.elapsed_time(t1) / 1e3))
        out[name] = -all_max(-best, device)  # the slowest rank's best
    del dev, host
    return out


# --------------------------------------------------------------------------------------
# CPU baseline: the reference's own saver / loader (oracle/_ref driven by oracle/ref_arm.py),
# or, where that build is absent, its restatement in oracle/cpu_path.py
# --------------------------------------------------------------------------------------
def cpu_sample(shard, budget_bytes: int):
    picked, total = [], 0
    for _, tensor, _, _ in shard:
        n = tensor.numel() * tensor.element_size()
        if total + n > budget_bytes and picked:
            break
        picked.append(tensor)
        total += n
    return picked, total


def reference_arm_unavailable():
    """None when the byte-compiled reference under oracle/_ref can run here, else the reason."""
    import ref_arm

    return ref_arm.unavailable_reason()


def run_reference_ranks(world_size: int, steps: int, warmup: int, workdir: str, layers: int, budget_s: float,
                        digest: bool = False, max_sample_bytes=None) -> dict:
    """``world_size`` ranks of the reference implementation saving at once on this host's cores
    (one fresh process per rank; see oracle/ref_arm.py). Returns the aggregate as a cpu_baseline dict."""
    import ref_arm

    r = ref_arm.run(world_size, steps, warmup, os.path.join(workdir, "reference_arm"), layers=layers,
                    budget_s=budget_s, digest=digest, max_sample_bytes=max_sample_bytes)
    out = {
        "value": r["value"],
        "unit": UNIT,
        "cores": r["cores"],
        "host_cpus": r["host_cpus"],
        "kind": "reference",
        "sample": r["sample"],
        "ranks": r["ranks"],
        "ms_per_step": r["ms_per_step"],
        "bytes_per_step_per_rank": r["bytes_per_step_per_rank"],
        "whole_shard": r["bytes_per_step_per_rank"] >= r["full_bytes_per_rank"],
        "blocking_stage_ms": r["blocking_stage_ms"],
        "write_ms": r["write_ms"],
        "restore_value": r.get("restore_value"),
        "restore_verified": r.get("restore_verified"),
    }
    if digest:
        out["objects"] = r["objects"]
    return out


def run_cpu_port(shard, workdir: str, budget_bytes: int, passes: int, ranks_on_host: int = 1) -> dict:
    """Fallback CPU baseline where oracle/_ref is absent: the restated host path of oracle/cpu_path.py
    (no buffer pool, one rank)."""
    import cpu_path

    tensors, nbytes = cpu_sample(shard, budget_bytes)
    path = os.path.join(workdir, "cpu_baseline.distcp")
    times = []
    stage = []
    cpu_path.timed_save(tensors, path, ranks_on_host)  # warm pages
    for _ in range(passes):
        r = cpu_path.timed_save(tensors, path, ranks_on_host)
        times.append(r["total_s"])
        stage.append(r["stage_s"])
    records = r["records"]
    targets = [torch.empty_like(t) for t in tensors]
    t0 = time.perf_counter()
    cpu_path.read_object(path, records, targets)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    restore_s = time.perf_counter() - t0
    ok = all(torch.equal(a, b) for a, b in zip(tensors, targets))
    os.remove(path)
    best = min(times)
    return {
        "value": nbytes / 1e9 / best,
        "unit": UNIT,
        "cores": cpu_path.reference_thread_count(ranks_on_host),
        "host_cpus": os.cpu_count(),
        "kind": "port",
        "sample": f"first {len(tensors)} tensors of the shard, {nbytes / 1e9:.2f} GB, GPU-sourced: stage to pageable host memory + copy_ into a fresh tmpfs mapping (no buffer pool); best of {passes} passes",
        "blocking_stage_ms": min(stage) * 1e3,
        "restore_value": nbytes / 1e9 / restore_s,
        "restore_verified": bool(ok),
    }


# --------------------------------------------------------------------------------------
# Main
# --------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="mlf_b200", choices=["mlf_b200", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="transformer layers in the synthetic state (32 = the named config)")
    ap.add_argument("--mode", default=None, choices=[None, "staged", "direct"], help="pack destination (default: staged)")
    ap.add_argument("--arena-limit-gb", type=float, default=0.0,
                    help="bound the HBM image arena (0 = hold the whole save): larger saves go through it piece by piece")
    ap.add_argument("--landing-chunk-mb", type=float, default=0.0,
                    help="replication: receive through a two-slot landing ring of this many MiB per slot (0 = whole-object landing buffer)")
    ap.add_argument("--no-restore", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-replication", action="store_true")
    ap.add_argument("--no-overlap-probe", action="store_true")
    ap.add_argument("--cpu-sample-gb", type=float, default=2.0, help="sample of the fallback CPU port (only without oracle/_ref)")
    ap.add_argument("--ref-budget-s", type=float, default=150.0, help="time budget of the reference arm's warm-up + timed saves")
    ap.add_argument("--cpu-baseline-budget-s", type=float, default=20.0, help="time budget of the CPU-baseline leg's saves")
    ap.add_argument("--workdir", default=None)
    ap.add_argument("--share-gpu", action="store_true", help="debug aid: all ranks use cuda:0 and gloo collectives")
    ap.add_argument("--probe", default=None, choices=[None, "host-link", "transpose", "footprint", "d2h-targets"],
                    help="host-link: plain copies between HBM and driver-allocated pinned memory in a process that "
                    "holds nothing else, rank by rank and all ranks at once; transpose: kernel-only pack / unpack "
                    "timing of transposed views through the C ABI; footprint: the pack kernel and the driver's own "
                    "device-to-device copy on flat buffers of 1 to 12 GiB; d2h-targets: the device-to-host copy of a shard-sized "
                    "buffer into driver-allocated pinned memory and into a page-locked tmpfs file, all ranks at once; each "
                    "prints one JSON line and exits")
    ap.add_argument("--probe-target-gb", type=float, default=14.0, help="d2h-targets probe: size of the large targets")
    ap.add_argument("--probe-case", default=None, help="transpose probe: run only the case with this name")
    ap.add_argument("--probe-feed-only", action="store_true", help="host-link probe: only the restore-feed part")
    ap.add_argument("--probe-idle-ms", type=float, default=0.0,
                    help="transpose probe: leave the GPU idle this long before every timed launch (a save's pack kernel "
                    "starts after the previous object's host transfer, with the SMs idle)")
    ap.add_argument("--probe-alone-ranks", default=None,
                    help="host-link probe: comma-separated ranks measured one at a time (default: every rank)")
    args = ap.parse_args()
    if args.probe == "host-link":
        run_host_link_probe(args)
        return
    if args.probe == "transpose":
        run_transpose_probe(args)
        return
    if args.probe == "footprint":
        run_footprint_probe(args)
        return
    if args.probe == "d2h-targets":
        run_d2h_targets_probe(args)
        return
    if args.impl == "mlf_b200":
        args.warmup = max(args.warmup, 3)  # fewer warm-up saves would time plan creation and buffer sizing

    rank, local_rank, world_size = world()
    if world_size > 1:
        if args.impl == "reference" and rank != 0:
            return  # the CPU arm runs on rank 0 alone
        if args.impl != "reference" and args.share_gpu:
            local_rank = 0
            dist.init_process_group("gloo")
        elif args.impl != "reference":
            torch.cuda.set_device(local_rank)
            import datetime

            # a rank that fails must not leave the others waiting for the default 10 minutes
            dist.init_process_group(
                "nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=240)
            )
    if torch.cuda.is_available():
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
    elif args.impl == "reference":
        device = torch.device("cpu")  # the CPU arm also runs where there is no GPU (nothing to stage then)
    else:
        raise SystemExit("bench.py needs a CUDA device: this implementation has no CPU data path")

    shm_root = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
    workdir = args.workdir or os.path.join(shm_root, f"mlf_bench_{os.getuid()}", f"rank{rank}")
    shutil.rmtree(workdir, ignore_errors=True)
    os.makedirs(workdir, exist_ok=True)
    try:
        if args.impl == "reference":
            run_reference_arm(args, device, workdir)
        else:
            run_native_arm(args, rank, world_size, device, workdir)
    except BaseException:
        # a failed rank must exit at once so that the launcher stops the others instead of letting
        # them wait in a collective
        import traceback

        traceback.print_exc()
        shutil.rmtree(workdir, ignore_errors=True)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)
    shutil.rmtree(workdir, ignore_errors=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def run_reference_arm(args, device, workdir: str) -> None:
    """The reference's own CPU implementation of the save, on this host's cores: ``--gpus`` ranks
    saving at once, each a process of its own with its own buffer pool, staged from its own GPU,
    as the reference runs them (rank 0 of the launch drives all of them and prints the line)."""
    world_size = max(1, args.gpus)
    payload_full = shard_payload_bytes(args.layers)
    why = reference_arm_unavailable()
    if why is None:
        cpu = run_reference_ranks(world_size, args.steps, max(args.warmup, 2), workdir, args.layers, args.ref_budget_s)
        value, ms_per_step = cpu["value"], cpu["ms_per_step"]
        warmup = max(args.warmup, 2)
    else:
        # no oracle/_ref on this machine: the restated host path, one rank, bounded sample
        import cpu_path

        shard = build_shard(0, device, layers=args.layers)
        tensors, nbytes = cpu_sample(shard, int(args.cpu_sample_gb * 1e9))
        path = os.path.join(workdir, "reference.distcp")
        warmup = max(args.warmup, 1)
        for _ in range(warmup):
            cpu_path.timed_save(tensors, path)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        stage_ms = [cpu_path.timed_save(tensors, path)["stage_s"] * 1e3 for _ in range(args.steps)]
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        value, ms_per_step = nbytes * args.steps / 1e9 / elapsed, elapsed / args.steps * 1e3
        cpu = {
            "value": value,
            "unit": UNIT,
            "cores": cpu_path.reference_thread_count(1),
            "host_cpus": os.cpu_count(),
            "kind": "port",
            "sample": f"{why}; restated host path instead: first {len(tensors)} tensors of one rank's shard "
            f"({nbytes / 1e9:.2f} of {payload_full / 1e9:.2f} GB) per step, one rank, no buffer pool",
            "blocking_stage_ms": statistics.median(stage_ms),
        }
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "u8",
        "data": "synthetic",
        "config": workload_config(args, payload_full),
        "per_gpu_value": value / world_size if cpu["kind"] == "reference" else value,
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_transpose_probe(args) -> None:
    """Kernel-only throughput of transposed views, pack and unpack, through the C ABI (one plan, one
    launch per direction, CUDA events, L2 flushed between launches), each result checked against
    torch. Read + write bytes per second. ``MLF_TRANSPOSE_FORM`` selects the form of wide pack
    transposes (matrix | vector | element)."""
    from ml_flashpoint import _native
    from ml_flashpoint.core.gpu_engine import _Plan, c_strides, fill_desc

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    gen = torch.Generator(device=device).manual_seed(7)

    def rnd(shape, dtype):
        if dtype in (torch.int64, torch.uint8):
            return torch.randint(0, 250, shape, dtype=dtype, device=device, generator=gen)
        return torch.randn(shape, device=device, generator=gen).to(dtype)

    def run(views):
        n = len(views)
        descs = (_native.CopyDesc * n)()
        offsets, at = [], 7
        for v in views:
            offsets.append(at)
            at += v.numel() * v.element_size() + 137
        image = torch.zeros(at + 64, dtype=torch.uint8, device=device)
        stream = torch.cuda.current_stream().cuda_stream
        rates = {}
        for direction in ("pack", "unpack"):
            if direction == "pack":
                ends = views
            else:
                ends = [torch.zeros_like(v._base if v._base is not None else v).as_strided(v.shape, v.stride(), v.storage_offset()) for v in views]
            for i, t in enumerate(ends):
                fill_desc(descs[i], t.data_ptr(), offsets[i], t.element_size(), t.shape, t.stride(), c_strides(t.shape))
            plan = _Plan(descs, n, _native.MLF_PACK if direction == "pack" else _native.MLF_UNPACK)
            times = []
            for it in range(5):
                flush.fill_(it)
                if args.probe_idle_ms > 0:
                    torch.cuda.synchronize()
                    time.sleep(args.probe_idle_ms / 1e3)
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                plan.launch(image.data_ptr(), image.numel(), stream)
                t1.record()
                torch.cuda.synchronize()
                plan.status()
                times.append(t0.elapsed_time(t1))
            ms = sorted(times[1:])[len(times[1:]) // 2]
            rates[direction] = 2 * plan.payload / 1e9 / (ms / 1e3)
            for v, t, o in zip(views, ends, offsets):
                if direction == "pack":
                    nbytes = v.numel() * v.element_size()
                    assert torch.equal(image[o : o + nbytes], v.contiguous().reshape(-1).view(torch.uint8)), "pack differs from torch"
                else:
                    assert torch.equal(t, v), "unpack differs from torch"
        return {"payload_mb": round(sum(v.numel() * v.element_size() for v in views) / 1e6, 1),
                "pack_gbs": round(rates["pack"]), "unpack_gbs": round(rates["unpack"])}

    def microbench_views(kind):
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import workloads

        tensors = list(workloads.packing_microbench(device).values())
        transposed = [t for t in tensors if not t.is_contiguous()]
        if kind == "wide":
            return [t for t in transposed if t.shape[-1] * t.element_size() >= 256]
        return transposed if kind == "transposed" else tensors

    cases = {
        "flat_bf16_1gib": lambda: [rnd((512 << 20,), torch.bfloat16)],
        # the same flat tensor beside one small transposed view: the plan then runs as mlf_plan_kernel_bulk
        "flat_bf16_1gib_in_a_bulk_plan": lambda: [rnd((512 << 20,), torch.bfloat16), rnd((64, 64), torch.bfloat16).t()],
        "uint8_square": lambda: [rnd((16384, 16384), torch.uint8).t()],
        "bf16_square_odd_pitch": lambda: [rnd((11585, 11585), torch.bfloat16).t()],
        "bf16_square_word_pitch": lambda: [rnd((11586, 11586), torch.bfloat16).t()],
        "fp32_square": lambda: [rnd((8192, 8192), torch.float32).t()],
        "fp32_square_odd_pitch": lambda: [rnd((8191, 8191), torch.float32).t()],
        "int64_square": lambda: [rnd((5792, 5792), torch.int64).t()],
        "bf16_weight_14336x4096": lambda: [rnd((14336, 4096), torch.bfloat16).t()],
        "bf16_weight_28672x8192": lambda: [rnd((28672, 8192), torch.bfloat16).t()],
        "fp32_weight_4096x14336": lambda: [rnd((4096, 14336), torch.float32).t()],
        "bf16_batched_64x1000x300": lambda: [rnd((64, 1000, 300), torch.bfloat16).mT],
        # narrow rows: image rows shorter than 256 bytes lying back to back
        "narrow_bf16_rows_of_2": lambda: [rnd((2, 32 << 20), torch.bfloat16).t()],
        "narrow_bf16_rows_of_3": lambda: [rnd((3, 21 << 20), torch.bfloat16).t()],
        "narrow_bf16_rows_of_8": lambda: [rnd((8, 8 << 20), torch.bfloat16).t()],
        "narrow_bf16_rows_of_82": lambda: [rnd((82, 800000), torch.bfloat16).t()],
        "narrow_fp32_rows_of_3": lambda: [rnd((3, 10 << 20), torch.float32).t()],
        "narrow_fp32_rows_of_19": lambda: [rnd((19, 1600000), torch.float32).t()],
        "narrow_int64_rows_of_12": lambda: [rnd((12, 1300000), torch.int64).t()],
        # the benchmark's own shard (1 164 contiguous tensors, 14.05 GB) through one plan and one launch
        "llama3_8b_shard": lambda: [t for _, t, _, _ in build_shard(0, device)],
        "microbench_transposed_wide_rows": lambda: microbench_views("wide"),
        "microbench_transposed_all": lambda: microbench_views("transposed"),
        "microbench_all_1024_tensors": lambda: microbench_views("all"),
    }
    results = {}
    for name, make in cases.items():
        if args.probe_case and name != args.probe_case:
            continue
        results[name] = run(make())
        torch.cuda.empty_cache()
    if args.probe_case == "microbench_each":  # every transposed view of the microbench of 8 MB or more, alone
        for v in microbench_views("transposed"):
            if v.numel() * v.element_size() >= (8 << 20):
                key = f"{str(v.dtype).split('.')[-1]} shape {tuple(v.shape)} stride {tuple(v.stride())}"
                copies = max(1, (256 << 20) // (v.numel() * v.element_size()))  # enough of them to outweigh the launch
                results[key] = run([v._base.clone().as_strided(v.shape, v.stride(), v.storage_offset()) for _ in range(copies)])
                torch.cuda.empty_cache()
    print(json.dumps({"probe": "transpose", "form": os.environ.get("MLF_TRANSPOSE_FORM", "matrix"),
                      "unit": "GB/s of read + write bytes, kernel only, median of 4 launches", "results": results}))


def run_footprint_probe(args) -> None:
    """HBM copy rate against the size of the buffers: one flat tensor packed by ``mlf_plan_kernel_stream``
    (one plan, one launch) beside the driver's device-to-device copy of the same bytes, for 1, 4 and
    12 GiB, image and tensor aligned to one another and 7 bytes apart. CUDA events, L2 flushed between launches, median of 4. Read + write bytes per second.
    Shows how much of the distance between a 14 GB shard and the copy peak measured on a small
    buffer belongs to the footprint and how much to the kernel."""
    from ml_flashpoint import _native
    from ml_flashpoint.core.gpu_engine import _Plan, c_strides, fill_desc

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    results = {}
    for gib, offset in ((1, 0), (4, 0), (12, 0), (4, 7), (12, 7)):
        nbytes = gib << 30
        src = torch.empty(nbytes, dtype=torch.uint8, device=device)
        src.random_(0, 255)
        image = torch.zeros(nbytes + 64, dtype=torch.uint8, device=device)
        descs = (_native.CopyDesc * 1)()
        fill_desc(descs[0], src.data_ptr(), offset, 1, src.shape, src.stride(), c_strides(src.shape))
        plan = _Plan(descs, 1, _native.MLF_PACK)

        def timed(fn):
            times = []
            for it in range(5):
                flush.fill_(it)
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                fn()
                t1.record()
                torch.cuda.synchronize()
                times.append(t0.elapsed_time(t1))
            return sorted(times[1:])[2]

        pack_ms = timed(lambda: plan.launch(image.data_ptr(), image.numel(), stream))
        plan.status()
        assert torch.equal(image[offset : offset + nbytes], src), "pack differs from the source"
        image.zero_()
        copy_ms = timed(lambda: image[offset : offset + nbytes].copy_(src))
        results[f"flat_{gib}gib_image_offset_{offset}"] = {
            "pack_kernel_gbs": round(2 * nbytes / 1e9 / (pack_ms / 1e3)),
            "driver_d2d_copy_gbs": round(2 * nbytes / 1e9 / (copy_ms / 1e3)),
        }
        del plan, src, image
        torch.cuda.empty_cache()
    print(json.dumps({"probe": "footprint", "unit": "GB/s of read + write bytes, median of 4 launches", "results": results}))


def run_d2h_targets_probe(args) -> None:
    """Device-to-host copy rate against what the host side of the copy is, in a fresh process per
    rank, all ranks at once: (a) the 2 GiB driver-allocated pinned buffer of the host-link probe,
    (b) a driver-allocated pinned buffer the size of a shard, (c) a tmpfs file of that size created and
    page-locked the way the buffer pool does it (``BufferObject.register_cuda``), written by the same
    ``mlf_memcpy_async`` a save uses, and (a) again while (b) and (c) still exist. Separates a limit of
    the host's inbound-write path from a cost of large or file-backed page-locked targets."""
    import ctypes

    from ml_flashpoint import _native
    from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

    rank, local_rank, world_size = world()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world_size > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _native.lib()
    small = 2 << 30
    large = int(args.probe_target_gb * (1 << 30)) // 4096 * 4096
    dev = torch.empty(large, dtype=torch.uint8, device=device)
    dev.random_(0, 255)
    stream = torch.cuda.Stream()
    raw = ctypes.c_void_p(stream.cuda_stream)

    def d2h(host_ptr, nbytes, reps):
        best = 0.0
        for _ in range(reps):
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record(stream)
            _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(host_ptr), ctypes.c_void_p(dev.data_ptr()), nbytes, _native.MLF_COPY_D2H, raw))
            t1.record(stream)
            stream.synchronize()
            best = max(best, nbytes / 1e9 / (t0.elapsed_time(t1) / 1e3))
        return best

    rates, seconds = {}, {}
    host_small = ctypes.c_void_p()
    _native.check(lib.mlf_host_alloc(small, ctypes.byref(host_small)))
    ctypes.memset(host_small, 1, small)
    d2h(host_small.value, small, 1)
    rates["pinned_2gib"] = d2h(host_small.value, small, 3)

    t = time.perf_counter()
    host_large = ctypes.c_void_p()
    _native.check(lib.mlf_host_alloc(large, ctypes.byref(host_large)))
    seconds["alloc_pinned_large"] = time.perf_counter() - t
    d2h(host_large.value, large, 1)  # first touch
    rates["pinned_large"] = d2h(host_large.value, large, 2)

    shm_root = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
    path = os.path.join(shm_root, f"mlf_probe_target_{os.getuid()}_{rank}.bin")
    file_obj = None
    try:
        t = time.perf_counter()
        file_obj = BufferObject(path, large, overwrite=True)
        file_obj.register_cuda()
        seconds["create_and_lock_tmpfs_file"] = time.perf_counter() - t
        d2h(file_obj.get_data_ptr(), large, 1)
        rates["locked_tmpfs_file_large"] = d2h(file_obj.get_data_ptr(), large, 2)
        rates["pinned_2gib_again"] = d2h(host_small.value, small, 3)
    finally:
        if file_obj is not None:
            file_obj.close()
        if os.path.exists(path):
            os.remove(path)
    lib.mlf_host_free(host_large)
    lib.mlf_host_free(host_small)
    gathered = [None] * world_size
    if world_size > 1:
        dist.all_gather_object(gathered, (rates, seconds))
    else:
        gathered = [(rates, seconds)]
    if rank == 0:
        out = {
            "probe": "d2h-targets", "n_gpus": world_size, "large_bytes": large, "host_cpus": os.cpu_count(),
            "what": "cudaMemcpyAsync device to host, all ranks at once, fresh process per rank, best of the repetitions, GB/s per rank",
            "results": {k: [round(g[0][k], 2) for g in gathered] for k in rates},
            "aggregate_gbs": {k: round(sum(g[0][k] for g in gathered), 1) for k in rates},
            "setup_seconds_rank0": {k: round(v, 2) for k, v in seconds.items()},
        }
        print(json.dumps(out))
    if world_size > 1:
        barrier()
        dist.destroy_process_group()


def run_host_link_probe(args) -> None:
    """What the host link gives this set of GPUs, measured with nothing else in the process: no
    pool files, no page-locked tmpfs, no arena. Per rank: copy-engine D2H and H2D between HBM and
    ``cudaHostAlloc`` memory, and the copy kernel storing into / loading from the same memory
    (``mlf_copy_kernel_launch``), first one rank at a time (the others idle), then all ranks at once.
    Tells a limit of the host apart from a cost of this library's own registered mappings."""
    import ctypes

    from ml_flashpoint import _native

    rank, local_rank, world_size = world()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world_size > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _native.lib()
    nbytes = 2 << 30
    host = ctypes.c_void_p()
    _native.check(lib.mlf_host_alloc(nbytes, ctypes.byref(host)))
    ctypes.memset(host, 1, nbytes)
    dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
    stream = torch.cuda.Stream()
    raw = ctypes.c_void_p(stream.cuda_stream)

    def timed(fn, reps=3, lockstep=False):
        best = 0.0
        for _ in range(reps):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if lockstep:
                barrier()  # every repetition starts on all ranks together: ranks that drift apart would overstate a shared ceiling
            t0.record(stream)
            fn()
            t1.record(stream)
            stream.synchronize()
            best = max(best, nbytes / 1e9 / (t0.elapsed_time(t1) / 1e3))
        return best

    ops = {
        "copy_engine_d2h": lambda: _native.check(lib.mlf_memcpy_async(host, ctypes.c_void_p(dev.data_ptr()), nbytes, _native.MLF_COPY_D2H, raw)),
        "copy_engine_h2d": lambda: _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(dev.data_ptr()), host, nbytes, _native.MLF_COPY_H2D, raw)),
        "kernel_store_to_host": lambda: _native.check(lib.mlf_copy_kernel_launch(host, ctypes.c_void_p(dev.data_ptr()), nbytes, raw, 32)),
        "kernel_load_from_host": lambda: _native.check(lib.mlf_copy_kernel_launch(ctypes.c_void_p(dev.data_ptr()), host, nbytes, raw, 32)),
    }
    for fn in ops.values():  # warm-up: first touch of the pinned pages by the device, kernel load
        fn()
    torch.cuda.synchronize()
    alone_ranks = (
        list(range(world_size)) if not args.probe_alone_ranks else [int(r) for r in args.probe_alone_ranks.split(",") if r != ""]
    )
    result = {}
    for name, fn in ({} if args.probe_feed_only else ops).items():
        alone = 0.0
        for turn in alone_ranks:  # one rank at a time
            barrier()
            if turn == rank:
                alone = timed(fn)
            barrier()
        barrier()
        together = timed(fn, lockstep=True)  # everybody at once
        barrier()
        gathered = [None] * world_size
        if world_size > 1:
            dist.all_gather_object(gathered, (alone, together))
        else:
            gathered = [(alone, together)]
        result[name] = {
            "alone_gbs_per_rank": [round(a, 2) for a, _ in gathered],
            "all_at_once_gbs_per_rank": [round(t, 2) for _, t in gathered],
            "all_at_once_aggregate_gbs": round(sum(t for _, t in gathered), 2),
        }
    lib.mlf_host_free(host)

    # ---- the restore feed: an object file on tmpfs, opened read-only by a process that has never
    # seen it (nothing page-locked), into HBM: pread() threads through the bounce ring, the same with
    # the lock lane beside them, and the lock lane alone
    from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject
    from ml_flashpoint.core.gpu_engine import default_host_threads

    shm_root = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
    path = os.path.join(shm_root, f"mlf_probe_{os.getuid()}_{rank}.bin")
    file_bytes = 4 << 30
    with open(path, "wb") as f:
        block = bytes(bytearray(os.urandom(1 << 20)) * 16)
        for _ in range(file_bytes // len(block)):
            f.write(block)
    big = torch.empty(file_bytes, dtype=torch.uint8, device=device)
    threads = default_host_threads(1.0)  # what a restore uses: all cores, divided between the ranks of the host
    feeds = {
        "pread_threads": (threads, 0),
        "pread_threads_plus_lock_lane": (threads, 256),
        "lock_lane_alone": (-1, 256),
    }
    if args.probe_feed_only:
        feeds = {"pread_threads": (threads, 0)}

    def feed_once(nthreads, run_mib):
        obj = BufferObject(path)  # a fresh read-only mapping each time
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        lane = obj.read_to_device(0, big.data_ptr(), file_bytes, threads=nthreads, lock_run_mib=run_mib)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        obj.close()
        return file_bytes / 1e9 / dt, lane

    feed_result = {}
    try:
        feed_once(threads, 0)  # warm-up: ring slots, streams
        for name, (nthreads, run_mib) in feeds.items():
            alone, lane_share = 0.0, 0.0
            for turn in alone_ranks:
                barrier()
                if turn == rank:
                    alone, lane_bytes = feed_once(nthreads, run_mib)
                    lane_share = lane_bytes / file_bytes
                barrier()
            barrier()
            together, _ = feed_once(nthreads, run_mib)
            barrier()
            gathered = [None] * world_size
            if world_size > 1:
                dist.all_gather_object(gathered, (alone, together, lane_share))
            else:
                gathered = [(alone, together, lane_share)]
            feed_result[name] = {
                "alone_gbs_per_rank": [round(a, 2) for a, _, _ in gathered],
                "all_at_once_gbs_per_rank": [round(t, 2) for _, t, _ in gathered],
                "all_at_once_aggregate_gbs": round(sum(t for _, t, _ in gathered), 2),
                "lane_share_alone": [round(s, 3) for _, _, s in gathered],
                "pread_threads_per_rank": threads if nthreads > 0 else 0,
            }
    finally:
        os.remove(path)
    result["restore_feed"] = {
        "what": "4 GiB object file on tmpfs opened read-only into HBM (wall clock of the blocking call), page cache warm",
        "bounce_chunk_kib": int(os.environ.get("MLF_BOUNCE_CHUNK_KIB", "0") or 0)
        or max(1024, 4096 // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1") or 1))),
        **feed_result,
    }
    if rank == 0:
        print(json.dumps({
            "probe": "host-link",
            "n_gpus": world_size,
            "visible_devices": os.environ.get("CUDA_VISIBLE_DEVICES"),
            "bytes_per_copy": nbytes,
            "host_cpus": os.cpu_count(),
            "what": "fresh process per rank, nothing else page-locked; best of 3 per figure, CUDA events",
            "results": result,
        }))
    if dist.is_initialized():
        dist.destroy_process_group()


def shard_payload_bytes(layers: int = 32) -> int:
    """Payload bytes of one rank's shard (14 bytes per parameter), from the shapes alone."""
    total = 0
    for _, shape in llama3_8b_params(layers):
        numel = shape[0] // FSDP_WORLD
        for d in shape[1:]:
            numel *= d
        total += numel * 14
    return total


def workload_config(args, payload_bytes: int) -> dict:
    return {
        "workload": f"Llama-3-8B bf16 weights + fp32 master + fp32 Adam moments, FSDP dim-0 shard 1/{FSDP_WORLD} per rank"
        + ("" if args.layers == 32 else f" (reduced to {args.layers} layers)"),
        "payload_bytes_per_rank": payload_bytes,
        "pack_mode": args.mode or "staged",
        "arena_limit_bytes": int(getattr(args, "arena_limit_gb", 0.0) * (1 << 30)),
        "cache": "inputs larger than L2 (14.05 GB per rank vs 126 MB)",
        "objects_per_rank": 1,
    }


def file_sha256(path: str) -> str:
    import hashlib

    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 24), b""):
            h.update(block)
    return h.hexdigest()


def run_replication(args, rank, world_size, device, workdir, com, engine, items, resolver, shard, state):
    """Replicates every rank's object to rank (r + 1) mod N, all ranks at once, two ways:

    * ``after_save``: the object is saved first, then ``ReplicationManager.async_replicate`` is timed
      alone (object in the partner's file when the future resolves);
    * ``with_save``: ``write_data_async(replicate_after_write=True)``: the push over NVLink is queued
      with the pack kernel and reads the HBM image while the copy engine drains it to the host.

    Uses the full object when /dev/shm can hold a second copy per rank, otherwise a prefix of the
    shard saved as an object of its own (and says so). After the last round every rank hashes the
    replica it received and compares it with the digest of the sender's primary object."""
    from ml_flashpoint.core.buffer_pool import BufferPool
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver
    from ml_flashpoint.replication import replication_manager as rm
    from ml_flashpoint.replication.transfer_service.transfer_service_ext import TransferService

    replica_root = os.path.join(workdir, "replicas")

    def mapper(object_id, source_rank):
        return os.path.join(replica_root, f"src{source_rank}", object_id.lstrip("/"))

    # how much may be replicated: every rank lands one more copy in the shared tmpfs
    stat = os.statvfs(workdir)
    free = stat.f_bavail * stat.f_frsize
    full = sum(t.numel() * t.element_size() for _, t, _, _ in shard)
    budget = int(0.8 * free / world_size)

    # replicas land in a page-locked pool file of their own, like primaries do
    landing_pool = BufferPool(os.path.join(workdir, "replica_pool"), rank, 1, min(full, budget) + (1 << 20), register_cuda=True)
    service = TransferService(replica_path_mapper=mapper, landing_pool=landing_pool,
                              landing_chunk_bytes=int(args.landing_chunk_mb * (1 << 20)))
    if service.initialize(0, threads=4, global_rank=rank) <= 0:
        raise RuntimeError("transfer service failed to start")
    addresses = [None] * world_size
    dist.all_gather_object(addresses, service.address)
    manager = rm.ReplicationManager()
    manager.initialize(com, replication_transfer_service=service, repl_strategy=rm.RingReplicationStrategy(addresses))
    saver = DefaultMLFlashpointCheckpointSaver(
        global_rank_getter=lambda: rank,
        local_rank_getter=lambda: rank,
        global_barrier_func=barrier,
        ckpt_obj_manager=com,
        replication_manager=manager,
        initial_buffer_size_bytes=full + (1 << 20),
        copy_engine=engine,
    )

    note = "full object"
    sub_items = items
    if full > budget:
        picked, total = [], 0
        for wi in items:
            t = resolver.resolve_data(wi)
            n = t.numel() * t.element_size()
            if total + n > budget and picked:
                break
            picked.append(wi)
            total += n
        sub_items = picked
        note = f"prefix of the shard ({total / 1e9:.2f} of {full / 1e9:.2f} GB): tmpfs cannot hold a second full copy per rank"

    def new_checkpoint():
        if state["prev"] is not None:
            com.delete_container(state["prev"])
        ckpt = CheckpointContainerId(os.path.join(workdir, "ckpt", f"step-{state['step']}_ckpt"))
        state["step"] += 1
        state["prev"] = ckpt
        saver.initialize_checkpoint(ckpt)
        return ckpt, saver.prepare_write_data(ckpt, sub_items, resolver, f"__{rank}_", bucket_count=1)

    times, hops = [], []
    both_s, to_hbm_wall_ms, to_hbm_dev_ms = [], [], []
    error = None
    held = 0
    buckets = None
    rounds = [("after_save", 0), ("after_save", 1), ("after_save", 2), ("with_save", 0), ("with_save", 1)]
    for k, (how, i) in enumerate(rounds):
        ckpt, buckets = new_checkpoint()
        try:
            if how == "after_save":
                saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=1)
                barrier()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                futures = manager.async_replicate(com.get_buffer(buckets[0].object_id))
                for f in futures:
                    f.result(timeout=200)
                dt = time.perf_counter() - t0
                if i:  # the first round opens IPC handles and allocates landing buffers
                    times.append(dt)
                    hops.append(service.last_put_stats)
            else:
                barrier()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                pending = saver.write_data_async(ckpt, buckets, replicate_after_write=True)
                pending.result()
                for f in pending.replication_futures:
                    f.result(timeout=200)
                dt = time.perf_counter() - t0
                stats = service.last_put_stats
                if i:
                    both_s.append(dt)
                    to_hbm_wall_ms.append((stats["in_peer_hbm_at"] - t0) * 1e3)
                    if stats.get("since_save_start_ms") is not None:
                        to_hbm_dev_ms.append(stats["since_save_start_ms"])
        except Exception as e:  # keep the collectives below symmetric; report instead of dying
            error = error or f"{type(e).__name__}: {e}"
        held = max(held, engine.held_device_bytes() + service.held_device_bytes())
        barrier()
        if k + 1 < len(rounds):
            shutil.rmtree(replica_root, ignore_errors=True)  # the partner's copy of this round
            barrier()

    # ---- are the replicas the primaries, byte for byte? (digests travel, files stay where they are)
    object_path = str(buckets[0].object_id)
    object_bytes = os.path.getsize(object_path)
    source = (rank - 1) % world_size
    mine = [None] * world_size
    digest_error = None
    try:
        box = {}
        worker = threading.Thread(target=lambda: box.__setitem__("primary", file_sha256(object_path)))
        worker.start()
        dist.all_gather_object(mine, (object_path, None))  # object ids first: the replica's path depends on the sender's
        replica_digest = file_sha256(mapper(mine[source][0], source))
        worker.join()
        digests = [None] * world_size
        dist.all_gather_object(digests, box["primary"])
        ok = replica_digest == digests[source]
    except Exception as e:
        digest_error = f"{type(e).__name__}: {e}"
        ok = False
    all_ok = all_max(0.0 if ok else 1.0, device) == 0.0

    failed = all_max(0.0 if error is None else 1.0, device)
    service.release_peers()  # importers close first ...
    barrier()
    manager.shutdown()  # ... then exporters free their landing buffers
    landing_pool.teardown()
    shutil.rmtree(replica_root, ignore_errors=True)
    if failed:
        return {"error": error or "a peer rank failed", "what": note}
    slow = all_max(statistics.mean(times), device)
    hop_ms = all_max(statistics.mean(h["hop_ms"] for h in hops), device)
    total_bytes = all_sum(object_bytes, device)
    out = {
        "e2e_value": total_bytes / 1e9 / slow,
        "unit": UNIT,
        "ms": slow * 1e3,
        "object_bytes_per_rank": object_bytes,
        "what": note,
        "nvlink_hop_ms": hop_ms,
        "nvlink_hop_gbs_per_gpu": object_bytes / 1e9 / (hop_ms / 1e3),
        "nvlink_frac_of_900": object_bytes / 1e9 / (hop_ms / 1e3) / 900.0,
        "nvlink_frac_of_measured_770": object_bytes / 1e9 / (hop_ms / 1e3) / 770.0,
        "source": "HBM image of the save" if hops[-1]["from_hbm_image"] else "host mapping via bounce ring",
        "partner": "(rank + 1) mod N",
        "bit_exact": bool(all_ok),
        "bit_exact_how": "SHA-256 of the replica each rank received vs the digest of the sender's primary object (all_gather_object)",
        "hbm_held_bytes": int(all_max(float(held), device)),
        "landing_chunk_bytes": int(args.landing_chunk_mb * (1 << 20)),
    }
    if digest_error:
        out["bit_exact_error"] = digest_error
    if both_s:
        out["with_save"] = {
            "what": "write_data_async(replicate_after_write=True): push queued with the pack kernel, NVLink hop overlaps the drain",
            "save_and_replica_on_partner_host_ms": all_max(statistics.mean(both_s), device) * 1e3,
            "ms_to_partner_hbm": all_max(statistics.mean(to_hbm_wall_ms), device),
            "ms_to_partner_hbm_device": all_max(statistics.mean(to_hbm_dev_ms), device) if to_hbm_dev_ms else None,
            "note": "ms_to_partner_hbm = wall time from the call to the last byte of the replica in the partner's HBM; "
            "the _device figure runs from the pack kernel's start event to the end of the copy kernel",
        }
    return out


def overlap_probe(saver, com, base, state, items, resolver, rank, device) -> dict:
    """Runs a fixed batch of bf16 GEMMs (standing in for training compute) alone and again while an
    overlapped save is in flight, and times both on the device."""
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId

    a = torch.randn(8192, 8192, device=device, dtype=torch.bfloat16)
    b = torch.randn(8192, 8192, device=device, dtype=torch.bfloat16)
    reps = 150

    def gemms():
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            torch.matmul(a, b)
        t1.record()
        return t0, t1

    for _ in range(2):
        t0, t1 = gemms()
        torch.cuda.synchronize()
    alone_ms = t0.elapsed_time(t1)

    if state["prev"] is not None:
        com.delete_container(state["prev"])
    ckpt = CheckpointContainerId(os.path.join(base, f"step-{state['step']}_ckpt"))
    state["step"] += 1
    state["prev"] = ckpt
    saver.initialize_checkpoint(ckpt)
    buckets = saver.prepare_write_data(ckpt, items, resolver, f"__{rank}_", bucket_count=1)
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    pending = saver.write_data_async(ckpt, buckets)
    t0, t1 = gemms()  # queued right behind the launch: runs while the pack kernel and the drain do
    results = pending.result()
    save_wall_ms = (time.perf_counter() - wall0) * 1e3
    torch.cuda.synchronize()
    with_save_ms = t0.elapsed_time(t1)
    return {
        "gemm_batch_ms_alone": alone_ms,
        "gemm_batch_ms_during_save": with_save_ms,
        "slowdown": with_save_ms / alone_ms,
        "save_wall_ms_with_gemms_running": save_wall_ms,
        "what": f"{reps} x 8192^3 bf16 matmul on the training stream, queued while write_data_async's kernel and transfer run",
        "_results": results,
        "_buckets": buckets,
    }


def run_native_arm(args, rank: int, world_size: int, device, workdir: str) -> None:
    import ctypes

    from ml_flashpoint import _native
    from ml_flashpoint.checkpoint_object_manager.buffer_metadata import METADATA_SIZE
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core import gpu_engine
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.core.checkpoint_loader import DefaultMLFlashpointCheckpointLoader
    from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    lib = _native.lib()
    shard = build_shard(rank, device, layers=args.layers)
    payload = sum(t.numel() * t.element_size() for _, t, _, _ in shard)
    items, resolver = write_items_for(shard)
    engine = gpu_engine.CudaCopyEngine(device=device, mode=args.mode, arena_limit_bytes=int(args.arena_limit_gb * (1 << 30)))
    gpu_engine.set_default_engine(engine)  # replication looks the HBM image up through the process-wide engine

    # size the pool buffer exactly: header sizes are known without touching the GPU
    layout = gpu_engine.plan_object_layout([(None, t) for _, t, _, _ in shard], [])
    object_bytes = METADATA_SIZE + layout.total_bytes
    t_reg0 = time.perf_counter()
    pool_cfg = BufferPoolConfig(os.path.join(workdir, "buffer_pool"), rank, 1, object_bytes, register_cuda=True)
    com = CheckpointObjectManager(pool_cfg)
    com._get_or_create_buffer_pool()
    register_s = time.perf_counter() - t_reg0

    saver = DefaultMLFlashpointCheckpointSaver(
        global_rank_getter=lambda: rank,
        local_rank_getter=lambda: rank,
        global_barrier_func=barrier,
        ckpt_obj_manager=com,
        replication_manager=None,
        initial_buffer_size_bytes=layout.total_bytes,
        copy_engine=engine,
    )
    loader = DefaultMLFlashpointCheckpointLoader(
        com,
        None,
        global_rank_getter=lambda: rank,
        local_rank_getter=lambda: rank,
        broadcast_object_list_func=lambda *a, **k: None,
        all_gather_object_func=lambda *a, **k: None,
        world_size_getter=lambda: world_size,
        copy_engine=engine,
    )
    base = os.path.join(workdir, "ckpt")
    state = {"step": 0, "prev": None}

    def one_save():
        if state["prev"] is not None:
            com.delete_container(state["prev"])  # frees the pool buffer for reuse
        ckpt = CheckpointContainerId(os.path.join(base, f"step-{state['step']}_ckpt"))
        state["step"] += 1
        saver.initialize_checkpoint(ckpt)
        buckets = saver.prepare_write_data(ckpt, items, resolver, f"__{rank}_", bucket_count=1)
        t0 = time.perf_counter()
        results = saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=1)
        wall = time.perf_counter() - t0
        state["prev"] = ckpt
        ticket = engine.last_ticket
        return ckpt, buckets, results, wall, ticket.kernel_ms(), ticket.total_ms()

    for _ in range(args.warmup):
        one_save()

    sampler = ClockSampler(device.index)
    launches0 = lib.mlf_launch_count()
    barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    region0 = time.perf_counter()
    walls, kernel_ms, device_ms = [], [], []
    for _ in range(args.steps):
        ckpt, buckets, results, wall, k_ms, d_ms = one_save()
        walls.append(wall)
        kernel_ms.append(k_ms)
        device_ms.append(d_ms)
    torch.cuda.synchronize()
    barrier()
    region_s = time.perf_counter() - region0
    clocks = sampler.stop() if rank == 0 else None
    launches = lib.mlf_launch_count() - launches0

    # ---- overlapped save: how long the caller is held before it may mutate the tensors again
    async_block_ms = []
    for _ in range(2):
        if state["prev"] is not None:
            com.delete_container(state["prev"])
        ckpt = CheckpointContainerId(os.path.join(base, f"step-{state['step']}_ckpt"))
        state["step"] += 1
        state["prev"] = ckpt
        saver.initialize_checkpoint(ckpt)
        buckets = saver.prepare_write_data(ckpt, items, resolver, f"__{rank}_", bucket_count=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        pending = saver.write_data_async(ckpt, buckets)
        pending.wait_safe_to_mutate()
        async_block_ms.append((time.perf_counter() - t0) * 1e3)
        results = pending.result()

    # ---- does a save in flight slow the training stream down? (background load: library GEMMs)
    overlap = None
    if world_size == 1 and not args.no_overlap_probe:
        overlap = overlap_probe(saver, com, base, state, items, resolver, rank, device)
        results, buckets = overlap.pop("_results"), overlap.pop("_buckets")

    # ---- restore (its own timed region; not part of the save step)
    restore = None
    if not args.no_restore:
        storage = {r.index: r.storage_data for r in results}
        sources = {wi.index: resolver.resolve_data(wi) for wi in items}
        targets = {idx: torch.empty_like(t) for idx, t in sources.items()}
        reqs = [
            ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * t.dim()), idx, torch.Size([0] * t.dim()), t.shape)
            for idx, t in targets.items()
        ]

        class _Planner:
            def resolve_tensor(self, req):
                return targets[req.dest_index]

            def commit_tensor(self, req, tensor):
                pass

        r_walls, r_h2d, r_kernel = [], [], []
        for i in range(1 + max(1, args.steps)):
            barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            loader.read_data(buckets[0].object_id, reqs, _Planner(), storage)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if i:  # first pass is warm-up
                r_walls.append(dt)
                r_h2d.append(engine.last_unpack_ms[0])
                r_kernel.append(engine.last_unpack_ms[1])
        verified = all(torch.equal(targets[idx], sources[idx]) for idx in targets)
        worst = all_max(statistics.mean(r_walls), device)
        restore = {
            "e2e_value": all_sum(payload, device) / 1e9 / worst,
            "unit": UNIT,
            "ms": worst * 1e3,
            "host_to_hbm_ms": statistics.mean(r_h2d),
            "kernel_ms": statistics.mean(r_kernel),
            "kernel_hbm_gbs": 2 * payload / 1e9 / (statistics.mean(r_kernel) / 1e3),
            "bit_exact": bool(verified),
            "h2d_bytes_per_step": layout.total_bytes,
        }
        del targets

    # ---- parity of the object just saved with the CPU oracle (its checker role): the whole shard
    # through a streaming SHA-256 on one GPU, a 64 MB prefix on every rank otherwise
    parity = None
    parity_prefix = None
    object_path = str(buckets[0].object_id)
    if not args.no_cpu_baseline:
        import mlf_oracle as oracle

        sample, _ = cpu_sample(shard, 64 << 20)
        want, _ = oracle.pack_object([(str(i), t.cpu()) for i, t in enumerate(sample)], [])
        with open(object_path, "rb") as f:
            got = f.read(len(want))
        # the oracle's metadata block carries the sample's length; compare the data section prefix
        mine_ok = got[METADATA_SIZE:] == want[METADATA_SIZE:]
        parity_prefix = all_max(0.0 if mine_ok else 1.0, device) == 0.0
        if world_size == 1:
            box = {}
            worker = threading.Thread(target=lambda: box.__setitem__("file", file_sha256(object_path)))
            worker.start()
            # tensors stay on the GPU; the oracle brings one at a time to the host while it hashes it
            want_sha, want_size = oracle.object_sha256([(str(i), t) for i, (_, t, _, _) in enumerate(shard)])
            worker.join()
            parity = {
                "whole_object_sha256_equal": box["file"] == want_sha and os.path.getsize(object_path) == want_size,
                "object_bytes": want_size,
                "file_sha256": box["file"],
                "oracle_sha256": want_sha,
                "how": "oracle.object_sha256 (headers and payloads hashed tensor by tensor) vs SHA-256 of the saved object file",
            }

    # ---- replication to the ring partner (only where there is a partner)
    replication = None
    if world_size > 1 and not args.no_replication:
        replication = run_replication(args, rank, world_size, device, workdir, com, engine, items, resolver, shard, state)

    hbm_held = int(all_max(float(engine.held_device_bytes()), device))
    pinned_peak = calibrate_host_link(device)

    total_payload = all_sum(payload, device)
    slow_device_s = all_max(sum(device_ms) / 1e3, device)
    slow_region_s = all_max(region_s, device)
    slow_wall_s = all_max(sum(walls), device)
    kernel_s = statistics.mean(kernel_ms) / 1e3
    peak, peak_src = measured_hbm_peak()

    cpu = None
    if rank == 0 and world_size == 1 and not args.no_cpu_baseline:
        engine.release_device_memory()  # the CPU baseline stages the same state from this GPU; free the image arena first
        if reference_arm_unavailable() is None:
            # the reference's own saver and loader, one rank, in a process of its own (its package has
            # the same name as this one); it also reports the SHA-256 of the object IT wrote
            cpu = run_reference_ranks(1, 2, 2, workdir, args.layers, args.cpu_baseline_budget_s, digest=True)
            theirs = cpu.pop("objects")[0]
            if parity is not None and cpu["whole_shard"]:
                parity["equal_to_reference_object"] = theirs["sha256"] == parity["file_sha256"] and theirs["size"] == parity["object_bytes"]
                parity["reference_how"] = "SHA-256 of the object the reference's own saver wrote for the same seeded shard (oracle/_ref)"
        else:
            cpu = run_cpu_port(shard, workdir, int(args.cpu_sample_gb * 1e9), passes=3)
            cpu["sample"] = reference_arm_unavailable() + "; " + cpu["sample"]

    if rank != 0:
        return
    achieved = 2 * payload / 1e9 / kernel_s
    if (args.mode or "staged") == "direct" or statistics.mean(device_ms) <= statistics.mean(kernel_ms):
        # the kernel's own stores cross the host link: kernel time is transfer time
        d2h_gbs = layout.total_bytes / 1e9 / (statistics.mean(device_ms) / 1e3)
    else:
        d2h_gbs = layout.total_bytes / 1e9 / ((statistics.mean(device_ms) - statistics.mean(kernel_ms)) / 1e3)
    if restore is not None:
        per_gpu = restore["e2e_value"] / world_size
        restore["roofline"] = {
            "bound": "host_link",
            "achieved": per_gpu,
            "peak": pinned_peak["h2d"],
            "unit": "GB/s",
            "frac": per_gpu / pinned_peak["h2d"],
            "peak_source": "plain pinned host-to-device copies, all ranks at once, slowest rank (this run)",
            "what": "end-to-end restore per GPU: object file -> HBM image -> unpack kernel -> target tensors",
        }
    line = {
        "metric": METRIC,
        "value": total_payload * args.steps / 1e9 / slow_device_s,
        "unit": UNIT,
        "n_gpus": world_size,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": slow_region_s / args.steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "u8",
        "data": "synthetic",
        "config": workload_config(args, payload),
        "per_gpu_value": total_payload * args.steps / 1e9 / slow_device_s / world_size,
        "blocking_save_ms": {
            "time_to_safe_mutate": statistics.mean(kernel_ms),
            "call_to_return": statistics.mean(walls) * 1e3,
            "overlapped_call_to_safe_mutate": min(async_block_ms),
            "note": "time_to_safe_mutate = pack kernel (device); call_to_return = blocking write_data; "
            "overlapped_call_to_safe_mutate = wall time write_data_async holds the caller (planning + launch + kernel)",
        },
        "e2e": {
            "value": total_payload * args.steps / 1e9 / slow_wall_s,
            "unit": UNIT,
            "h2d_bytes_per_step": layout.host_blob_size(),
            "d2h_bytes_per_step": layout.total_bytes,
            "api": "DefaultMLFlashpointCheckpointSaver.write_data (object closed on return)",
        },
        "restore": restore,
        "hbm_held_bytes": hbm_held,
        "hbm_held_note": "HBM the data path holds beyond the caller's tensors during a save (the image arena); "
        "replication adds landing and bounce buffers, see replication.hbm_held_bytes",
        "overlap": overlap,
        "replication": replication,
        "roofline": {
            "kernel": "mlf_plan_kernel_stream<PACK>",
            "bound": "hbm",
            "achieved": achieved,
            "peak": peak,
            "unit": "GB/s",
            "frac": achieved / peak,
            "peak_source": peak_src,
            "algorithmic_bytes_per_launch": 2 * payload,
            "kernel_ms": statistics.mean(kernel_ms),
            "traffic": NCU_DRAM_BYTES_PER_PAYLOAD_BYTE * payload,
            "traffic_source": "ncu capture of a 2.6 GB case scaled by payload bytes",
        },
        "host_link": {
            "d2h_gbs": d2h_gbs,
            "note": "copy-engine drain of the HBM image into the page-locked object mapping (staged), "
            "or the kernel's own stores into it (direct)",
            "pinned_copy_peak_d2h_gbs": pinned_peak["d2h"],
            "pinned_copy_peak_h2d_gbs": pinned_peak["h2d"],
            "peak_note": "plain copies to/from driver-allocated pinned memory, all ranks at once, slowest rank",
            "frac_of_pinned_peak": d2h_gbs / pinned_peak["d2h"],
            "frac_of_pcie_gen5_x16_63gbs": d2h_gbs / 63.0,
        },
        "cpu_baseline": cpu,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "parity_vs_oracle": parity,
        "parity_vs_oracle_prefix": parity_prefix,
        "pool_register_s": register_s,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
