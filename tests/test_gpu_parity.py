"""GPU parity: the CUDA pack / unpack path against the golden vectors and the CPU oracle.

Everything here goes through the C ABI of libmlf_b200.so (directly via ctypes plans, or through the
saver / loader, which call the same entry points). Integer/byte work: the bar is bit-exact.
"""

import ctypes
import hashlib
import os

import numpy as np
import pytest
import torch

import cases
import mlf_oracle as oracle
from helpers import case_to_device, golden_object_bytes, load_golden, make_loader, make_saver, tensor_bytes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine():
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    return CudaCopyEngine(mode="staged")


@pytest.fixture(scope="module")
def direct_engine():
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    return CudaCopyEngine(mode="direct")


def _save(case, tmp_path, engine, **kw):
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId

    saver, com = make_saver(copy_engine=engine, **kw)
    ckpt = CheckpointContainerId(str(tmp_path / "step-1_ckpt"))
    saver.initialize_checkpoint(ckpt)
    items, resolver = cases.write_items_and_resolver(case)
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=case["bucket_count"])
    results = saver.write_data(ckpt, buckets, replicate_after_write=False, thread_count=1)
    return saver, com, ckpt, buckets, results


@pytest.mark.parametrize("mode", ["staged", "direct"])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_saved_objects_match_reference_bytes(name, mode, shm_path, golden_dir, engine, direct_engine):
    gold = load_golden(golden_dir, f"{name}.json")
    case = case_to_device(cases.CASES[name](), "cuda")
    _, _, ckpt, buckets, results = _save(case, shm_path, engine if mode == "staged" else direct_engine)
    assert [b.object_name for b in buckets] == [o["name"] for o in gold["objects"]]
    for bucket, g in zip(buckets, gold["objects"]):
        with open(str(bucket.object_id), "rb") as f:
            data = f.read()
        assert len(data) == g["size"]
        if "file" in g:
            want = golden_object_bytes(golden_dir, g)
            if data != want:
                first = next(i for i in range(len(want)) if data[i] != want[i])
                pytest.fail(f"{bucket.object_name}: first differing byte at {first}")
        assert hashlib.sha256(data).hexdigest() == g["sha256"]
    got = sorted((r.storage_data.relative_path, r.storage_data.offset, r.storage_data.length, r.index.fqn, r.size_in_bytes) for r in results)
    want = [(w["relative_path"], w["offset"], w["length"], w["index"]["fqn"], w["size_in_bytes"]) for w in gold["write_results"]]
    assert got == want


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_restore_round_trip_is_bit_exact(name, tmp_path, engine):
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    case = case_to_device(cases.CASES[name](), "cuda")
    _, com, ckpt, buckets, results = _save(case, tmp_path, engine)
    loader = make_loader(com, copy_engine=engine)
    storage = {r.index: r.storage_data for r in results}
    by_fqn = {r.index.fqn: r.index for r in results}
    targets, blobs = {}, {}

    class _Planner:
        def resolve_tensor(self, req):
            return targets[req.dest_index.fqn]

        def commit_tensor(self, req, tensor):
            pass

        def load_bytes(self, req, value):
            blobs[req.dest_index.fqn] = value.read()

    per_object = {}
    for fqn, t in case["tensors"].items():
        if t.numel() == 0:
            continue  # zero-element tensors cannot be loaded by the reference either
        idx = by_fqn[fqn]
        # strided targets on purpose for 2-D tensors: restore must honour destination strides
        if t.dim() == 2:
            targets[fqn] = torch.zeros((t.shape[1], t.shape[0]), dtype=t.dtype, device="cuda").t()
        else:
            targets[fqn] = torch.zeros(t.shape, dtype=t.dtype, device="cuda")
        req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * t.dim()), idx, torch.Size([0] * t.dim()), torch.Size(t.shape))
        per_object.setdefault(storage[idx].relative_path, []).append(req)
    for fqn in case["blobs"]:
        idx = by_fqn[fqn]
        req = ReadItem(LoadItemType.BYTE_IO, idx, None, idx, None, None)
        per_object.setdefault(storage[idx].relative_path, []).append(req)
    for bucket in buckets:
        loader.read_data(bucket.object_id, per_object.get(bucket.object_name, []), _Planner(), storage)
    torch.cuda.synchronize()
    for fqn, target in targets.items():
        assert tensor_bytes(target) == tensor_bytes(case["tensors"][fqn]), fqn
    assert blobs == dict(case["blobs"])


def test_narrow_reads_match_reference(tmp_path, golden_dir, engine):
    from torch.distributed.checkpoint.metadata import MetadataIndex
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    rows = load_golden(golden_dir, "narrow.json")
    tensors = {f"n.{i}": cases.narrow_source(i).cuda() for i in range(len(cases.NARROW_CASES))}
    _, com, ckpt, buckets, results = _save({"tensors": tensors, "blobs": {}, "bucket_count": 1}, tmp_path, engine)
    loader = make_loader(com, copy_engine=engine)
    storage = {r.index: r.storage_data for r in results}
    for device in ("cuda", "cpu"):
        for row in rows:
            shape, dtype, offs, lens = cases.NARROW_CASES[row["i"]]
            idx = MetadataIndex(f"n.{row['i']}", torch.Size([0] * len(shape)))
            target = torch.zeros(lens, dtype=dtype, device=device)
            req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * len(lens)), idx, torch.Size(offs), torch.Size(lens))

            class _Planner:
                def resolve_tensor(self, r):
                    return target

                def commit_tensor(self, r, t):
                    pass

            loader.read_data(buckets[0].object_id, [req], _Planner(), {idx: storage[idx]})
            assert tensor_bytes(target).hex() == row["hex"], (device, row["i"])


def _flat_copy(dst_ptr, src_ptr, n):
    from ml_flashpoint import _native

    _native.check(_native.lib().mlf_copy_kernel_launch(ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr), n, None, 0))


def test_flat_copy_every_misalignment_and_small_size():
    """All 16 x 16 source/destination residues, sizes 0..257 and around the tile size."""
    torch.cuda.synchronize()
    g = torch.Generator().manual_seed(7)
    src_host = torch.randint(0, 256, (1 << 18,), generator=g, dtype=torch.uint8)
    src = src_host.cuda()
    sizes = list(range(0, 258)) + [4095, 4096, 4097, 65535, 65536, 65537, 131072 + 5]
    for so in range(16):
        for do in range(16):
            dst = torch.full((1 << 18,), 0xA5, dtype=torch.uint8, device="cuda")
            # a few sizes per residue pair keeps the sweep fast; every size is hit for some pair
            picked = sizes[(so * 16 + do) % 7 :: 7] + [257, 65537]
            pos = 64
            spans = []
            for n in picked:
                if pos + do + n + 64 > dst.numel():
                    break
                _flat_copy(dst.data_ptr() + pos + do, src.data_ptr() + 32 + so, n)
                spans.append((pos + do, n))
                pos += ((n + do + 31) // 16 + 2) * 16
            torch.cuda.synchronize()
            out = dst.cpu()
            expect = torch.full_like(out, 0xA5)
            for at, n in spans:
                expect[at : at + n] = src_host[32 + so : 32 + so + n]
            assert torch.equal(out, expect), (so, do)  # also proves nothing outside the spans was touched


def test_bounded_device_wait_gives_up_and_reports_through_the_status_word():
    """The kernels' waits are bounded: a wait on a barrier that nothing completes returns after its
    budget, the kernel records MLF_ERR_TIMEOUT and exits, and the context stays usable."""
    import time

    from ml_flashpoint import _native

    lib = _native.lib()
    t0 = time.perf_counter()
    rc = lib.mlf_selftest_wait_timeout(2_000_000, None)  # 2 ms budget
    elapsed = time.perf_counter() - t0
    assert rc == _native.MLF_ERR_TIMEOUT
    assert b"gave up" in lib.mlf_last_error()
    assert elapsed < 1.0
    with pytest.raises(_native.NativeError) as refused:
        _native.check(lib.mlf_selftest_wait_timeout(10**9, None))  # budgets above 100 ms are refused
    assert refused.value.code == _native.MLF_ERR_INVALID
    # the context is intact: an ordinary copy still works
    src = torch.arange(100000, dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    _flat_copy(dst.data_ptr(), src.data_ptr(), src.numel() * 4)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)


def test_plan_rejects_out_of_window_launch(engine):
    from ml_flashpoint import _native

    t = torch.arange(1024, dtype=torch.int32, device="cuda")
    desc = (_native.CopyDesc * 1)()
    from ml_flashpoint.core.gpu_engine import fill_desc

    fill_desc(desc[0], t.data_ptr(), 100, 4, (1024,), (1,), (1,))
    plan = ctypes.c_void_p()
    lib = _native.lib()
    _native.check(lib.mlf_plan_create(desc, 1, _native.MLF_PACK, ctypes.byref(plan)))
    try:
        assert lib.mlf_plan_image_extent(plan) == 100 + 4096
        assert lib.mlf_plan_payload_bytes(plan) == 4096
        image = torch.zeros(8192, dtype=torch.uint8, device="cuda")
        rc = lib.mlf_plan_launch(plan, ctypes.c_void_p(image.data_ptr()), 4000, None, 0)
        assert rc == _native.MLF_ERR_BOUNDS
        assert b"only 4000" in lib.mlf_last_error()
        _native.check(lib.mlf_plan_launch(plan, ctypes.c_void_p(image.data_ptr()), 8192, None, 0))
        torch.cuda.synchronize()
        assert bytes(image[100 : 100 + 4096].cpu().numpy()) == t.cpu().numpy().tobytes()
        assert int(image[:100].sum()) == 0 and int(image[4196:].sum()) == 0
    finally:
        lib.mlf_plan_destroy(plan)


@pytest.mark.parametrize("esize,dtype", [(1, torch.uint8), (2, torch.int16), (4, torch.int32), (8, torch.int64)])
def test_large_transposed_and_row_sliced_sources(esize, dtype, engine, tmp_path):
    """Transposes larger than one tile, ragged edges, every image residue class via a blob prefix."""
    g = torch.Generator().manual_seed(esize)
    for prefix in (0, 1, 3, 6, 13):
        base = torch.randint(0, 120, (201, 333), generator=g, dtype=torch.int64).to(dtype).cuda()
        big = torch.randint(0, 120, (70, 5000), generator=g, dtype=torch.int64).to(dtype).cuda()
        tensors = {
            "pad": torch.zeros(prefix, dtype=torch.uint8, device="cuda"),
            "t": base.t(),
            "rows": big[:, 17:4900],
            "rows_long": big[3:60, 8:],
            "batch_t": torch.randint(0, 99, (3, 65, 130), generator=g, dtype=torch.int64).to(dtype).cuda().transpose(1, 2),
        }
        case = {"tensors": tensors, "blobs": {}, "bucket_count": 1}
        _, _, _, buckets, _ = _save(case, tmp_path / f"p{prefix}", engine)
        with open(str(buckets[0].object_id), "rb") as f:
            data = f.read()
        cpu_case = {"tensors": {k: v.cpu() for k, v in tensors.items()}, "blobs": {}, "bucket_count": 1}
        ((_, want, _),) = oracle.save_case(cpu_case)
        assert data == want, (esize, prefix)


def _views_for_regimes(dtype, g):
    """Views that land in every staged regime of the plan kernel: narrow and wide transposes, with
    and without batch dimensions, ragged in both directions, and short rows cut out of wider ones."""

    def rnd(*shape):
        if dtype == torch.complex128:
            return torch.view_as_complex(torch.randn(*shape, 2, generator=g, dtype=torch.float64)).cuda()
        return torch.randint(0, 120, shape, generator=g, dtype=torch.int64).to(dtype).cuda()

    out = []
    for rows in (1, 3, 17, 64, 100, 127, 128, 129, 255):  # image row length of x.t(), in elements
        out.append(rnd(rows, 2311).t())
    out.append(rnd(64, 33000).t())  # more than four sub-tiles of narrow rows per tile
    out.append(rnd(300, 1000).t())
    out.append(rnd(1029, 515).t())  # wide rows, several sub-tiles along the row, ragged edges
    out.append(rnd(3, 65, 130).transpose(1, 2))
    out.append(rnd(2, 3, 40, 50).transpose(-1, -2))
    out.append(rnd(5, 70, 11).permute(2, 0, 1))
    out.append(rnd(6, 9, 200).permute(1, 2, 0))
    wide = rnd(700, 300)
    for cols in (1, 3, 16, 64, 100, 127):  # short rows, back to back in the image only
        out.append(wide[:, 5 : 5 + cols])
    out.append(rnd(4, 600, 40)[:, :, 5:30])
    out.append(wide[::2, 7:90])
    return out


@pytest.mark.parametrize(
    "dtype", [torch.uint8, torch.int16, torch.int32, torch.int64, torch.complex128], ids=lambda d: str(d).split(".")[-1]
)
def test_every_staged_regime_packs_and_unpacks_bit_exactly(dtype):
    """Plans through the C ABI, both directions, image offsets of every residue class mod 16:
    the packed bytes equal the oracle's C-order payload, the unpacked views equal the sources and
    nothing outside a view or a payload is written."""
    from ml_flashpoint import _native
    from ml_flashpoint.core.gpu_engine import _Plan, c_strides, fill_desc

    g = torch.Generator().manual_seed(11)
    views = _views_for_regimes(dtype, g)
    n = len(views)
    descs = (_native.CopyDesc * n)()
    offsets, at = [], 5
    for i, v in enumerate(views):
        offsets.append(at)
        at += v.numel() * v.element_size() + 16 + (i % 16)  # gaps walk through all residues
    image = torch.full((at + 64,), 0xA5, dtype=torch.uint8, device="cuda")
    for i, v in enumerate(views):
        fill_desc(descs[i], v.data_ptr(), offsets[i], v.element_size(), v.shape, v.stride(), c_strides(v.shape))
    plan = _Plan(descs, n, _native.MLF_PACK)
    plan.launch(image.data_ptr(), image.numel(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    plan.status()
    got = image.cpu().numpy().tobytes()
    expect = bytearray(b"\xa5" * image.numel())
    for v, o in zip(views, offsets):
        payload = oracle.tensor_payload(v.cpu())
        expect[o : o + len(payload)] = payload
    assert got == bytes(expect)

    targets, bases = [], []
    for v in views:
        base = torch.zeros_like(v._base)
        bases.append(base)
        targets.append(base.as_strided(v.shape, v.stride(), v.storage_offset()))
    for i, t in enumerate(targets):
        fill_desc(descs[i], t.data_ptr(), offsets[i], t.element_size(), t.shape, t.stride(), c_strides(t.shape))
    plan = _Plan(descs, n, _native.MLF_UNPACK)
    plan.launch(image.data_ptr(), image.numel(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    plan.status()
    for v, t, base in zip(views, targets, bases):
        want = torch.zeros_like(v._base)
        want.as_strided(v.shape, v.stride(), v.storage_offset()).copy_(v)
        assert torch.equal(torch.view_as_real(base) if base.is_complex() else base, torch.view_as_real(want) if want.is_complex() else want)


def _random_view(rng, dtype):
    """A random strided view: random rank and extents, then a random permutation, random slices
    (sometimes stepped) and now and then an expanded dimension."""
    rank = rng.randint(1, 5)
    budget = rng.choice([40, 3000, 200000, 1500000])
    dims = []
    for _ in range(rank):
        d = max(1, int(round(budget ** (rng.random() / rank * 2))))
        dims.append(min(d, 700))
    base = torch.randint(0, 120, tuple(dims), dtype=torch.int64).to(dtype)
    view = base.permute(*rng.sample(range(rank), rank)) if rank > 1 and rng.random() < 0.7 else base
    index = []
    for n in view.shape:
        kind = rng.random()
        if kind < 0.5 or n < 3:
            index.append(slice(None))
        elif kind < 0.85:
            a = rng.randint(0, n - 2)
            index.append(slice(a, rng.randint(a + 1, n)))
        else:
            index.append(slice(rng.randint(0, 1), None, rng.randint(2, 3)))
    view = view[tuple(index)]
    return base.cuda().as_strided(view.shape, view.stride(), view.storage_offset())


@pytest.mark.parametrize("seed", range(6))
def test_random_views_pack_and_unpack_like_the_oracle(seed):
    """Differential test over random strided views (permutations, slices, steps) of every element
    size: packed bytes equal the oracle's C-order payload, unpacking into zeroed copies of the
    same views restores exactly the viewed elements and nothing else."""
    import random as _random

    from ml_flashpoint import _native
    from ml_flashpoint.core.gpu_engine import _Plan, c_strides, fill_desc

    rng = _random.Random(1000 + seed)
    torch.manual_seed(seed)
    dtypes = [torch.uint8, torch.int16, torch.int32, torch.int64]
    views = [_random_view(rng, rng.choice(dtypes)) for _ in range(40)]
    views = [v for v in views if v.numel() > 0]
    n = len(views)
    descs = (_native.CopyDesc * n)()
    offsets, at = [], rng.randint(0, 15)
    for v in views:
        offsets.append(at)
        at += v.numel() * v.element_size() + rng.randint(0, 40)
    image = torch.full((at + 64,), 0x5A, dtype=torch.uint8, device="cuda")
    for i, v in enumerate(views):
        fill_desc(descs[i], v.data_ptr(), offsets[i], v.element_size(), v.shape, v.stride(), c_strides(v.shape))
    stream = torch.cuda.current_stream().cuda_stream
    plan = _Plan(descs, n, _native.MLF_PACK)
    plan.launch(image.data_ptr(), image.numel(), stream)
    torch.cuda.synchronize()
    plan.status()
    expect = bytearray(b"\x5a" * image.numel())
    for v, o in zip(views, offsets):
        payload = oracle.tensor_payload(v.cpu())
        expect[o : o + len(payload)] = payload
    got = image.cpu().numpy().tobytes()
    if got != bytes(expect):
        bad = next(i for i in range(len(got)) if got[i] != expect[i])
        which = max(k for k, o in enumerate(offsets) if o <= bad)
        pytest.fail(f"seed {seed}: byte {bad} differs, view {which}: shape {tuple(views[which].shape)} stride {views[which].stride()} {views[which].dtype}")

    targets, bases = [], []
    for v in views:
        base = torch.zeros_like(v._base if v._base is not None else v)
        bases.append(base)
        targets.append(base.as_strided(v.shape, v.stride(), v.storage_offset()))
    for i, t in enumerate(targets):
        fill_desc(descs[i], t.data_ptr(), offsets[i], t.element_size(), t.shape, t.stride(), c_strides(t.shape))
    plan = _Plan(descs, n, _native.MLF_UNPACK)
    plan.launch(image.data_ptr(), image.numel(), stream)
    torch.cuda.synchronize()
    plan.status()
    for k, (v, base) in enumerate(zip(views, bases)):
        want = torch.zeros_like(base)
        want.as_strided(v.shape, v.stride(), v.storage_offset()).copy_(v)
        assert torch.equal(base, want), f"seed {seed}: view {k}: shape {tuple(v.shape)} stride {v.stride()} {v.dtype}"


def test_overlapped_save_reads_sources_before_safe_to_mutate(shm_path, golden_dir, engine):
    """After ``wait_safe_to_mutate`` the sources may be overwritten: the object still holds the old values."""
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId

    gold = load_golden(golden_dir, "gpt2_tiny.json")
    case = case_to_device(cases.CASES["gpt2_tiny"](), "cuda")
    CheckpointObjectManager._worker_pool = None
    pool = BufferPoolConfig(str(shm_path / "pool"), 0, 1, 1 << 20, register_cuda=True)  # page-locked: the drain is asynchronous
    saver, com = make_saver(copy_engine=engine, pool_config=pool)
    ckpt = CheckpointContainerId(str(shm_path / "step-1_ckpt"))
    saver.initialize_checkpoint(ckpt)
    items, resolver = cases.write_items_and_resolver(case)
    buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=1)
    pending = saver.write_data_async(ckpt, buckets)
    pending.wait_safe_to_mutate()
    for t in case["tensors"].values():
        t.zero_()  # the optimizer step of the next iteration
    torch.cuda.synchronize()
    results = pending.result()
    data = open(str(buckets[0].object_id), "rb").read()
    assert hashlib.sha256(data).hexdigest() == gold["objects"][0]["sha256"]
    assert len(results) == len(gold["write_results"])
    com.teardown_pool()


def test_overlapped_save_of_several_objects_packs_them_back_to_back(shm_path):
    """A save that writes two objects per rank: the second object's pack kernel does not wait for the
    first object's transfer to the host, both objects match the oracle, and both images stay
    resident in HBM for replication."""
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    engine = CudaCopyEngine(mode="staged")
    g = torch.Generator(device="cuda").manual_seed(21)
    tensors = {f"w{i}": torch.randint(-100, 100, (128 << 20,), device="cuda", dtype=torch.int32, generator=g) for i in range(4)}
    case = {"tensors": tensors, "blobs": {"note": b"two objects"}, "bucket_count": 2}
    CheckpointObjectManager._worker_pool = None
    pool = BufferPoolConfig(str(shm_path / "pool"), 0, 2, (1 << 30) + (1 << 20), register_cuda=True)
    saver, com = make_saver(copy_engine=engine, pool_config=pool)
    ckpt = CheckpointContainerId(str(shm_path / "step-1_ckpt"))
    items, resolver = cases.write_items_and_resolver(case)
    for step in range(2):  # the first save sizes the arena, the second one runs in the steady state
        saver.initialize_checkpoint(ckpt)
        buckets = saver.prepare_write_data(ckpt, items, resolver, "__0_", bucket_count=2)
        assert len(buckets) == 2
        pending = saver.write_data_async(ckpt, buckets)
        pending.wait_safe_to_mutate()
        pending.result()
        tickets = [part[3] for part in pending._parts]
    first, second = tickets
    second_packed = first.start_event.elapsed_time(second.mutate_event)
    first_drained = first.start_event.elapsed_time(first.done_event)
    assert second_packed < first_drained, (second_packed, first_drained)
    cpu_case = {"tensors": {k: v.cpu() for k, v in tensors.items()}, "blobs": case["blobs"], "bucket_count": 2}
    want = {name: data for name, data, _ in oracle.save_case(cpu_case)}
    for bucket in buckets:
        with open(str(bucket.object_id), "rb") as f:
            data = f.read()
        assert data == want[bucket.object_name], bucket.object_name
        assert engine.resident_image(str(bucket.object_id), len(data) - 4096) is not None
    com.teardown_pool()


def test_page_locked_buffer_resizes_in_place_and_copies_cross_its_chunks(shm_path):
    """A registered buffer larger than one page-lock chunk: copy-engine transfers and kernel stores
    that span chunk boundaries land byte-exactly, and shrinking / growing the buffer keeps it
    registered at the same address with its contents, re-locking only its tail."""

    from ml_flashpoint import _native
    from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

    lib = _native.lib()
    chunk = 512 << 20
    size = 3 * chunk + 12345
    buf = BufferObject(str(shm_path / "big.distcp"), size, overwrite=True)
    buf.register_cuda()
    assert buf.is_cuda_registered and buf.get_device_ptr() == buf.get_data_ptr()
    base = buf.get_data_ptr()
    g = torch.Generator(device="cuda").manual_seed(5)
    src = torch.randint(0, 256, (size,), device="cuda", dtype=torch.uint8, generator=g)
    stream = torch.cuda.current_stream().cuda_stream

    def check(offset, nbytes):
        got = bytes(memoryview(buf)[offset : offset + nbytes])
        assert got == bytes(src[offset : offset + nbytes].cpu().numpy()), (offset, nbytes)

    # copy engine: one call across all four chunks, at an odd offset
    _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(base + 7), ctypes.c_void_p(src.data_ptr() + 7), size - 7, _native.MLF_COPY_D2H, ctypes.c_void_p(stream)))
    torch.cuda.synchronize()
    for edge in (chunk, 2 * chunk, 3 * chunk):
        check(edge - 4096, 8192)
    check(7, 4096)
    check(size - 4096, 4096)
    # kernel stores into the mapping across the first chunk boundary
    memoryview(buf)[chunk - 1000 : chunk + 1000] = bytes(2000)
    _native.check(lib.mlf_copy_kernel_launch(ctypes.c_void_p(buf.get_device_ptr() + chunk - 1000), ctypes.c_void_p(src.data_ptr() + chunk - 1000), 2000, ctypes.c_void_p(stream), 4))
    torch.cuda.synchronize()
    check(chunk - 1000, 2000)

    # shrink to a size that is neither chunk- nor page-aligned: same address, still registered
    smaller = 2 * chunk + 300 * 1024 * 1024 + 123
    buf.resize(smaller)
    assert buf.get_capacity() == smaller and os.path.getsize(buf.get_id()) == smaller
    assert buf.is_cuda_registered and buf.get_data_ptr() == base
    check(2 * chunk - 4096, 8192)
    check(smaller - 4096, 4096)
    back = torch.zeros(smaller, dtype=torch.uint8, device="cuda")
    _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(back.data_ptr()), ctypes.c_void_p(base), smaller, _native.MLF_COPY_H2D, ctypes.c_void_p(stream)))
    torch.cuda.synchronize()
    assert torch.equal(back[7:], src[7:smaller])  # the first copy started at byte 7

    # grow again: registered afterwards wherever the mapping ends up, old bytes kept, new bytes zero
    buf.resize(size)
    assert buf.is_cuda_registered and buf.get_capacity() == size
    check(7, 4096)
    check(smaller - 4096, 4096)
    assert bytes(memoryview(buf)[smaller : smaller + 4096]) == bytes(4096)
    base = buf.get_data_ptr()
    _native.check(lib.mlf_memcpy_async(ctypes.c_void_p(base + smaller - 100), ctypes.c_void_p(src.data_ptr() + smaller - 100), size - smaller + 100, _native.MLF_COPY_D2H, ctypes.c_void_p(stream)))
    torch.cuda.synchronize()
    check(smaller - 100, size - smaller + 100)
    buf.close()


def test_read_tensor_per_item_api_matches_reference(tmp_path, golden_dir, engine):
    """The per-item ``read_tensor(view, req, use_optimized_loader=True)`` call of the reference API."""
    from torch.distributed.checkpoint.metadata import MetadataIndex
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem
    from torch.distributed.checkpoint.utils import _create_file_view

    rows = load_golden(golden_dir, "narrow.json")
    tensors = {f"n.{i}": cases.narrow_source(i).cuda() for i in range(len(cases.NARROW_CASES))}
    _, com, ckpt, buckets, results = _save({"tensors": tensors, "blobs": {}, "bucket_count": 1}, tmp_path, engine)
    loader = make_loader(com, copy_engine=engine)
    storage = {r.index.fqn: r.storage_data for r in results}
    with com.get_buffer(buckets[0].object_id) as stream:
        for row in rows:
            shape, dtype, offs, lens = cases.NARROW_CASES[row["i"]]
            if len(shape) == 0:
                continue
            idx = MetadataIndex(f"n.{row['i']}", torch.Size([0] * len(shape)))
            req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * len(lens)), idx, torch.Size(offs), torch.Size(lens))
            info = storage[f"n.{row['i']}"]
            got = loader.read_tensor(_create_file_view(stream, info.offset, info.length), req, use_optimized_loader=True)
            assert got.device.type == "cpu" and tuple(got.shape) == tuple(lens)
            assert tensor_bytes(got).hex() == row["hex"], row["i"]


def test_resharded_reads_of_large_tensors(tmp_path, engine):
    """Sub-block restores as a different sharding would issue them: long rows (chunked through the
    staging ring), short rows, leading-dimension ranges and strided targets, against torch slicing."""
    from torch.distributed.checkpoint.metadata import MetadataIndex
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    g = torch.Generator().manual_seed(11)
    big = torch.randint(-9999, 9999, (48, 40000), generator=g, dtype=torch.int32).cuda()
    wide = torch.randn((300, 515), generator=g).to(torch.bfloat16).cuda()
    cube = torch.randint(0, 255, (20, 33, 70), generator=g, dtype=torch.uint8).cuda()
    tensors = {"pad": torch.zeros(3, dtype=torch.uint8, device="cuda"), "big": big, "wide": wide, "cube": cube}
    _, com, ckpt, buckets, results = _save({"tensors": tensors, "blobs": {}, "bucket_count": 1}, tmp_path, engine)
    loader = make_loader(com, copy_engine=engine)
    storage = {r.index.fqn: (r.index, r.storage_data) for r in results}
    reads = [
        ("big", (0, 1000), (48, 29000)),     # rows of 116 KB: chunked rows
        ("big", (5, 0), (17, 40000)),        # leading-dimension range: one flat run
        ("big", (7, 39990), (30, 10)),       # 40-byte rows
        ("wide", (10, 3), (200, 500)),
        ("wide", (0, 0), (300, 515)),
        ("cube", (3, 4, 5), (10, 20, 60)),
    ]
    for fqn, offs, lens in reads:
        idx, info = storage[fqn]
        source = tensors[fqn]
        want = source[tuple(slice(o, o + n) for o, n in zip(offs, lens))]
        for strided in (False, True):
            if strided and len(lens) == 2:
                target = torch.zeros((lens[1], lens[0]), dtype=source.dtype, device="cuda").t()
            else:
                target = torch.zeros(lens, dtype=source.dtype, device="cuda")
            req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0] * len(lens)), idx, torch.Size(offs), torch.Size(lens))

            class _Planner:
                def resolve_tensor(self, r):
                    return target

                def commit_tensor(self, r, t):
                    pass

            loader.read_data(buckets[0].object_id, [req], _Planner(), {idx: info})
            torch.cuda.synchronize()
            assert torch.equal(target, want), (fqn, offs, lens, strided)


def test_single_tensor_larger_than_4_gib(shm_path, engine):
    """64-bit offsets inside one segment: a 4.5 GiB tensor behind an odd-sized prefix."""
    import numpy as np

    free_dev = torch.cuda.mem_get_info()[0]
    free_shm = os.statvfs(str(shm_path)).f_bavail * os.statvfs(str(shm_path)).f_frsize
    n = (9 << 29) + 12345  # 4.5 GiB and a bit
    if free_dev < 3 * n or free_shm < 2 * n:
        pytest.skip("not enough memory for a > 4 GiB object on this box")
    huge = torch.empty(n, dtype=torch.uint8, device="cuda")
    huge.random_(0, 256)
    tensors = {"pad": torch.arange(7, dtype=torch.uint8, device="cuda"), "huge": huge}
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager

    CheckpointObjectManager._worker_pool = None
    _, com, ckpt, buckets, results = _save({"tensors": tensors, "blobs": {}, "bucket_count": 1}, shm_path, engine, initial_buffer_size_bytes=n + (1 << 20))
    info = {r.index.fqn: r.storage_data for r in results}["huge"]
    header = len(oracle.header_bytes("uint8", (n,)))
    mapped = np.memmap(str(buckets[0].object_id), dtype=np.uint8, mode="r")
    payload_at = 4096 + info.offset + header
    assert info.length == header + n and mapped.shape[0] == 4096 + info.offset + info.length
    # spot checks around the 4 GiB boundary, both ends and tile edges, then a strided full compare on the GPU
    host = huge.cpu().numpy()
    for at in (0, 65535, 65536, (1 << 32) - 70000, (1 << 32) - 1, 1 << 32, (1 << 32) + 65537, n - 4097, n - 1):
        lo, hi = max(0, at - 100), min(n, at + 100)
        assert bytes(mapped[payload_at + lo : payload_at + hi]) == bytes(host[lo:hi]), at
    back = torch.zeros(n, dtype=torch.uint8, device="cuda")
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    idx = {r.index.fqn: r.index for r in results}["huge"]
    req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0]), idx, torch.Size([0]), torch.Size([n]))

    class _Planner:
        def resolve_tensor(self, r):
            return back

        def commit_tensor(self, r, t):
            pass

    make_loader(com, copy_engine=engine).read_data(buckets[0].object_id, [req], _Planner(), {idx: info})
    torch.cuda.synchronize()
    assert torch.equal(back, huge)


def test_legacy_torch_save_format_on_the_gpu(shm_path, engine):
    """``use_optimized_save=False``: every tensor travels as a ``torch.save`` stream under the
    ``TORCH___`` signature, moved by the same pack kernel as byte items; the loader reads the streams
    back (reference: core/checkpoint_saver.py:665-673, core/checkpoint_loader.py:212-218)."""
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    case = case_to_device(cases.CASES["mixed"](), "cuda")
    _, com, ckpt, buckets, results = _save(case, shm_path, engine, use_optimized_save=False)
    raw = open(str(buckets[0].object_id), "rb").read()
    assert raw[8:16] == b"TORCH___"
    assert int.from_bytes(raw[:8], "little") == len(raw) - 4096
    # every tensor item is a self-contained torch.save stream holding the tensor's values
    import io

    by_fqn = {r.index.fqn: r for r in results}
    for fqn, t in case["tensors"].items():
        info = by_fqn[fqn].storage_data
        stored = torch.load(io.BytesIO(raw[4096 + info.offset : 4096 + info.offset + info.length]), map_location="cpu", weights_only=True)
        assert tensor_bytes(stored) == tensor_bytes(t), fqn
    loader = make_loader(com, copy_engine=engine)
    storage = {r.index: r.storage_data for r in results}
    targets, blobs, reqs = {}, {}, []
    for r in results:
        fqn = r.index.fqn
        if fqn in case["blobs"]:
            reqs.append(ReadItem(LoadItemType.BYTE_IO, r.index, None, r.index, None, None))
            continue
        t = case["tensors"][fqn]
        if t.numel() == 0:
            continue
        targets[fqn] = torch.zeros(t.shape, dtype=t.dtype, device="cuda")
        reqs.append(ReadItem(LoadItemType.TENSOR, r.index, torch.Size([0] * t.dim()), r.index, torch.Size([0] * t.dim()), torch.Size(t.shape)))

    class _Planner:
        def resolve_tensor(self, req):
            return targets[req.dest_index.fqn]

        def commit_tensor(self, req, tensor):
            pass

        def load_bytes(self, req, value):
            blobs[req.dest_index.fqn] = value.read()

    loader.read_data(buckets[0].object_id, reqs, _Planner(), storage)
    torch.cuda.synchronize()
    for fqn, target in targets.items():
        assert tensor_bytes(target) == tensor_bytes(case["tensors"][fqn]), fqn
    assert blobs == dict(case["blobs"])


def test_restore_converts_when_the_target_dtype_differs(tmp_path, engine):
    """An fp32 checkpoint loaded into bf16 parameters: the reference's ``target.copy_(tensor)`` converts
    (core/checkpoint_loader.py:331-336); here the block is unpacked in its stored dtype and converted."""
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    src = torch.randn(37, 53, device="cuda")
    _, com, ckpt, buckets, results = _save({"tensors": {"w": src}, "blobs": {}, "bucket_count": 1}, tmp_path, engine)
    loader = make_loader(com, copy_engine=engine)
    idx = results[0].index
    for device in ("cuda", "cpu"):
        target = torch.zeros(5, 53, dtype=torch.bfloat16, device=device)
        req = ReadItem(LoadItemType.TENSOR, idx, torch.Size([0, 0]), idx, torch.Size([3, 0]), torch.Size([5, 53]))

        class _Planner:
            def resolve_tensor(self, r):
                return target

            def commit_tensor(self, r, t):
                pass

        loader.read_data(buckets[0].object_id, [req], _Planner(), {idx: results[0].storage_data})
        assert torch.equal(target.cpu(), src[3:8].to(torch.bfloat16).cpu())


@pytest.mark.parametrize("offset,trim", [(4096, 0), (4096 + 48, 12345)])
def test_hybrid_restore_read_moves_exactly_the_files_bytes(shm_path, offset, trim):
    """Restore feed with the lock lane beside the pread() threads: whatever share either side
    takes, HBM ends up holding exactly the requested bytes of the object, for page-aligned and
    ragged ends alike; with the file made read-only the lane cannot start and the threads move all."""
    from ml_flashpoint import _native
    from ml_flashpoint.checkpoint_object_manager.buffer_object.buffer_object_ext import BufferObject

    nbytes = (192 << 20) + 4096 + 777
    data = np.random.default_rng(5).integers(0, 256, nbytes, dtype=np.uint8)
    path = str(shm_path / "object.bin")
    data.tofile(path)
    want = torch.from_numpy(data[offset : nbytes - trim])
    for writable in (True, False):
        os.chmod(path, 0o644 if writable else 0o444)
        obj = BufferObject(path)
        got = torch.zeros(want.numel(), dtype=torch.uint8, device="cuda")
        lane = obj.read_to_device(offset, got.data_ptr(), want.numel(), threads=3, lock_run_mib=16)
        torch.cuda.synchronize()
        assert torch.equal(got.cpu(), want)
        assert 0 <= lane <= want.numel()
        if not writable and os.geteuid() != 0:
            assert lane == 0
        obj.close()
    assert int(_native.lib().mlf_last_lock_lane_bytes()) >= 0


@pytest.fixture(scope="module")
def bounded_engine():
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    return CudaCopyEngine(mode="staged", arena_limit_bytes=16 << 10)


@pytest.mark.parametrize("pooled", [False, True])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_bounded_arena_saves_reference_bytes_and_restores_them(name, pooled, shm_path, golden_dir, bounded_engine):
    """With the image arena capped (here at 16 KiB, so every golden object takes several pieces) a
    save is packed and drained piece by piece through two arena halves, into a page-locked pool file
    or a plain file: same object bytes, same records, and the piecewise restore gives the tensors back."""
    from torch.distributed.checkpoint.planner import LoadItemType, ReadItem

    from ml_flashpoint.core.buffer_pool import BufferPoolConfig

    gold = load_golden(golden_dir, f"{name}.json")
    case = case_to_device(cases.CASES[name](), "cuda")
    kw = {}
    if pooled:
        kw["pool_config"] = BufferPoolConfig(str(shm_path / "pool"), 0, 2, 1 << 20, register_cuda=True)
    saver, com, ckpt, buckets, results = _save(case, shm_path, bounded_engine, **kw)
    try:
        for bucket, g in zip(buckets, gold["objects"]):
            with open(str(bucket.object_id), "rb") as f:
                data = f.read()
            assert len(data) == g["size"] and hashlib.sha256(data).hexdigest() == g["sha256"], bucket.object_name
        got = sorted((r.storage_data.relative_path, r.storage_data.offset, r.storage_data.length) for r in results)
        assert got == [(w["relative_path"], w["offset"], w["length"]) for w in gold["write_results"]]
        assert bounded_engine.held_device_bytes() <= max(1 << 20, 2 * max(t.numel() * t.element_size() for t in case["tensors"].values()) + 4096)

        loader = make_loader(com, copy_engine=bounded_engine)
        storage = {r.index: r.storage_data for r in results}
        targets, per_object = {}, {}
        for r in results:
            fqn = r.index.fqn
            if fqn in case["blobs"]:
                continue
            t = case["tensors"][fqn]
            if t.numel() == 0:
                continue
            targets[fqn] = torch.zeros(t.shape, dtype=t.dtype, device="cuda")
            req = ReadItem(LoadItemType.TENSOR, r.index, torch.Size([0] * t.dim()), r.index, torch.Size([0] * t.dim()), torch.Size(t.shape))
            per_object.setdefault(r.storage_data.relative_path, []).append(req)

        class _Planner:
            def resolve_tensor(self, req):
                return targets[req.dest_index.fqn]

            def commit_tensor(self, req, tensor):
                pass

        for bucket in buckets:
            loader.read_data(bucket.object_id, per_object.get(bucket.object_name, []), _Planner(), storage)
        torch.cuda.synchronize()
        for fqn, target in targets.items():
            assert tensor_bytes(target) == tensor_bytes(case["tensors"][fqn]), fqn
    finally:
        com.teardown_pool()


def test_bounded_arena_at_size_keeps_the_arena_small(shm_path):
    """256 MB of tensors through a 32 MiB arena into a page-locked pool file: the arena never grows
    past its bound (two halves of 16 MiB), the object equals the unbounded engine's byte for byte."""
    from ml_flashpoint.core.buffer_pool import BufferPoolConfig
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    g = torch.Generator(device="cuda").manual_seed(11)
    tensors = {f"t{i}": torch.randint(0, 1 << 30, (n,), device="cuda", dtype=torch.int32, generator=g)
               for i, n in enumerate([1 << 20, 3 << 20, 1 << 18, 2 << 20, 5, 4 << 20, 1 << 22] * 4)}
    case = {"tensors": tensors, "blobs": {"cfg": b"x" * 333}, "bucket_count": 1}
    digests = []
    for limit in (0, 32 << 20):
        engine = CudaCopyEngine(mode="staged", arena_limit_bytes=limit)
        pool = BufferPoolConfig(str(shm_path / f"pool{limit}"), 0, 1, 300 << 20, register_cuda=True)
        saver, com, ckpt, buckets, results = _save(case, shm_path / f"run{limit}", engine, pool_config=pool, initial_buffer_size_bytes=300 << 20)
        try:
            with open(str(buckets[0].object_id), "rb") as f:
                digests.append(hashlib.sha256(f.read()).hexdigest())
            if limit:
                assert engine.held_device_bytes() <= limit + 8192
            else:
                assert engine.held_device_bytes() >= sum(t.numel() * 4 for t in tensors.values())
        finally:
            com.teardown_pool()
    assert digests[0] == digests[1]


def _pack_and_unpack_against_oracle(views, first_offset=3):
    """Packs ``views`` with one plan, compares every byte of the image with the oracle's payloads,
    then unpacks into zeroed twins of the views' storages and compares those with the sources."""
    from ml_flashpoint import _native
    from ml_flashpoint.core.gpu_engine import _Plan, c_strides, fill_desc

    n = len(views)
    descs = (_native.CopyDesc * n)()
    offsets, at = [], first_offset
    for i, v in enumerate(views):
        offsets.append(at)
        at += v.numel() * v.element_size() + 7 + (i % 16)
    image = torch.full((at + 64,), 0xC3, dtype=torch.uint8, device="cuda")
    for i, v in enumerate(views):
        fill_desc(descs[i], v.data_ptr(), offsets[i], v.element_size(), v.shape, v.stride(), c_strides(v.shape))
    stream = torch.cuda.current_stream().cuda_stream
    plan = _Plan(descs, n, _native.MLF_PACK)
    plan.launch(image.data_ptr(), image.numel(), stream)
    torch.cuda.synchronize()
    plan.status()
    expect = bytearray(b"\xc3" * image.numel())
    for v, o in zip(views, offsets):
        payload = oracle.tensor_payload(v.cpu())
        expect[o : o + len(payload)] = payload
    got = image.cpu().numpy().tobytes()
    if got != bytes(expect):
        bad = next(i for i in range(len(got)) if got[i] != expect[i])
        which = max(k for k, o in enumerate(offsets) if o <= bad)
        pytest.fail(f"byte {bad} differs, view {which}: shape {tuple(views[which].shape)} stride {views[which].stride()} {views[which].dtype}")
    targets, bases = [], []
    for v in views:
        base = torch.zeros_like(v._base)
        bases.append(base)
        targets.append(base.as_strided(v.shape, v.stride(), v.storage_offset()))
    for i, t in enumerate(targets):
        fill_desc(descs[i], t.data_ptr(), offsets[i], t.element_size(), t.shape, t.stride(), c_strides(t.shape))
    plan = _Plan(descs, n, _native.MLF_UNPACK)
    plan.launch(image.data_ptr(), image.numel(), stream)
    torch.cuda.synchronize()
    plan.status()
    for k, (v, base) in enumerate(zip(views, bases)):
        want = torch.zeros_like(base)
        want.as_strided(v.shape, v.stride(), v.storage_offset()).copy_(v)
        assert torch.equal(base, want), f"view {k}: shape {tuple(v.shape)} stride {v.stride()} {v.dtype}"


@pytest.mark.parametrize("dtype", [torch.uint8, torch.int16, torch.int32, torch.int64], ids=lambda d: str(d).split(".")[-1])
def test_wide_transposes_in_vector_form_at_every_edge(dtype):
    """Wide transposed views (image rows of 256 bytes or more) move through 16-byte granules on the
    tensor side. Extents straddle the tile (112 bytes along the tensor's contiguous dimension, 128 and
    512 elements along the image rows); row pitches and column offsets put the tensor rows on every
    residue class of 16 bytes, so granules are shifted, partial at both ends, or exactly aligned."""
    g = torch.Generator().manual_seed(29)
    esize = torch.empty((), dtype=dtype).element_size()
    per = 112 // esize  # image rows per tile
    views = []
    for n_c, n_l, pitch_extra, off in [
        (1, 300, 0, 0), (1, 300, 3, 1), (per - 1, 129, 1, 1), (per, 512, 0, 0), (per + 1, 513, 5, 3),
        (2 * per + 1, 700, 7, 5), (3, 1100, 13, 2), (per, 128, 16 // esize, 0), (5 * per, 384, 16 // esize, 16 // esize),
    ]:
        n_l = max(n_l, 256 // esize)  # keep the image rows wide
        base = torch.randint(0, 250, (n_l, n_c + off + pitch_extra), generator=g, dtype=torch.int64).to(dtype).cuda()
        views.append(base[:, off : off + n_c].t())
    views.append(torch.randint(0, 250, (2, 600, 70), generator=g, dtype=torch.int64).to(dtype).cuda().transpose(1, 2))  # batched
    _pack_and_unpack_against_oracle(views)


@pytest.mark.parametrize("dtype", [torch.int16, torch.int32], ids=["16bit", "32bit"])
def test_transposes_in_matrix_form_at_every_edge(dtype):
    """16- and 32-bit transposed views whose tensor rows all start on 16-byte boundaries go through
    warp-level matrix loads (blocks of 32 rows by one granule) and a per-row carry between stages of
    128 rows. Extents straddle the tile (128 bytes along the tensor's contiguous dimension, 128 and
    1024 elements along the image rows), images start on every byte residue, and batched and
    column-offset views are in the mix. The second group has rows that start on 4-byte boundaries
    only (every residue of 4 within a granule): those stages are fed by 4-byte copies."""
    g = torch.Generator().manual_seed(31)
    esize = torch.empty((), dtype=dtype).element_size()
    cols, gran, word = 128 // esize, 16 // esize, 4 // esize  # elements per tile row / 16-byte granule / 4-byte word

    def base(rows, pitch):
        return torch.randint(-30000, 30000, (rows, pitch), generator=g, dtype=torch.int64).to(dtype).cuda()

    views = []
    for n_c, n_l, pitch, off in [
        (cols, 1024, cols, 0), (cols - 1, 1023, cols, 0), (cols + 1, 1025, cols + gran, 0), (1, 128, gran, 0),
        (7, 129, 2 * gran, gran), (2 * cols, 2049, 2 * cols + gran, gran), (200, 300, 208, 0), (cols, 127, cols, 0),
        (300, 5000, 304, 0), (cols, 135, cols, 0), (33, 1030, 40, 0),
        # word-aligned rows
        (cols, 1024, cols + word, 0), (cols - 1, 1023, cols + 3 * word, word), (cols + 1, 1025, cols + gran + word, 2 * word),
        (1, 128, word, 0), (5, 129, 2 * gran + word, 3 * word), (2 * cols + 1, 2049, 2 * cols + gran, word),
        (200, 300, 200 + 2 * word, word), (300, 5000, 302 + word * (esize // 4), 0), (33, 1030, 33 + (33 * esize % 4) // esize, 0),
    ]:
        views.append(base(n_l, pitch)[:, off : off + n_c].t())
    float_dtype = torch.bfloat16 if esize == 2 else torch.float32
    views.append(torch.randint(-9, 9, (3, 700, 80), generator=g, dtype=torch.int64).to(float_dtype).cuda().transpose(1, 2))
    for first_offset in (0, 1, 2, 9, 15):
        _pack_and_unpack_against_oracle(views, first_offset=first_offset)


def test_narrow_transposed_rows_across_tiles_and_alignments():
    """Transposed views whose image rows are shorter than 256 bytes: the tensor side is read in
    aligned 16-byte granules, several sub-tiles ahead. Extents span several tiles of sixteen
    sub-tiles with ragged last tiles and sub-tiles; column offsets and odd pitches put the tensor
    rows on every residue of 16 bytes; images start on odd bytes."""
    g = torch.Generator().manual_seed(37)

    def base(rows, pitch, dtype):
        return torch.randint(0, 250, (rows, pitch), generator=g, dtype=torch.int64).to(dtype).cuda()

    views = []
    for dtype, n_l, n_c, extra, off in [
        (torch.int16, 3, 50001, 0, 0), (torch.int16, 2, 70000, 3, 1), (torch.int16, 82, 3000, 5, 3), (torch.int16, 1, 40000, 1, 1),
        (torch.int16, 127, 1500, 0, 0), (torch.int32, 19, 9000, 1, 1), (torch.int32, 3, 40000, 0, 0), (torch.int32, 63, 700, 2, 1),
        (torch.int64, 12, 30011, 1, 0), (torch.int64, 5, 20000, 0, 0), (torch.uint8, 7, 60013, 5, 2), (torch.uint8, 100, 5000, 9, 7),
        (torch.int16, 8, 33, 0, 0), (torch.int32, 2, 1, 0, 0),
        # 32- and 64-bit rows of up to 127 elements take the same form
        (torch.int32, 92, 3000, 0, 0), (torch.int32, 127, 900, 3, 1), (torch.int64, 100, 700, 1, 1), (torch.int64, 127, 300, 0, 0),
        (torch.int32, 128, 600, 0, 0),
    ]:
        views.append(base(n_l, n_c + off + extra, dtype)[:, off : off + n_c].t())
    views.append(torch.randint(0, 250, (37, 11, 700), generator=g, dtype=torch.int64).to(torch.int16).cuda().transpose(1, 2))  # batched
    views.append(torch.randint(0, 250, (5, 3, 30000), generator=g, dtype=torch.int64).to(torch.int32).cuda().transpose(1, 2))
    for first_offset in (0, 1, 7):
        _pack_and_unpack_against_oracle(views, first_offset=first_offset)
