"""The allocation-free pack entry point against the regular plan path.

``mlf_pack_noalloc`` exists for savers that must run when the process cannot get any more device
memory (an emergency checkpoint after an out-of-memory error; a trainer whose caching allocator owns
the whole GPU): it keeps its tables in a fixed array inside the library instead of allocating them.
The array is shared by all calls and keeps the previous call's contents, so the check is done on
two calls in a row with different descriptor sets: each must produce exactly the bytes that
``mlf_plan_create`` + ``mlf_plan_launch`` produce for the same descriptors (byte work: bit-exact).

This file sorts last on purpose, so that a run stopping at the first failure has already run every
other test; it also passes when run alone in a fresh process.
"""

import ctypes

import pytest
import torch

import mlf_oracle as oracle

pytestmark = pytest.mark.gpu


def _descs_for(tensors, offsets):
    from ml_flashpoint import _native
    from ml_flashpoint.core.gpu_engine import c_strides, fill_desc

    descs = (_native.CopyDesc * len(tensors))()
    for k, (t, off) in enumerate(zip(tensors, offsets)):
        fill_desc(descs[k], t.data_ptr(), off, t.element_size(), t.shape, t.stride(), c_strides(t.shape))
    return descs


def _layout(tensors, first_offset):
    offsets, pos = [], first_offset
    for t in tensors:
        offsets.append(pos)
        pos += t.numel() * t.element_size() + 5  # odd gaps: every payload lands on a new byte residue
    return offsets, pos


def _tensor_sets():
    g = torch.Generator().manual_seed(2024)

    def rnd(shape, dtype):
        return torch.randint(-100, 100, shape, generator=g, dtype=torch.int64).to(dtype).cuda()

    first = [
        rnd((300000,), torch.int32),  # flat, several tiles
        rnd((129, 257), torch.int16).t(),  # transposed view
        rnd((64, 1000), torch.int64)[:, 10:900],  # row-sliced view
        rnd((7,), torch.uint8),
        rnd((33, 5, 9), torch.int32)[::2],  # stepped view: element-wise path
    ]
    second = [
        rnd((70001,), torch.uint8),
        rnd((3, 40, 50), torch.int16).permute(2, 0, 1),
        rnd((500000,), torch.int64),
    ]
    return first, second


def _pack_with_plan(descs, n, image):
    from ml_flashpoint import _native

    lib = _native.lib()
    plan = ctypes.c_void_p()
    _native.check(lib.mlf_plan_create(descs, n, _native.MLF_PACK, ctypes.byref(plan)))
    try:
        _native.check(lib.mlf_plan_launch(plan, ctypes.c_void_p(image.data_ptr()), image.numel(), None, 0))
        torch.cuda.synchronize()
        _native.check(lib.mlf_plan_status(plan))
    finally:
        lib.mlf_plan_destroy(plan)


def test_noalloc_pack_matches_plan_pack_on_consecutive_calls():
    from ml_flashpoint import _native

    lib = _native.lib()
    torch.cuda.synchronize()
    for tensors, first_offset in zip(_tensor_sets(), (3, 17)):
        offsets, total = _layout(tensors, first_offset)
        descs = _descs_for(tensors, offsets)
        want = torch.full((total + 64,), 0x5A, dtype=torch.uint8, device="cuda")
        got = torch.full((total + 64,), 0x5A, dtype=torch.uint8, device="cuda")
        _pack_with_plan(descs, len(tensors), want)
        _native.check(lib.mlf_pack_noalloc(descs, len(tensors), ctypes.c_void_p(got.data_ptr()), got.numel(), None))
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert int((want != 0x5A).sum()) > 0  # the reference image was actually written
        # and directly against the CPU oracle: every payload is the tensor's logical C-order bytes
        image = bytes(got.cpu().numpy())
        for t, off in zip(tensors, offsets):
            raw = oracle.tensor_payload(t.cpu())
            assert image[off : off + len(raw)] == raw


def test_noalloc_pack_on_a_stream_of_the_callers():
    """The tables are uploaded on the caller's stream ahead of the kernel, so a non-default stream
    works the same; the call may wait for earlier work on that stream (pageable upload)."""
    from ml_flashpoint import _native

    lib = _native.lib()
    side = torch.cuda.Stream()
    tensors, _ = _tensor_sets()
    offsets, total = _layout(tensors, 9)
    descs = _descs_for(tensors, offsets)
    want = torch.zeros(total + 64, dtype=torch.uint8, device="cuda")
    got = torch.zeros(total + 64, dtype=torch.uint8, device="cuda")
    _pack_with_plan(descs, len(tensors), want)
    torch.cuda.synchronize()  # the inputs were produced on the default stream
    for _ in range(2):
        got.zero_()
        torch.cuda.synchronize()
        _native.check(lib.mlf_pack_noalloc(descs, len(tensors), ctypes.c_void_p(got.data_ptr()), got.numel(), ctypes.c_void_p(side.cuda_stream)))
        side.synchronize()
        assert torch.equal(got, want)


def test_noalloc_pack_rejects_oversized_and_out_of_window_requests():
    from ml_flashpoint import _native

    lib = _native.lib()
    t = torch.zeros(16, dtype=torch.uint8, device="cuda")
    image = torch.zeros(64, dtype=torch.uint8, device="cuda")
    too_many = _native.MLF_NOALLOC_MAX_DESCS + 1
    descs = _descs_for([t] * too_many, [0] * too_many)
    rc = lib.mlf_pack_noalloc(descs, too_many, ctypes.c_void_p(image.data_ptr()), image.numel(), None)
    assert rc == _native.MLF_ERR_TOO_LARGE
    assert b"at most" in lib.mlf_last_error()
    descs = _descs_for([t], [60])
    rc = lib.mlf_pack_noalloc(descs, 1, ctypes.c_void_p(image.data_ptr()), image.numel(), None)
    assert rc == _native.MLF_ERR_BOUNDS
    torch.cuda.synchronize()
    assert int(image.sum()) == 0
