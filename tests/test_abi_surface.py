"""The C-ABI library loads without a GPU and exports every entry point the header declares."""

import ctypes
import os
import re

import pytest

import conftest


def _declared_functions():
    with open(os.path.join(conftest.REPO_ROOT, "include", "mlf_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(mlf_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_entry_point_is_exported_and_bound():
    from ml_flashpoint import _native

    lib = _native.lib()
    declared = _declared_functions()
    assert len(declared) >= 40
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in mlf_b200.h but not exported"
    assert set(declared) == set(_native.EXPORTED_SYMBOLS)


def test_version_and_error_text():
    from ml_flashpoint import _native

    lib = _native.lib()
    assert b"sm_100a" in lib.mlf_version()
    out = ctypes.c_void_p()
    rc = lib.mlf_buf_open_ro(b"/definitely/not/here", ctypes.byref(out))
    assert rc == _native.MLF_ERR_IO
    assert b"No such file" in lib.mlf_last_error()
    with pytest.raises(_native.NativeError) as info:
        _native.check(rc)
    assert info.value.code == _native.MLF_ERR_IO


def test_plan_validation_happens_before_any_device_work():
    from ml_flashpoint import _native

    lib = _native.lib()
    plan = ctypes.c_void_p()
    desc = (_native.CopyDesc * 1)()
    desc[0].tensor_ptr = 4096
    desc[0].elem_size = 3  # not a supported element size
    desc[0].ndim = 1
    desc[0].shape[0] = 4
    desc[0].tensor_stride[0] = 1
    desc[0].image_stride[0] = 1
    assert lib.mlf_plan_create(desc, 1, _native.MLF_PACK, ctypes.byref(plan)) == _native.MLF_ERR_INVALID
    assert b"elem_size" in lib.mlf_last_error()
    desc[0].elem_size = 4
    desc[0].ndim = 9
    assert lib.mlf_plan_create(desc, 1, _native.MLF_PACK, ctypes.byref(plan)) == _native.MLF_ERR_INVALID
    desc[0].ndim = 1
    desc[0].tensor_stride[0] = -1
    assert lib.mlf_plan_create(desc, 1, _native.MLF_PACK, ctypes.byref(plan)) == _native.MLF_ERR_INVALID
    desc[0].tensor_stride[0] = 1
    desc[0].tensor_ptr = 4098  # misaligned for 4-byte elements
    assert lib.mlf_plan_create(desc, 1, _native.MLF_PACK, ctypes.byref(plan)) == _native.MLF_ERR_INVALID
    assert lib.mlf_plan_create(desc, 1, 7, ctypes.byref(plan)) == _native.MLF_ERR_INVALID
    assert lib.mlf_plan_image_extent(None) == 0


def test_plan_rejects_shapes_whose_byte_arithmetic_overflows():
    """Caller-supplied shapes and strides are multiplied with overflow checks: an extent that wraps
    around 2^64 must never pass the image-capacity guard of a launch."""
    from ml_flashpoint import _native

    lib = _native.lib()
    plan = ctypes.c_void_p()

    def desc(shape, tstride, istride, esize=8, image_off=0):
        d = (_native.CopyDesc * 1)()
        d[0].tensor_ptr = 1 << 20
        d[0].image_off = image_off
        d[0].elem_size = esize
        d[0].ndim = len(shape)
        for k, (n, ts, st) in enumerate(zip(shape, tstride, istride)):
            d[0].shape[k], d[0].tensor_stride[k], d[0].image_stride[k] = n, ts, st
        return d

    big = (1 << 62) + 1
    cases = [
        desc((1 << 31, 1 << 31, 4), (1 << 33, 4, 1), (1 << 33, 4, 1)),        # numel * elem_size wraps
        desc((2, 2), (1, 1), (big, 1)),                                          # image span wraps
        desc((2, 2), (big, 1), (2, 1)),                                          # tensor span wraps
        desc((4,), (1,), (1,), esize=4, image_off=(1 << 64) - 8),               # image_off + extent wraps
        desc((1 << 40, 1 << 21), (1 << 21, 1), (1 << 21, 1), esize=16),         # beyond the 2^62 byte bound
    ]
    for d in cases:
        assert lib.mlf_plan_create(d, 1, _native.MLF_PACK, ctypes.byref(plan)) == _native.MLF_ERR_INVALID
        assert b"overflow" in lib.mlf_last_error()
    # an empty box is still fine whatever its other extents are
    empty = desc((0, 1 << 62), (1, 1), (1, 1))
    rc = lib.mlf_plan_create(empty, 1, _native.MLF_PACK, ctypes.byref(plan))
    assert rc in (0, _native.MLF_ERR_CUDA)  # validation passed; without a device the plan stops at cudaGetDevice
    if rc == 0:
        lib.mlf_plan_destroy(plan)


def test_copy_desc_layout_matches_header():
    from ml_flashpoint import _native

    # 8 + 8 + 4 + 4 + 3 * 8 * 8
    assert ctypes.sizeof(_native.CopyDesc) == 216
    assert _native.CopyDesc.shape.offset == 24
    assert _native.CopyDesc.image_stride.offset == 24 + 128


def test_engine_refuses_to_run_without_cuda():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from ml_flashpoint.core.gpu_engine import CudaCopyEngine

    with pytest.raises(RuntimeError, match="no CPU data path"):
        CudaCopyEngine()
