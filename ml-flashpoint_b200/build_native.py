"""Builds libmlf_b200.so (the C-ABI over the sm_100a kernels) in-tree with nvcc.

Usage: ``python build_native.py [--force] [--verbose]``. The library lands next to the Python
package (``ml_flashpoint/libmlf_b200.so``) so that a source checkout is directly importable.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OUT = os.path.join(HERE, "ml_flashpoint", "libmlf_b200.so")
SOURCES = ["buffer_object.cpp", "plan.cu", "movers.cu"]
HEADERS = ["common.h", "copy_device.cuh", "bulk_pipeline.cuh", "plan_seg.cuh", "transpose_tiles.cuh"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return found


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(INCLUDE, "mlf_b200.h"), __file__]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, out: str = OUT, defines: tuple = ()) -> str:
    """Builds the library. ``defines`` (e.g. ``("MLF_RING_STAGES=8",)``) and ``out`` produce tuning
    variants next to the default build; load one with the ``MLF_B200_LIB`` environment variable."""
    if out == OUT and not defines and not force and not _stale():
        return OUT
    cmd = [
        _nvcc(),
        "-gencode",
        "arch=compute_100a,code=sm_100a",
        "-O3",
        "-std=c++17",
        "-lineinfo",
        "-shared",
        "-Xcompiler",
        "-fPIC,-Wall,-Wextra",
        "-x",
        "cu",
        "-I",
        INCLUDE,
        "-I",
        CSRC,
        "-DMLF_BUILD",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [f"-D{d}" for d in defines]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-o", out, "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
