"""Shared pytest configuration: marker registration and import paths."""

import os
import sys

import pytest

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE_ROOT = os.path.join(REPO_ROOT, "ml-flashpoint_b200")
GOLDEN_DIR = os.path.join(REPO_ROOT, "tests", "golden")

for _p in (REPO_ROOT, PACKAGE_ROOT, GOLDEN_DIR, os.path.join(REPO_ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

os.environ.setdefault("MLFLASHPOINT_LOG_LEVEL", "WARNING")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture
def golden_dir():
    return GOLDEN_DIR


@pytest.fixture
def shm_path():
    """Scratch directory on tmpfs: page-locking a file mapping for CUDA only works for memory-backed files."""
    import pathlib
    import shutil
    import tempfile

    root = "/dev/shm" if os.path.isdir("/dev/shm") else None
    path = tempfile.mkdtemp(prefix="mlf_test_", dir=root)
    try:
        yield pathlib.Path(path)
    finally:
        shutil.rmtree(path, ignore_errors=True)
