"""dcp.save / dcp.load through MemoryStorageWriter / MemoryStorageReader with two gloo ranks.

This is the CPU-runnable configuration (GPT-2-shaped state plus Adam moments, every rank holding a
full replica, scaled down): it exercises the multi-rank host path - plan reduce-scatter, per-rank
object naming, write-result gather, coordinator metadata - with the numpy stand-in engine. The same
worker runs with the CUDA engine in the GPU suite.
"""

import ast
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

import dcp_worker


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(tmp_path, engine_kind, world=2):
    result = str(tmp_path / "result")
    mp.spawn(dcp_worker.run_rank, args=(world, str(tmp_path), _free_port(), engine_kind, result), nprocs=world, join=True)
    return [ast.literal_eval(open(f"{result}.{r}").read()) for r in range(world)]


def test_dcp_round_trip_two_gloo_ranks_on_cpu(tmp_path):
    outcomes = _run(tmp_path, "numpy")
    for o in outcomes:
        assert o["ok"], o
        assert o["markers"] == []  # finalize removed both ranks' dirty markers
    listing = outcomes[0]["listing"]
    assert ".metadata" in listing
    # replicated tensors are deduplicated by the planner: both ranks wrote an object of their own
    assert "__0__0_src0.distcp" in listing and "__1__0_src1.distcp" in listing


@pytest.mark.gpu
def test_dcp_round_trip_two_ranks_with_cuda_engine(shm_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    outcomes = _run(shm_path, "cuda")
    assert all(o["ok"] for o in outcomes), outcomes


def test_dcp_async_save_snapshots_the_state(tmp_path):
    """``MemoryStorageWriter.stage`` must snapshot: tensors zeroed right after ``async_save`` returns
    still load back with their old values."""
    result = str(tmp_path / "async_result")
    mp.spawn(dcp_worker.run_async_save, args=(str(tmp_path), _free_port(), result), nprocs=1, join=True)
    assert ast.literal_eval(open(result).read())["ok"]
