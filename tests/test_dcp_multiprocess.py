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


def test_gpt2_shaped_objects_equal_the_oracle_two_gloo_ranks(tmp_path):
    """The GPT-2 + Adam configuration, scaled down, on the CPU: what each rank wrote equals the oracle's
    bytes for the items the planner assigned to it (the full-size run is in the GPU suite)."""
    result = str(tmp_path / "gpt2_scaled")
    mp.spawn(dcp_worker.run_gpt2_small, args=(2, str(tmp_path), _free_port(), result, "numpy", False), nprocs=2, join=True)
    outcomes = [ast.literal_eval(open(f"{result}.{r}").read()) for r in range(2)]
    assert all(o["ok"] for o in outcomes), outcomes
    assert all(o["items_in_my_object"] > 0 for o in outcomes)


@pytest.mark.gpu
def test_dcp_async_save_with_cuda_engine(shm_path):
    """The same through the CUDA engine with the state in HBM: ``stage`` snapshots on the device,
    the pack kernel reads the snapshot, the zeroed originals do not leak into the object."""
    result = str(shm_path / "async_result")
    mp.spawn(dcp_worker.run_async_save, args=(str(shm_path), _free_port(), result, "cuda"), nprocs=1, join=True)
    assert ast.literal_eval(open(result).read())["ok"]


@pytest.mark.gpu
def test_gpt2_small_with_adam_at_full_size_two_ranks(shm_path):
    """The CPU-runnable benchmark configuration at its stated size (124 M parameters, fp32 weights and
    Adam moments, 1.49 GB, every rank a full replica, world size 2) through the DCP adapter with the
    CUDA engine: every rank's object equals the oracle's bytes for the items the planner gave it,
    and the state loads back bit-exactly."""
    result = str(shm_path / "gpt2_small")
    mp.spawn(dcp_worker.run_gpt2_small, args=(2, str(shm_path), _free_port(), result), nprocs=2, join=True)
    outcomes = [ast.literal_eval(open(f"{result}.{r}").read()) for r in range(2)]
    assert all(o["ok"] for o in outcomes), outcomes
    assert outcomes[0]["state_bytes"] > 1.49e9
    # replicated tensors are written once: the two objects together hold the state once
    assert abs(sum(o["object_bytes"] for o in outcomes) - outcomes[0]["state_bytes"]) < 2e6
