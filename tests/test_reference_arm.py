"""The reference arm: ``oracle/_ref`` (the reference package, byte-compiled by oracle/build_ref.py)
driven by ``oracle/ref_arm.py``. Pins three things on the CPU: the build recipe produces an
importable package without copying sources, the object the REFERENCE's own saver writes for a seeded
shard equals what the oracle computes for the same tensors (so oracle and ``_ref`` agree on real
workload shapes, beyond the golden vectors), and the multi-rank driver aggregates as documented."""

import os
import sys

import pytest

import conftest

sys.path.insert(0, conftest.REPO_ROOT)

import build_ref  # noqa: E402
import ref_arm  # noqa: E402

needs_ref = pytest.mark.skipif(ref_arm.unavailable_reason() is not None, reason="oracle/_ref is not built here")


def test_build_recipe_outputs_bytecode_only():
    if not build_ref.reference_available():
        pytest.skip("no reference checkout on this machine")
    out = build_ref.build()
    assert build_ref.is_current()
    import zipfile

    assert sorted(os.listdir(out)) == ["manifest.json", "reference_bytecode.zip"]
    names = zipfile.ZipFile(os.path.join(out, "reference_bytecode.zip")).namelist()
    assert "ml_flashpoint/core/checkpoint_saver.pyc" in names
    assert all(n.endswith(".pyc") or n.endswith("/") for n in names)  # bytecode and directories, no sources


@needs_ref
def test_reference_object_equals_the_oracle_and_ranks_aggregate(tmp_path):
    import torch

    import bench
    import mlf_oracle as oracle

    sample_cap = 400 << 20  # the bf16 embedding shard (131 MB) and its fp32 master copy (263 MB)
    out = ref_arm.run(world=2, steps=1, warmup=1, workdir=str(tmp_path / "ref"), layers=0, budget_s=60.0,
                      max_sample_bytes=sample_cap, digest=True, force_cpu=True)
    assert out["ranks"] == 2 and out["restore_verified"] is True and out["value"] > 0
    assert out["bytes_per_step_per_rank"] <= sample_cap and "prefix: requested size" in out["sample"]
    assert out["cores"] == 2 * out["torch_threads_per_rank"]
    for entry in out["objects"]:
        shard = bench.build_shard(entry["rank"], torch.device("cpu"), layers=0)
        picked, total = [], 0
        for _, t, _, _ in shard:
            n = t.numel() * t.element_size()
            if total + n > sample_cap and picked:
                break
            picked.append(t)
            total += n
        want_sha, want_size = oracle.object_sha256([(str(i), t) for i, t in enumerate(picked)])
        assert (entry["sha256"], entry["size"]) == (want_sha, want_size), entry["rank"]
