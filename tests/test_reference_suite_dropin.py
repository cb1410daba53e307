"""Drop-in acceptance: the reference project's own host-side tests, run unmodified against this package.

If a checkout of the reference project sits next to this repository (or ``MLF_REFERENCE_ROOT`` names
one), its test files are executed in place with ``PYTHONPATH`` pointing at this package. They construct
the same classes through the same module paths, so every pass is evidence that the public surface is
call-compatible. Tests that move checkpoint bytes through the saver are not part of this list: here
bytes are moved by CUDA kernels only, and those paths have their own GPU parity tests.
"""

import concurrent.futures
import os
import subprocess
import sys

import pytest

import conftest

REFERENCE_ROOT = os.environ.get("MLF_REFERENCE_ROOT") or os.path.join(os.path.dirname(conftest.REPO_ROOT), "reference")

# (test file, tests expected to pass, tests deselected with the reason)
SUITES = [
    ("core/test_checkpoint_id_types.py", 53),
    ("core/test_hfid.py", 9),
    ("core/test_utils.py", 41),
    ("core/test_mlf_logging.py", 18),
    ("core/test_buffer_pool.py", 17),
    ("checkpoint_object_manager/test_buffer_io.py", 112),
    ("checkpoint_object_manager/test_checkpoint_object_manager.py", 56),
    ("replication/test_pairwise_replication_strategy.py", 17),
    ("replication/test_replication_manager.py", 19),
    ("adapter/pytorch/test_memory_storage_reader.py", 11),
    ("adapter/pytorch/test_custom_state_dict_saver.py", 18),
    # deselected: asserts that stage() moves tensors to the CPU; here stage() snapshots them in HBM on purpose
    ("adapter/pytorch/test_memory_storage_writer.py", 76, ["TestStage::test_stage_moves_all_to_cpu"]),
    # deselected: calls read_tensor on optimized-format bytes, which here runs the CUDA unpack kernel
    ("core/test_checkpoint_loader.py", 56, ["TestReadTensor::test_read_tensor_optimized_format"]),
    ("checkpoint_object_manager/buffer_object/test_buffer_object_bindings.py", 8),
    # two services on 127.0.0.1; without a CUDA device they negotiate the TCP transport
    ("replication/test_transer_service.py", 6),
    ("replication/test_replication_manager_e2e.py", 2),
    ("adapter/nemo/test_nemo_checkpoint_loader.py", 2),
]

# Adapter test files import megatron-core / nemo / lightning at module level. Those packages are not
# installed here, so these files run with the stand-in modules of tests/megatron_standins.py.
# Deselected in the Megatron save strategy file: tests asserting that the writer process moves the
# bytes. Here the trainer process queues pack + transfer inside async_save, the async function has
# nothing left to do and a fourth finalize function publishes the results.
ADAPTER_SUITES = [
    ("adapter/megatron/test_load_strategies.py", 12),
    ("adapter/megatron/test_save_strategies.py", 14, [
        "test_async_save_async_fn_call_success", "test_async_save_async_fn_failure", "test_async_save_finalize_fns_calls",
        "test_finalize_fns_failure", "test_async_save_ensure_metadata_deepcopy",
    ]),
    ("adapter/nemo/test_auto_resume.py", 12),
    ("adapter/nemo/test_checkpoint_callback.py", 43),
    ("adapter/nemo/test_checkpoint_io.py", 47),
    ("adapter/nemo/test_event_logging_callback.py", 18),
    ("adapter/nemo/test_wrapper_util.py", 54),
]


# The reference's saver tests build savers over CPU tensors and check names, offsets, results, markers,
# threading and error paths. Without a GPU the byte moves are done by the numpy test double of
# tests/helpers.py instead of the CUDA engine (MLF_REFSUITE_HOST_ENGINE, see refsuite_plugin.py).
# Deselected: tests of the reference's host copy internals, which have no counterpart here: staging
# to the CPU (TestStageData), the private per-tensor memcpy (_save_tensor_optimized, _clone_if_needed)
# and the torch intra-op thread count that write_data sets for that memcpy.
HOST_ENGINE_SUITES = [
    ("core/test_checkpoint_saver.py", 107, [
        "test_write_data_resets_num_threads", "test_stage_data_defaults_to_non_blocking", "test_stage_data_moves_all_to_cpu_mocked",
        "test_stage_data_cuda_synchronization[True-True]", "test_save_tensor_optimized_writes_correct_header_and_data",
        "test_prepare_write_data_clone_if_needed_logic",
    ]),
]


def _launch(entry, workdir, standins, host_engine=False):
    suite = entry[0]
    deselected = entry[2] if len(entry) > 2 else []
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([conftest.PACKAGE_ROOT, os.path.join(conftest.REPO_ROOT, "tests")])
    env.pop("MLFLASHPOINT_LOG_LEVEL", None)
    if standins:
        env["MLF_REFSUITE_STANDINS"] = "1"
    if host_engine:
        env["MLF_REFSUITE_HOST_ENGINE"] = "1"
    cmd = [
        sys.executable, "-m", "pytest", os.path.join(REFERENCE_ROOT, "tests", suite),
        "-q", "-p", "refsuite_plugin", "-p", "no:cacheprovider", "--rootdir", workdir, "-c", os.devnull,
    ]
    if deselected:
        cmd += ["-k", " and ".join("not " + name.split("::")[-1] for name in deselected)]
    return subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=workdir, timeout=900)


@pytest.fixture(scope="module")
def suite_runs(tmp_path_factory):
    """All files are started at once on a small pool (each costs a torch import); tests collect their own result."""
    pool = concurrent.futures.ThreadPoolExecutor(max_workers=max(2, min(6, (os.cpu_count() or 2) // 2)))
    runs = {}
    for standins, entries in ((False, SUITES), (True, ADAPTER_SUITES)):
        for entry in entries:
            workdir = str(tmp_path_factory.mktemp("refsuite"))
            runs[entry[0]] = pool.submit(_launch, entry, workdir, standins)
    for entry in HOST_ENGINE_SUITES:
        runs[entry[0]] = pool.submit(_launch, entry, str(tmp_path_factory.mktemp("refsuite")), False, True)
    yield runs
    pool.shutdown(wait=False, cancel_futures=True)


def _check(entry, suite_runs):
    run = suite_runs[entry[0]].result()
    tail = run.stdout[-3000:] + run.stderr[-1500:]
    assert run.returncode == 0, tail
    assert f"{entry[1]} passed" in run.stdout, tail


_needs_reference = pytest.mark.skipif(
    not os.path.isdir(os.path.join(REFERENCE_ROOT, "tests")), reason="no reference checkout available"
)


@_needs_reference
@pytest.mark.parametrize("entry", SUITES, ids=[e[0] for e in SUITES])
def test_reference_test_file_passes_against_this_package(entry, suite_runs):
    _check(entry, suite_runs)


@_needs_reference
@pytest.mark.parametrize("entry", ADAPTER_SUITES, ids=[e[0] for e in ADAPTER_SUITES])
def test_reference_adapter_test_file_passes_with_standin_frameworks(entry, suite_runs):
    _check(entry, suite_runs)


@_needs_reference
@pytest.mark.parametrize("entry", HOST_ENGINE_SUITES, ids=[e[0] for e in HOST_ENGINE_SUITES])
def test_reference_saver_test_file_passes_with_host_engine_double(entry, suite_runs):
    _check(entry, suite_runs)
