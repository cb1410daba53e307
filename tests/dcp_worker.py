"""Worker body for the multi-process DCP tests (imported by spawned ranks)."""

import concurrent.futures
import os
import sys


def run_rank(rank: int, world: int, root: str, port: int, engine_kind: str, result_path: str) -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    repo = os.path.dirname(here)
    for p in (here, os.path.join(here, "golden"), os.path.join(repo, "oracle"), os.path.join(repo, "ml-flashpoint_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(
        MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
        NNODES="1", MLFLASHPOINT_LOG_LEVEL="ERROR",
    )
    import torch
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    import torch.multiprocessing as torch_mp

    import cases
    from helpers import NumpyCopyEngine, tensor_bytes
    from ml_flashpoint.adapter.pytorch.memory_storage_reader import MemoryStorageReader
    from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter
    from ml_flashpoint.checkpoint_object_manager.checkpoint_object_manager import CheckpointObjectManager
    from ml_flashpoint.core.checkpoint_id_types import CheckpointContainerId
    from ml_flashpoint.core.checkpoint_loader import DefaultMLFlashpointCheckpointLoader
    from ml_flashpoint.core.checkpoint_saver import DefaultMLFlashpointCheckpointSaver

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if engine_kind == "cuda":
            from ml_flashpoint.core.gpu_engine import CudaCopyEngine

            torch.cuda.set_device(rank % torch.cuda.device_count())
            engine = CudaCopyEngine()
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            engine = NumpyCopyEngine()
            device = torch.device("cpu")

        case = cases.CASES["gpt2_tiny"]()  # every rank holds the full replica, as in the CPU config
        state = {k: v.to(device) for k, v in case["tensors"].items()}
        state["extra.rank_note"] = {"saved_by_world": world}

        class _NoRepl:
            def async_replicate(self, buffer_io):
                com.close_buffer(buffer_io, skip_close_if_symlink=True)
                return []

        com = CheckpointObjectManager()
        saver = DefaultMLFlashpointCheckpointSaver(
            global_rank_getter=dist.get_rank,
            local_rank_getter=dist.get_rank,
            global_barrier_func=dist.barrier,
            ckpt_obj_manager=com,
            replication_manager=_NoRepl(),
            initial_buffer_size_bytes=4 << 20,
            copy_engine=engine,
        )
        manager_future = concurrent.futures.Future()
        manager = torch_mp.Manager()
        manager_future.set_result(manager)
        ckpt = os.path.join(root, "step-100_ckpt")
        writer = MemoryStorageWriter(saver, manager_future)
        dcp.save(state, checkpoint_id=ckpt, storage_writer=writer)
        saver.finalize_checkpoint(CheckpointContainerId(ckpt))

        loader = DefaultMLFlashpointCheckpointLoader(
            com,
            None,
            global_rank_getter=dist.get_rank,
            local_rank_getter=dist.get_rank,
            broadcast_object_list_func=dist.broadcast_object_list,
            all_gather_object_func=dist.all_gather_object,
            world_size_getter=dist.get_world_size,
            copy_engine=engine,
        )
        fresh = {k: torch.zeros_like(v) for k, v in state.items() if isinstance(v, torch.Tensor)}
        fresh["extra.rank_note"] = {"saved_by_world": -1}
        dcp.load(fresh, checkpoint_id=ckpt, storage_reader=MemoryStorageReader(ckpt, loader))
        bad = [k for k, v in case["tensors"].items() if tensor_bytes(fresh[k]) != tensor_bytes(v)]
        if fresh["extra.rank_note"] != {"saved_by_world": world}:
            bad.append("extra.rank_note")
        ok = not bad
        listing = sorted(os.listdir(ckpt))
        markers = [n for n in os.listdir(root) if n.endswith("unfinished")]
        with open(f"{result_path}.{rank}", "w") as f:
            f.write(repr({"ok": ok, "bad": bad[:5], "listing": listing, "markers": markers}))
        manager.shutdown()
    finally:
        dist.destroy_process_group()


def run_async_save(rank: int, root: str, port: int, result_path: str) -> None:
    """``dcp.async_save`` through the writer: the tensors are overwritten as soon as the call returns."""
    here = os.path.dirname(os.path.abspath(__file__))
    repo = os.path.dirname(here)
    for p in (here, os.path.join(here, "golden"), os.path.join(repo, "oracle"), os.path.join(repo, "ml-flashpoint_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(
        MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", NNODES="1",
        MLFLASHPOINT_LOG_LEVEL="ERROR",
    )
    import torch
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    import torch.multiprocessing as torch_mp

    import cases
    from helpers import NumpyCopyEngine, make_loader, make_saver, tensor_bytes
    from ml_flashpoint.adapter.pytorch.memory_storage_reader import MemoryStorageReader
    from ml_flashpoint.adapter.pytorch.memory_storage_writer import MemoryStorageWriter

    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        engine = NumpyCopyEngine()

        class _NoRepl:
            def async_replicate(self, buffer_io):
                buffer_io.close()
                return []

        saver, com = make_saver(copy_engine=engine, replication_manager=_NoRepl())
        manager = torch_mp.Manager()
        fut = concurrent.futures.Future()
        fut.set_result(manager)
        state = dict(cases.CASES["gpt2_tiny"]()["tensors"])
        originals = {k: v.clone() for k, v in state.items()}
        ckpt = os.path.join(root, "step-1_ckpt")
        handle = dcp.async_save(state, checkpoint_id=ckpt, storage_writer=MemoryStorageWriter(saver, fut))
        for v in state.values():
            v.zero_()
        handle.result()
        fresh = {k: torch.zeros_like(v) for k, v in originals.items()}
        dcp.load(fresh, checkpoint_id=ckpt, storage_reader=MemoryStorageReader(ckpt, make_loader(com, copy_engine=engine)))
        ok = all(tensor_bytes(fresh[k]) == tensor_bytes(v) for k, v in originals.items())
        with open(result_path, "w") as f:
            f.write(repr({"ok": ok}))
        manager.shutdown()
    finally:
        dist.destroy_process_group()
