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


def run_async_save(rank: int, root: str, port: int, result_path: str, engine_kind: str = "numpy") -> None:
    """``dcp.async_save`` through the writer: the tensors are overwritten as soon as the call returns.
    With ``engine_kind="cuda"`` the state lives on the GPU and the CUDA engine moves the bytes."""
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
        if engine_kind == "cuda":
            from ml_flashpoint.core.gpu_engine import CudaCopyEngine

            torch.cuda.set_device(0)
            engine = CudaCopyEngine()
            device = torch.device("cuda", 0)
        else:
            engine = NumpyCopyEngine()
            device = torch.device("cpu")

        class _NoRepl:
            def async_replicate(self, buffer_io):
                buffer_io.close()
                return []

        saver, com = make_saver(copy_engine=engine, replication_manager=_NoRepl())
        manager = torch_mp.Manager()
        fut = concurrent.futures.Future()
        fut.set_result(manager)
        state = {k: v.to(device) for k, v in cases.CASES["gpt2_tiny"]()["tensors"].items()}
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


def run_gpt2_small(rank: int, world: int, root: str, port: int, result_path: str, engine_kind: str = "cuda", full_size: bool = True) -> None:
    """GPT-2 small with Adam state at its full 1.49 GB, every rank holding the full replica, saved
    and loaded through ``dcp.save`` / ``dcp.load`` with the CUDA engine. Each rank then rebuilds the
    object it wrote with the CPU oracle, from the storage records in ``.metadata`` (which tensor
    went into which object at which offset is the planner's decision), and compares SHA-256 digests."""
    here = os.path.dirname(os.path.abspath(__file__))
    repo = os.path.dirname(here)
    for p in (here, os.path.join(here, "golden"), os.path.join(repo, "oracle"), os.path.join(repo, "ml-flashpoint_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(
        MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
        NNODES="1", MLFLASHPOINT_LOG_LEVEL="ERROR",
    )
    import hashlib
    import pickle

    import torch
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    import torch.multiprocessing as torch_mp

    import mlf_oracle as oracle
    import workloads
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
            device = torch.device("cuda", torch.cuda.current_device())
            engine = CudaCopyEngine()
        else:
            from helpers import NumpyCopyEngine

            device = torch.device("cpu")
            engine = NumpyCopyEngine()
        state = workloads.gpt2_small_adam(device, seed=0) if full_size else workloads.gpt2_small_adam(
            device, seed=0, layers=2, d_model=64, d_ff=256, vocab=503, ctx=32)
        total_bytes = sum(v.numel() * v.element_size() for v in state.values())

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
            initial_buffer_size_bytes=total_bytes + (1 << 20),
            copy_engine=engine,
        )
        manager_future = concurrent.futures.Future()
        manager = torch_mp.Manager()
        manager_future.set_result(manager)
        ckpt = os.path.join(root, "step-1000_ckpt")
        dcp.save(state, checkpoint_id=ckpt, storage_writer=MemoryStorageWriter(saver, manager_future))
        saver.finalize_checkpoint(CheckpointContainerId(ckpt))

        # ---- the object this rank wrote, rebuilt by the oracle from the plan's storage records
        with open(os.path.join(ckpt, ".metadata"), "rb") as f:
            metadata = pickle.load(f)
        mine = sorted(
            (info.offset, index.fqn, info.length)
            for index, info in metadata.storage_data.items()
            if info.relative_path.endswith(f"_src{rank}.distcp")
        )
        names = {info.relative_path for info in metadata.storage_data.values() if info.relative_path.endswith(f"_src{rank}.distcp")}
        ok_object = len(names) == 1
        written = 0
        if ok_object:
            path = os.path.join(ckpt, names.pop())
            want_sha, want_size = oracle.object_sha256([(fqn, state[fqn]) for _, fqn, _ in mine])
            h = hashlib.sha256()
            with open(path, "rb") as f:
                for block in iter(lambda: f.read(1 << 24), b""):
                    h.update(block)
            written = os.path.getsize(path)
            ok_object = h.hexdigest() == want_sha and written == want_size
            # the records are contiguous from offset 0
            at = 0
            for offset, _, length in mine:
                ok_object = ok_object and offset == at
                at += length

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
        fresh = {k: torch.zeros_like(v) for k, v in state.items()}
        dcp.load(fresh, checkpoint_id=ckpt, storage_reader=MemoryStorageReader(ckpt, loader))
        bad = [k for k, v in state.items() if not torch.equal(fresh[k], v)]
        with open(f"{result_path}.{rank}", "w") as f:
            f.write(repr({"ok": ok_object and not bad, "object_ok": ok_object, "bad": bad[:5], "state_bytes": total_bytes,
                          "object_bytes": written, "items_in_my_object": len(mine)}))
        manager.shutdown()
    finally:
        dist.destroy_process_group()
