"""Small distributed helpers (barrier + device sync; rendezvous defaults)."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def torch_dist_barrier_and_cuda_sync() -> None:
    """Barrier over the default group followed by a device synchronize (after checkpoints, syncs and offloads)."""
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def init_process_group(backend: str | None = None, timeout_minutes: int = 60) -> tuple[int, int, int]:
    """Initialise the default group from torchrun-style environment variables. Returns (rank, local_rank, world)."""
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device(f"cuda:{local}")
        dist.init_process_group(backend, timeout=datetime.timedelta(minutes=timeout_minutes), **kw)
    return rank, local, world


def stateless_process_group(host: str, port: int, rank: int, world: int, backend: str = "gloo", device=None,
                            timeout_s: int = 1800):
    """A process group next to (and independent of) the default one, over its own TCP store.

    The trainer world and the rollout world of a placement with separate rollout GPUs are two torch.distributed
    worlds; the weight-update group that spans trainer rank 0 and all rollout ranks is built with this helper
    (the reference builds the same kind of extra group: openrlhf/utils/distributed_util.py:17-26,
    openrlhf/trainer/ray/ppo_actor.py:163-217). Returns a backend object with ``broadcast([tensor], opts)``."""
    to = datetime.timedelta(seconds=timeout_s)
    store = dist.TCPStore(host, int(port), world, is_master=(rank == 0), timeout=to)
    store = dist.PrefixStore("weight_update", store)
    if backend == "gloo":
        return dist.ProcessGroupGloo(store, rank, world, to)
    if backend == "nccl":
        if device is not None and torch.device(device).type == "cuda":
            torch.cuda.set_device(device)
        opts = dist.ProcessGroupNCCL.Options()
        opts._timeout = to
        return dist.ProcessGroupNCCL(store, rank, world, opts)
    raise ValueError(f"unknown backend {backend}")


def stateless_init_process_group(master_address, master_port, rank, world_size, device):
    """Same call as the reference's helper of this name (openrlhf/utils/distributed_util.py:13-26): a communicator
    between training processes and rollout workers that is independent of the default process group. NCCL for a
    CUDA device, gloo otherwise."""
    backend = "nccl" if device is not None and torch.device(device).type == "cuda" else "gloo"
    return stateless_process_group(master_address, master_port, rank, world_size, backend=backend, device=device)
