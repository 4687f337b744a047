"""Helpers shared by the multi-process tests: free rendezvous ports and a spawner for gloo ranks."""
import os
import socket
import traceback

import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        q.put((rank, True, fn(rank, world, *args)))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, False, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_gloo_ranks(fn, world: int, *args, timeout: float = 300.0) -> list:
    """Run fn(rank, world, *args) in `world` spawned processes joined by a gloo group; returns the results by rank.
    `fn` must be a module-level function (spawned processes import it by name)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, ok, val = q.get(timeout=timeout)
            assert ok, f"rank {rank} failed:\n{val}"
            out[rank] = val
    finally:
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.terminate()
    return [out[r] for r in range(world)]
