"""Small worker classes used by the runtime's own tests (they must be importable in spawned processes)."""
from __future__ import annotations

import asyncio
import os
import time

import torch


class EchoWorker:
    def __init__(self, tag: str = "w", use_dist: bool = False):
        self.tag = tag
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if use_dist and self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("gloo")

    def whoami(self):
        return (self.tag, self.rank, self.world, os.getpid())

    def add(self, t: torch.Tensor, k: float = 1.0):
        return t + k

    def execute_batch(self, method_name, chunk):
        return [getattr(self, method_name)(**{k: v[i] for k, v in chunk.items()})
                for i in range(len(next(iter(chunk.values()))))]

    def square(self, x):
        return (self.rank, x * x)

    def all_reduce_sum(self, x: float):
        import torch.distributed as dist

        t = torch.tensor([x])
        dist.all_reduce(t)
        return float(t)

    async def slow_echo(self, x, delay: float = 0.05):
        await asyncio.sleep(delay)
        return x

    def boom(self):
        raise ValueError("intended failure")

    def hang(self, seconds: float):
        time.sleep(seconds)
        return "woke"

    def die(self):
        os._exit(3)


class EnvWorker:
    def env(self, keys):
        return {k: os.environ.get(k) for k in keys}
