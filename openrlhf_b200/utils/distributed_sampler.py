"""Data-parallel sampler that can resume in the middle of an epoch by skipping ``consumed_samples`` (the resume
contract of openrlhf/utils/distributed_sampler.py:16-150)."""
from __future__ import annotations

import math
from typing import Iterator, Optional

import torch
import torch.distributed as dist
from torch.utils.data import Dataset, Sampler


class DistributedSampler(Sampler):
    def __init__(self, dataset: Dataset, num_replicas: Optional[int] = None, rank: Optional[int] = None,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = False, consumed_samples: int = 0):
        if num_replicas is None:
            num_replicas = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if not 0 <= rank < num_replicas:
            raise ValueError(f"rank {rank} outside [0, {num_replicas - 1}]")
        self.dataset, self.num_replicas, self.rank = dataset, num_replicas, rank
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch = 0
        n = len(dataset)
        self.num_samples = n // num_replicas if (drop_last and n % num_replicas) else math.ceil(n / num_replicas)
        self.total_size = self.num_samples * num_replicas
        self.consumed_indicies = consumed_samples // num_replicas

    def __iter__(self) -> Iterator[int]:
        n = len(self.dataset)
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            idx = torch.randperm(n, generator=g).tolist()
        else:
            idx = list(range(n))
        if self.drop_last:
            idx = idx[: self.total_size]
        elif len(idx) < self.total_size:
            pad = self.total_size - len(idx)
            idx += (idx * math.ceil(pad / max(len(idx), 1)))[:pad]
        mine = idx[self.rank:self.total_size:self.num_replicas]
        return iter(mine[self.consumed_indicies:])

    def __len__(self) -> int:
        return self.num_samples - self.consumed_indicies

    def set_epoch(self, epoch: int, consumed_samples: int = 0) -> None:
        self.epoch = epoch
        self.consumed_indicies = consumed_samples // self.num_replicas
