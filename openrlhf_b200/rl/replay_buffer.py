"""Replay buffer of single-sample experiences with optional token-budget ("dynamic") micro-batching.

Same contract as the reference's ``NaiveReplayBuffer`` (openrlhf/trainer/ppo_utils/replay_buffer.py:14-177):
``append`` splits a batch into unpadded samples, ``collate_fn`` re-batches, and ``setup_dynamic_batch`` precomputes,
for every optimizer step, the micro-batch partition (first-fit count agreed across data-parallel ranks, then
Karmarkar-Karp balancing) and the global normalisers / optimizer-step flags the trainer needs.
"""
from __future__ import annotations

import random

import torch
import torch.distributed as dist

from ..utils.seqlen_balancing import get_minimum_num_micro_batch_size, get_seqlen_balanced_partitions
from .experience import Experience, make_experience_batch, remove_padding_in_sequences, split_experience_batch


def _all_reduce(value: float, op: str, group) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op={"min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op], group=group)
    return float(t.item())


class NaiveReplayBuffer:
    def __init__(self, sample_batch_size: int, limit: int = 0, cpu_offload: bool = True,
                 packing_samples: bool = False, dynamic_batch: bool = False) -> None:
        self.sample_batch_size, self.limit = sample_batch_size, limit          # limit <= 0: unbounded
        self.cpu_offload, self.packing_samples, self.dynamic_batch = cpu_offload, packing_samples, dynamic_batch
        self.target_device = (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                              else torch.device("cpu"))
        self.items: list[Experience] = []
        self._reset_dynamic()

    def _reset_dynamic(self):
        self.dynamic_indices: list[list[int]] = []
        self.dynamic_sample_loss_scale: list[float] = []
        self.dynamic_batch_num_tokens: list[float] = []
        self.dynamic_global_batch_size: list[float] = []
        self.dynamic_optimizer_step: list[int] = []

    @torch.no_grad()
    def append(self, experience: Experience) -> None:
        if self.cpu_offload:
            experience.to_device(torch.device("cpu"))
        self.items += remove_padding_in_sequences(split_experience_batch(experience))
        if self.limit > 0 and len(self.items) > self.limit:
            self.items = self.items[len(self.items) - self.limit:]

    def clear(self) -> None:
        self.items.clear()
        self._reset_dynamic()

    @torch.no_grad()
    def sample(self) -> Experience:
        exp = make_experience_batch(random.sample(self.items, self.sample_batch_size), self.packing_samples)
        return exp.to_device(self.target_device) if self.cpu_offload else exp

    def __len__(self) -> int:
        return len(self.dynamic_indices) if self.dynamic_batch else len(self.items)

    def __getitem__(self, idx: int):
        if self.dynamic_batch:
            return [self.items[i] for i in self.dynamic_indices[idx]]
        return self.items[idx]

    def collate_fn(self, batch) -> Experience:
        return make_experience_batch(batch[0] if self.dynamic_batch else batch, self.packing_samples)

    def setup_dynamic_batch(self, strategy) -> None:
        args = strategy.args
        group = strategy.dp_group() if hasattr(strategy, "dp_group") else None
        dp = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        lengths = [int(it.total_length.item()) for it in self.items]
        local_bs = max(args.train.batch_size // dp, 1)
        expected = args.rollout.batch_size * args.rollout.n_samples_per_prompt // args.train.batch_size
        # a short buffer (async / partial rollout at an episode boundary) must yield the same step count everywhere
        steps = int(_all_reduce(min(expected, len(lengths) // local_bs), "min", group))
        self._reset_dynamic()
        self.sample_batch_size = 1
        if steps == 0:
            return
        windows = [(i * local_bs, (i + 1) * local_bs) for i in range(steps)]
        n_mbs = [get_minimum_num_micro_batch_size(lengths[a:b], args.train.max_tokens_per_gpu, args.ds.ring_attn_size,
                                                  args.ds.tensor_parallel_size) for a, b in windows]
        n_mbs = [int(_all_reduce(n, "max", group)) for n in n_mbs]
        for (a, b), n in zip(windows, n_mbs):
            n = min(n, b - a)
            parts = [[a + i for i in p] for p in get_seqlen_balanced_partitions(lengths[a:b], n, equal_size=False)]
            total = sum(len(p) for p in parts)
            n_valid = sum(int(self.items[i].action_mask.sum().item() > 0) for p in parts for i in p)
            n_tok = sum(int(self.items[i].action_mask.sum().item()) for p in parts for i in p)
            g_valid, g_tok = _all_reduce(n_valid, "sum", group), _all_reduce(n_tok, "sum", group)
            self.dynamic_indices += parts
            self.dynamic_sample_loss_scale += [len(p) / total for p in parts]
            self.dynamic_batch_num_tokens += [g_tok] * len(parts)
            self.dynamic_global_batch_size += [g_valid] * len(parts)
            self.dynamic_optimizer_step += [0] * (len(parts) - 1) + [1]
