"""Advantage estimation for every estimator of the reference (gae, reinforce, rloo, reinforce_baseline, group_norm,
dr_grpo): group baselines on the raw rewards, KL-in-reward shaping, GAE / discounted returns and global whitening.

The per-token part runs in the fused kernels of ``ops.rl`` on whatever device the experiences live on (the reference
does it with Python loops on CPU tensors in the controller: openrlhf/trainer/ppo_utils/experience_maker.py:237-411).
"""
from __future__ import annotations

import torch

from ..ops import rl as K
from .length_penalty import apply_length_penalties

GROUP_ESTIMATORS = ("rloo", "reinforce_baseline", "group_norm", "dr_grpo")
WHITENED = ("gae", "reinforce", "reinforce_baseline")


def group_baseline(rewards: torch.Tensor, n: int, estimator: str) -> tuple[torch.Tensor, torch.Tensor | None]:
    """rewards (P*n,) in prompt order -> (shaped rewards (P*n,), per-sample group std or None)."""
    r = rewards.reshape(-1, n).float()
    std = r.std(-1, keepdim=True).expand(-1, n).reshape(-1) if n > 1 else None
    if estimator == "rloo":
        r = r - (r.sum(-1, keepdim=True) - r) / (n - 1)
    elif estimator in ("reinforce_baseline", "dr_grpo"):
        r = r - r.mean(-1, keepdim=True)
    elif estimator == "group_norm":
        r = (r - r.mean(-1, keepdim=True)) / (r.std(-1, keepdim=True) + 1e-9)
    return r.reshape(-1), std


@torch.no_grad()
def compute_advantages_and_returns(experiences, args, kl_value: float, dist_group=None, distributed: bool = False):
    """In place on `experiences` (each batched, with .index = original sample positions). Returns the list.

    distributed=True: the experiences are this rank's share of the rollout batch; the whitening statistics are summed
    over `dist_group` (None = the default group) so that every rank normalises with the mean / variance of the whole
    batch, as the reference's controller does (openrlhf/trainer/ppo_utils/experience_maker.py:314-328)."""
    est = args.algo.advantage.estimator
    n = args.rollout.n_samples_per_prompt
    apply_length_penalties(experiences, args)

    sizes = [len(e.index) for e in experiences]
    order = torch.tensor([i for e in experiences for i in e.index], dtype=torch.long)
    raw = torch.cat([e.rewards.float().cpu() for e in experiences])
    in_prompt_order = torch.empty_like(raw)
    in_prompt_order[order] = raw
    shaped, gstd = group_baseline(in_prompt_order, n, est)
    if gstd is not None:
        for e, s in zip(experiences, gstd[order].split(sizes)):
            e.info["group_reward_std"] = s
    per_exp = shaped[order].split(sizes)

    gamma = args.algo.advantage.gamma
    if est in GROUP_ESTIMATORS and gamma != 1.0:
        gamma = args.algo.advantage.gamma = 1.0
    clip = getattr(args.reward, "clip_range", None) or (-10.0, 10.0)
    beta = max(float(kl_value), 0.0)
    for e, r in zip(experiences, per_exp):
        dev = e.action_mask.device
        values = e.values if est == "gae" else None
        if est == "gae" and values is None:
            raise ValueError("the gae estimator needs critic values")
        adv, ret, rsum = K.gae_advantages(values, e.kl, r.to(dev), e.action_mask.float(), beta=beta, gamma=gamma,
                                          lambd=args.algo.advantage.lambd if est == "gae" else 1.0,
                                          clip=(float(clip[0]), float(clip[1])))
        e.advantages, e.returns = adv, ret
        e.info["return"] = rsum
        e.kl = None

    if est in WHITENED:
        # the statistics stay on the experiences' device: no host round trip, and NCCL can reduce them in place
        stats = sum(K.masked_stats(e.advantages.float(), e.action_mask.float()) for e in experiences)
        if distributed or dist_group is not None:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized() and dist.get_world_size(dist_group) > 1:
                if stats.device.type == "cpu" and dist.get_backend(dist_group) == "nccl":
                    dev_stats = stats.cuda()
                    dist.all_reduce(dev_stats, group=dist_group)
                    stats = dev_stats.cpu()
                else:
                    stats = stats.contiguous()
                    dist.all_reduce(stats, group=dist_group)
        for e in experiences:
            e.advantages = K.masked_whiten(e.advantages.float().contiguous(), e.action_mask.float(),
                                           std_norm=not args.algo.advantage.no_std_norm,
                                           stats=stats.to(e.advantages.device))
    return experiences
