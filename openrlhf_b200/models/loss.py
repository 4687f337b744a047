"""Loss modules with the reference's public classes and call signatures (openrlhf/models/loss.py:11-335), built on one
idea: every reduction is a weighted sum ``sum(loss * w)`` where ``w`` carries the mask, the token- or sample-level
normaliser, the global batch totals and the data-parallel compensation. The fused CUDA kernels of ``ops.rl`` consume
the same weights, so the PPO / value losses run as a single launch on the GPU and as plain PyTorch on CPU.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import rl as K
from .utils import masked_mean


def aggregation_weights(loss_mask: torch.Tensor, token_level_loss: bool = True, dp_size: int = 1,
                        batch_num_tokens: Optional[float] = None,
                        global_batch_size: Optional[float] = None) -> torch.Tensor:
    """Per-element weights w such that sum(loss * w) is the requested mean.

    token level:  w = mask * dp_size / batch_num_tokens           (plain masked mean when no global total is given)
    sample level: w = mask / (tokens_in_row + 1e-8) * [row non-empty] * dp_size / global_batch_size
    """
    m = loss_mask.float()
    if token_level_loss:
        if batch_num_tokens is None:
            return m / m.sum().clamp_min(1e-8)
        return m * (dp_size / batch_num_tokens)
    cnt = m.sum(-1, keepdim=True)
    live = (cnt > 0).float()
    per_row = m / (cnt + 1e-8) * live
    if global_batch_size is None:
        return per_row / live.sum().clamp_min(1e-8)
    return per_row * (dp_size / global_batch_size)


def aggregate_loss(loss: torch.Tensor, loss_mask: torch.Tensor, token_level_loss: bool = True, dp_size: int = 1,
                   batch_num_tokens: Optional[float] = None, global_batch_size: Optional[float] = None) -> torch.Tensor:
    """Scalar from a per-token loss matrix: global token-mean or mean over sequences of per-sequence token-means."""
    return (loss * aggregation_weights(loss_mask, token_level_loss, dp_size, batch_num_tokens, global_batch_size)).sum()


class GPTLMLoss(nn.Module):
    """Next-token cross entropy on logits (labels == -100 ignored); with a context-parallel group every rank scores
    its contiguous slice of the labels and the scalar is averaged over the group."""

    IGNORE_INDEX = -100

    def __init__(self, ring_attn_group=None):
        super().__init__()
        self.ring_attn_group = ring_attn_group
        if ring_attn_group is not None:
            self.ring_attn_rank = dist.get_rank(ring_attn_group)
            self.ring_attn_world_size = dist.get_world_size(ring_attn_group)

    def forward(self, logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        if self.ring_attn_group is not None:
            per = labels.size(-1) // self.ring_attn_world_size
            lo = self.ring_attn_rank * per
            labels = labels[..., lo:min(lo + per, labels.size(-1))]
        z = logits[..., :-1, :].reshape(-1, logits.size(-1))
        y = labels[..., 1:].reshape(-1)
        if self.ring_attn_group is not None and bool((y == self.IGNORE_INDEX).all()):
            loss = z.mean() * 0
        else:
            loss = F.cross_entropy(z.float(), y, ignore_index=self.IGNORE_INDEX)
        if self.ring_attn_group is not None:
            dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=self.ring_attn_group)
            loss = loss / self.ring_attn_world_size
        return loss


class SFTLoss(nn.Module):
    def __init__(self, token_level_loss: bool = True):
        super().__init__()
        self.token_level_loss = token_level_loss

    def forward(self, per_token_logps, loss_mask, dp_size: int = 1, batch_num_tokens=None, global_batch_size=None):
        return aggregate_loss(-per_token_logps, loss_mask, self.token_level_loss, dp_size, batch_num_tokens,
                              global_batch_size)


class PolicyLoss(nn.Module):
    """PPO clipped surrogate with asymmetric clipping, dual-clip, GSPO sequence-level ratios and rollout-engine
    importance-sampling correction (tis / icepop / seq-mask-tis). Returns (loss, clip_ratio, ppo_kl, vllm_kl)."""

    def __init__(self, clip_eps_low: float = 0.2, clip_eps_high: float = 0.2, dual_clip: float = None,
                 token_level_loss: bool = True, policy_loss_type: str = "ppo", enable_vllm_is_correction: bool = False,
                 vllm_is_truncated_threshold: list = None, vllm_is_correction_type: str = "tis") -> None:
        super().__init__()
        if dual_clip is not None and not dual_clip > 1.0:
            raise AssertionError(f"dual_clip must be > 1.0, got {dual_clip}")
        if vllm_is_correction_type not in ("tis", "icepop", "seq-mask-tis"):
            raise ValueError(f"Invalid vllm_is_correction_type: {vllm_is_correction_type}, must be one of "
                             "tis/icepop/seq-mask-tis")
        if policy_loss_type not in ("ppo", "gspo"):
            raise ValueError(f"Invalid policy loss type: {policy_loss_type}")
        self.clip_eps_low, self.clip_eps_high, self.dual_clip = clip_eps_low, clip_eps_high, dual_clip
        self.policy_loss_type = policy_loss_type
        self.token_level_loss = token_level_loss and policy_loss_type != "gspo"   # GSPO aggregates per sequence
        self.enable_vllm_is_correction = enable_vllm_is_correction
        self.vllm_is_truncated_threshold = vllm_is_truncated_threshold
        self.vllm_is_correction_type = vllm_is_correction_type

    def forward(self, log_probs, old_log_probs, advantages, action_mask=None, rollout_log_probs=None,
                dp_size: int = 1, batch_num_tokens=None, global_batch_size=None):
        if action_mask is None:
            action_mask = torch.ones_like(log_probs)
        mask = action_mask.float()
        w = aggregation_weights(mask, self.token_level_loss, dp_size, batch_num_tokens, global_batch_size)
        is_on = self.enable_vllm_is_correction and self.policy_loss_type == "ppo"
        fused_ok = self.policy_loss_type == "ppo" and not (is_on and self.vllm_is_correction_type == "seq-mask-tis")
        if fused_ok:
            lo, hi = self.vllm_is_truncated_threshold if is_on else (0.0, 0.0)
            out = K.ppo_loss(log_probs, old_log_probs, advantages, mask,
                             rollout_logp=rollout_log_probs if is_on else None, weight=w, eps_low=self.clip_eps_low,
                             eps_high=self.clip_eps_high, dual_clip=self.dual_clip,
                             is_mode=self.vllm_is_correction_type if is_on else None, is_lo=lo, is_hi=hi)
            return out["loss"], out["clip_ratio"], out["ppo_kl"], (out["vllm_kl"] if is_on else None)
        # sequence-level variants: plain PyTorch
        raw = log_probs - old_log_probs
        if self.policy_loss_type == "gspo":
            lr = (log_probs - rollout_log_probs) if self.enable_vllm_is_correction else raw
            ratio = ((lr * mask).sum(-1) / mask.sum(-1).clamp(min=1)).exp().unsqueeze(-1) * mask
        else:
            ratio = raw.clamp(-20.0, 20.0).exp()
        s1 = ratio * advantages
        s2 = ratio.clamp(1 - self.clip_eps_low, 1 + self.clip_eps_high) * advantages
        lower = torch.min(s1, s2)
        if self.dual_clip is not None:
            lower = torch.where(advantages < 0, torch.max(lower, self.dual_clip * advantages), lower)
        loss = -lower
        vllm_kl = None
        if is_on:  # seq-mask-tis: keep whole sequences by their geometric-mean ratio, weight tokens by the raw ratio
            lo, hi = self.vllm_is_truncated_threshold
            d = old_log_probs - rollout_log_probs
            seq = masked_mean(d, mask, dim=-1).exp()
            keep = ((seq >= lo) & (seq <= hi)).unsqueeze(-1)
            loss = keep * d.exp().detach() * loss
            vllm_kl = masked_mean(rollout_log_probs - old_log_probs, mask, dim=None)
        total = (loss * w).sum()
        clip_ratio = masked_mean((s2 < s1).float(), mask, dim=None)
        ppo_kl = masked_mean(-raw.detach(), mask, dim=None)
        return total, clip_ratio, ppo_kl, vllm_kl


class ValueLoss(nn.Module):
    def __init__(self, clip_eps: float = None, token_level_loss: bool = True) -> None:
        super().__init__()
        self.clip_eps, self.token_level_loss = clip_eps, token_level_loss

    def forward(self, values, old_values, returns, action_mask=None, dp_size: int = 1, batch_num_tokens=None,
                global_batch_size=None):
        if action_mask is None:
            action_mask = torch.ones_like(values)
        w = aggregation_weights(action_mask, self.token_level_loss, dp_size, batch_num_tokens, global_batch_size)
        return K.value_loss(values, old_values, returns, action_mask.float(), clip_eps=self.clip_eps, weight=w)


class PairWiseLoss(nn.Module):
    """-log sigmoid(r_chosen - r_rejected [- margin])"""

    def forward(self, chosen_reward, reject_reward, margin=None):
        gap = chosen_reward - reject_reward
        if margin is not None:
            gap = gap - margin
        return -F.logsigmoid(gap).mean()


class LogExpLoss(nn.Module):
    """log(1 + exp(r_rejected - r_chosen)) (https://arxiv.org/abs/2204.05862)"""

    def forward(self, chosen_reward, reject_reward, margin=None):
        return torch.log1p(torch.exp(reject_reward - chosen_reward)).mean()


class DPOLoss(nn.Module):
    """DPO, conservative DPO (label smoothing) and IPO on summed response log-probs."""

    def __init__(self, beta: float, label_smoothing: float = 0.0, ipo: bool = False) -> None:
        super().__init__()
        self.beta, self.label_smoothing, self.ipo = beta, label_smoothing, ipo

    def forward(self, policy_chosen_logps, policy_rejected_logps, reference_chosen_logps,
                reference_rejected_logps) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        z = (policy_chosen_logps - policy_rejected_logps) - (reference_chosen_logps - reference_rejected_logps)
        if self.ipo:
            losses = (z - 1 / (2 * self.beta)) ** 2
        else:
            ls = self.label_smoothing
            losses = -F.logsigmoid(self.beta * z) * (1 - ls) - F.logsigmoid(-self.beta * z) * ls
        chosen = self.beta * (policy_chosen_logps - reference_chosen_logps).detach()
        rejected = self.beta * (policy_rejected_logps - reference_rejected_logps).detach()
        return losses.mean(), chosen, rejected
