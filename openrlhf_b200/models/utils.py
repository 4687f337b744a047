"""Model-side math helpers with the reference's names (openrlhf/models/utils.py:64-186)."""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch


def compute_approx_kl(log_probs: torch.Tensor, log_probs_base: torch.Tensor, kl_estimator: str = "k1") -> torch.Tensor:
    """Per-token KL estimate between policy and reference (k1 = log-ratio, k2 = half squared log-ratio,
    k3 = exp(-d) - 1 + d; http://joschu.net/blog/kl-approx.html), clamped to [-10, 10]."""
    d = log_probs.float() - log_probs_base.float()
    if kl_estimator == "k1":
        kl = d
    elif kl_estimator == "k2":
        kl = d ** 2 / 2.0
    elif kl_estimator == "k3":
        kl = torch.exp(-d) - 1 + d
    else:
        raise ValueError(f"unknown kl estimator {kl_estimator}")
    return kl.clamp(min=-10, max=10)


def compute_reward(r: Union[torch.Tensor, float], kl_coef: float, kl: torch.Tensor,
                   action_mask: Optional[torch.Tensor] = None,
                   reward_clip_range: Tuple[float, float] = None) -> torch.Tensor:
    """Per-token reward: -kl_coef * kl everywhere plus the (clipped) sequence reward at the last action position."""
    kl_coef = max(float(kl_coef), 0.0)
    if reward_clip_range:
        r = r.clamp(min=reward_clip_range[0], max=reward_clip_range[1])
    out = -kl_coef * kl
    A = action_mask.size(1)
    last = A - 1 - action_mask.long().fliplr().argmax(dim=1, keepdim=True)
    return out + torch.zeros_like(kl).scatter_(1, last, r.unsqueeze(1).to(kl.dtype))


def log_probs_from_logits(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """log softmax(logits / T)[labels] without materialising the full log-softmax (row-chunked logsumexp)."""
    if temperature != 1.0:
        logits = logits / temperature
    picked = logits.gather(-1, labels.unsqueeze(-1)).squeeze(-1).float()
    flat = logits.reshape(-1, logits.shape[-1])
    lse = torch.cat([torch.logsumexp(flat[i:i + 1024].float(), dim=-1) for i in range(0, flat.shape[0], 1024)])
    return picked - lse.view(picked.shape)


def masked_mean(tensor: torch.Tensor, mask: Optional[torch.Tensor], dim: int = None) -> torch.Tensor:
    if mask is None:
        return tensor.mean(dim=dim)
    mask = mask.to(tensor.dtype) if tensor.is_floating_point() else mask.float()
    if dim is None:
        return (tensor * mask).sum() / mask.sum().clamp_min(1e-8)
    return (tensor * mask).sum(dim=dim) / mask.sum(dim=dim).clamp_min(1e-8)


def masked_normalize(tensor: torch.Tensor, mask: torch.Tensor, dim: int = 1, eps: float = 1e-8) -> torch.Tensor:
    tensor = tensor * mask
    mean = masked_mean(tensor, mask, dim=dim).unsqueeze(dim) if dim is not None else masked_mean(tensor, mask)
    centered = tensor - mean
    var = masked_mean(centered ** 2, mask, dim=dim)
    var = var.unsqueeze(dim) if dim is not None else var
    return centered * var.clamp(min=eps).rsqrt()


def compute_entropy(logits: torch.Tensor) -> torch.Tensor:
    """H = logsumexp(z) - sum softmax(z) * z"""
    z = logits.float()
    p = torch.softmax(z, dim=-1)
    return torch.logsumexp(z, dim=-1) - (p * z).sum(-1)
