"""Fused RL math: PPO clipped loss with KL / importance-sampling correction, clipped value loss, reward shaping +
GAE / discounted returns, masked whitening. CUDA tensors run the kernels of ``csrc/rl_ops.cu``; the ``*_reference``
functions restate the same math in PyTorch (CPU path and test oracle).

Semantics follow openrlhf/models/loss.py:116-269, openrlhf/models/utils.py:64-126 and
openrlhf/trainer/ppo_utils/experience_maker.py:275-411 of the reference.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_KL = {"k1": 1, "k2": 2, "k3": 3}
_IS = {None: 0, "": 0, "tis": 1, "icepop": 2}


def token_mean_weight(mask: torch.Tensor, num_tokens: float | None = None, dp_size: int = 1) -> torch.Tensor:
    """Per-token aggregation weight of a token-mean: mask * dp_size / num_tokens (num_tokens defaults to mask.sum())."""
    n = mask.sum().clamp_min(1.0) if num_tokens is None else num_tokens
    return mask.float() * (dp_size / n)


def seq_mean_weight(mask: torch.Tensor, global_batch_size: float | None = None, dp_size: int = 1) -> torch.Tensor:
    """Per-token weight of a mean over sequences of per-sequence token means (empty sequences excluded)."""
    cnt = mask.float().sum(-1, keepdim=True)
    nz = (cnt > 0).float()
    n = nz.sum().clamp_min(1.0) if global_batch_size is None else global_batch_size
    return mask.float() / (cnt + 1e-8) * nz * (dp_size / n)


def approx_kl_reference(logp, ref_logp, estimator="k1"):
    d = logp.float() - ref_logp.float()
    if estimator == "k1":
        kl = d
    elif estimator == "k2":
        kl = 0.5 * d * d
    else:
        kl = torch.exp(-d) - 1 + d
    return kl.clamp(-10, 10)


def ppo_loss_reference(logp, old_logp, adv, mask, ref_logp=None, rollout_logp=None, weight=None, eps_low=0.2,
                       eps_high=0.2, dual_clip=None, kl_coef=0.0, kl_estimator="k1", is_mode=None, is_lo=0.5,
                       is_hi=2.0):
    mask = mask.float()
    w = token_mean_weight(mask) if weight is None else weight
    lr = logp - old_logp
    ratio = torch.exp(lr.clamp(-20, 20))
    s1 = ratio * adv
    s2 = ratio.clamp(1 - eps_low, 1 + eps_high) * adv
    loss = -torch.min(s1, s2)
    if dual_clip is not None and dual_clip > 1:
        floor_v = dual_clip * adv
        loss = torch.where(adv < 0, -torch.max(torch.min(s1, s2), floor_v), loss)
    vllm_kl = torch.zeros((), device=logp.device)
    if rollout_logp is not None:
        d = (old_logp - rollout_logp).detach()
        vllm_kl = ((-d) * mask).sum() / mask.sum().clamp_min(1)
        if _IS[is_mode] == 1:
            loss = torch.exp(d).clamp(is_lo, is_hi) * loss
        elif _IS[is_mode] == 2:
            wr = torch.exp(d)
            loss = torch.where((wr >= is_lo) & (wr <= is_hi), wr, torch.zeros_like(wr)) * loss
    policy_loss = (loss * w).sum()
    kl_loss = torch.zeros((), device=logp.device)
    kl_mean = torch.zeros((), device=logp.device)
    if ref_logp is not None:
        kl = approx_kl_reference(logp, ref_logp, kl_estimator)
        kl_loss = (kl * w).sum()
        kl_mean = ((kl * mask).sum() / mask.sum().clamp_min(1)).detach()
    n = mask.sum().clamp_min(1)
    return {
        "loss": policy_loss + kl_coef * kl_loss,
        "policy_loss": policy_loss.detach(),
        "kl_loss": kl_loss.detach(),
        "clip_ratio": (((s2 < s1).float() * mask).sum() / n).detach(),
        "ppo_kl": ((-lr * mask).sum() / n).detach(),
        "vllm_kl": vllm_kl.detach(),
        "kl": kl_mean,
    }


class _PpoLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, old_logp, adv, weight, mask, ref_logp, rollout_logp, cfg):
        n = logp.numel()
        dlogp = torch.empty_like(logp, dtype=torch.float32)
        acc = torch.zeros(8, dtype=torch.float32, device=logp.device)
        f = lambda t: None if t is None else t.contiguous().float()
        args = [f(logp), f(old_logp), f(adv), f(weight), f(mask), f(ref_logp), f(rollout_logp)]
        rc = _lib.lib().b200_ppo_loss(
            *[_lib.ptr(a) for a in args], _lib.ptr(dlogp), _lib.ptr(acc), ctypes.c_longlong(n),
            ctypes.c_float(cfg["eps_low"]), ctypes.c_float(cfg["eps_high"]), ctypes.c_float(cfg["dual_clip"] or 0.0),
            ctypes.c_float(cfg["kl_coef"]), ctypes.c_int(_KL[cfg["kl_estimator"]]), ctypes.c_int(_IS[cfg["is_mode"]]),
            ctypes.c_float(cfg["is_lo"]), ctypes.c_float(cfg["is_hi"]), _lib.stream_ptr())
        _lib.check_rc(rc, "ppo_loss")
        ctx.save_for_backward(dlogp)
        ctx.kl_coef = cfg["kl_coef"]
        ctx.mark_non_differentiable(acc)
        return acc[0] + cfg["kl_coef"] * acc[1], acc

    @staticmethod
    def backward(ctx, g, _):
        (dlogp,) = ctx.saved_tensors
        return g * dlogp, None, None, None, None, None, None, None


def ppo_loss(logp, old_logp, adv, mask, ref_logp=None, rollout_logp=None, weight=None, eps_low=0.2, eps_high=0.2,
             dual_clip=None, kl_coef=0.0, kl_estimator="k1", is_mode=None, is_lo=0.5, is_hi=2.0):
    """Clipped-surrogate policy loss + kl_coef * KL(logp || ref) in one kernel launch, with the PPO metrics.

    All tensors share one shape; `weight` holds the aggregation weight of each token (see token_mean_weight /
    seq_mean_weight) so that token-level and sample-level means, global normalisers and dp_size compensation
    (openrlhf/models/loss.py:11-39) are all expressed by the caller. Returns a dict with `loss` (differentiable
    w.r.t. logp) and detached `policy_loss, kl_loss, clip_ratio, ppo_kl, vllm_kl, kl`.
    """
    kw = dict(eps_low=eps_low, eps_high=eps_high, dual_clip=dual_clip, kl_coef=kl_coef, kl_estimator=kl_estimator,
              is_mode=is_mode, is_lo=is_lo, is_hi=is_hi)
    if not logp.is_cuda:
        return ppo_loss_reference(logp, old_logp, adv, mask, ref_logp, rollout_logp, weight, **kw)
    mask = mask.float()
    if weight is None:
        weight = token_mean_weight(mask)
    loss, acc = _PpoLoss.apply(logp, old_logp, adv, weight, mask, ref_logp, rollout_logp, kw)
    n = acc[5].clamp_min(1)
    return {"loss": loss, "policy_loss": acc[0], "kl_loss": acc[1], "clip_ratio": acc[2] / n, "ppo_kl": acc[3] / n,
            "vllm_kl": acc[4] / n, "kl": acc[6] / n}


def value_loss_reference(values, old_values, returns, mask, clip_eps=None, weight=None):
    w = token_mean_weight(mask.float()) if weight is None else weight
    if clip_eps is not None and clip_eps > 0:
        vc = old_values + (values - old_values).clamp(-clip_eps, clip_eps)
        loss = torch.max((vc - returns) ** 2, (values - returns) ** 2)
    else:
        loss = (values - returns) ** 2
    return 0.5 * (loss * w).sum()


class _ValueLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, old_values, returns, weight, clip_eps):
        dv = torch.empty_like(values, dtype=torch.float32)
        acc = torch.zeros(1, dtype=torch.float32, device=values.device)
        f = lambda t: t.contiguous().float()
        rc = _lib.lib().b200_value_loss(_lib.ptr(f(values)), _lib.ptr(f(old_values)), _lib.ptr(f(returns)),
                                        _lib.ptr(f(weight)), _lib.ptr(dv), _lib.ptr(acc),
                                        ctypes.c_longlong(values.numel()), ctypes.c_float(clip_eps or 0.0),
                                        _lib.stream_ptr())
        _lib.check_rc(rc, "value_loss")
        ctx.save_for_backward(dv)
        return acc[0]

    @staticmethod
    def backward(ctx, g):
        (dv,) = ctx.saved_tensors
        return g * dv, None, None, None, None


def value_loss(values, old_values, returns, mask, clip_eps=None, weight=None):
    """0.5 * mean(max((clip(V, V_old +- eps) - R)^2, (V - R)^2)) (openrlhf/models/loss.py:233-269)."""
    if not values.is_cuda:
        return value_loss_reference(values, old_values, returns, mask, clip_eps, weight)
    if weight is None:
        weight = token_mean_weight(mask.float())
    return _ValueLoss.apply(values, old_values, returns, weight, clip_eps)


def gae_advantages_reference(values, kl, seq_reward, mask, beta=0.0, gamma=1.0, lambd=1.0, clip=(-10.0, 10.0)):
    mask = mask.float()
    B, A = mask.shape
    r_seq = seq_reward.float().clamp(clip[0], clip[1])
    last = A - 1 - mask.flip(-1).argmax(-1)
    rewards = (-beta * kl.float()) if kl is not None else torch.zeros_like(mask)
    rewards = rewards.clone()
    rewards[torch.arange(B, device=mask.device), last] += r_seq
    rewards = rewards * mask
    adv = torch.zeros_like(mask)
    if values is not None:
        v = values.float() * mask
        last_adv = torch.zeros(B, device=mask.device)
        for t in reversed(range(A)):
            nv = v[:, t + 1] if t < A - 1 else torch.zeros(B, device=mask.device)
            delta = rewards[:, t] + gamma * nv - v[:, t]
            last_adv = delta + gamma * lambd * last_adv
            adv[:, t] = last_adv
        ret = adv + v
    else:
        run = torch.zeros(B, device=mask.device)
        for t in reversed(range(A)):
            run = rewards[:, t] + gamma * run
            adv[:, t] = run
        ret = adv.clone()
    return adv, ret, rewards.sum(-1)


def gae_advantages(values, kl, seq_reward, mask, beta=0.0, gamma=1.0, lambd=1.0, clip=(-10.0, 10.0)):
    """Reward shaping (-beta*kl per token, clipped sequence reward at the last action token) followed by GAE when
    `values` is given, else discounted cumulative returns. Returns (advantages, returns, per-sequence reward sum)."""
    if not mask.is_cuda:
        return gae_advantages_reference(values, kl, seq_reward, mask, beta, gamma, lambd, clip)
    mask = mask.contiguous().float()
    B, A = mask.shape
    adv = torch.empty_like(mask)
    ret = torch.empty_like(mask)
    rsum = torch.empty(B, dtype=torch.float32, device=mask.device)
    f = lambda t: None if t is None else t.contiguous().float()
    values, kl, seq_reward = f(values), f(kl), f(seq_reward)
    rc = _lib.lib().b200_gae(_lib.ptr(values), _lib.ptr(kl), _lib.ptr(seq_reward), _lib.ptr(mask), _lib.ptr(adv),
                             _lib.ptr(ret), _lib.ptr(rsum), ctypes.c_int(B), ctypes.c_int(A), ctypes.c_float(beta),
                             ctypes.c_float(gamma), ctypes.c_float(lambd), ctypes.c_float(clip[0]),
                             ctypes.c_float(clip[1]), _lib.stream_ptr())
    _lib.check_rc(rc, "gae")
    return adv, ret, rsum


def masked_whiten_reference(x, mask, std_norm=True, stats=None):
    mask = mask.float()
    if stats is None:
        n = mask.sum().clamp_min(1)
        mean = (x * mask).sum() / n
        var = (((x - mean) ** 2) * mask).sum() / n
    else:
        s, ss, n = stats
        n = max(n, 1.0)
        mean = s / n
        var = max(ss / n - mean * mean, 0.0)
    rs = torch.rsqrt(torch.as_tensor(var, dtype=torch.float32).clamp_min(1e-8)) if std_norm else 1.0
    return (x - mean) * rs


def masked_stats(x, mask):
    """[sum(x*m), sum(x^2*m), sum(m)] as a 3-element fp32 tensor (all-reduce it across ranks for global whitening)."""
    if not x.is_cuda:
        m = mask.float()
        return torch.stack([(x * m).sum(), (x * x * m).sum(), m.sum()])
    acc = torch.zeros(4, dtype=torch.float32, device=x.device)
    xc, mc = x.contiguous().float(), mask.contiguous().float()
    rc = _lib.lib().b200_masked_stats(_lib.ptr(xc), _lib.ptr(mc), ctypes.c_longlong(xc.numel()), _lib.ptr(acc),
                                      _lib.stream_ptr())
    _lib.check_rc(rc, "masked_stats")
    return acc[:3]


def masked_whiten(x, mask, std_norm=True, stats=None):
    """(x - mean) * rsqrt(max(var, 1e-8)) over masked entries; in place on CUDA. `stats` overrides the local statistics."""
    if not x.is_cuda:
        st = None if stats is None else [float(s) for s in stats]
        return masked_whiten_reference(x, mask, std_norm, st)
    if stats is None:
        stats = masked_stats(x, mask)
    acc = torch.zeros(4, dtype=torch.float32, device=x.device)
    acc[:3] = stats
    assert x.is_contiguous() and x.dtype == torch.float32
    rc = _lib.lib().b200_whiten_apply(_lib.ptr(x), ctypes.c_longlong(x.numel()), _lib.ptr(acc),
                                      ctypes.c_int(int(std_norm)), _lib.stream_ptr())
    _lib.check_rc(rc, "whiten_apply")
    return x
