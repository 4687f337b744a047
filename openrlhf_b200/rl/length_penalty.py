"""Reward adjustments that depend on response length: the DAPO overlong penalty and the ProRL stop-properly penalty.
Vectorised over each experience batch; semantics of openrlhf/trainer/ppo_utils/length_penalty.py:16-153."""
from __future__ import annotations

import logging

import torch

logger = logging.getLogger(__name__)


def apply_overlong_penalty(experiences, max_new_tokens: int, overlong_buffer_len: float,
                           overlong_penalty_factor: float = 1.0) -> int:
    """r += -min(len - (max_new - buffer), buffer) / buffer * factor for responses longer than max_new - buffer."""
    if max_new_tokens < overlong_buffer_len:
        raise AssertionError(f"max_new_tokens ({max_new_tokens}) must be >= overlong_buffer_len ({overlong_buffer_len})")
    soft_limit = max_new_tokens - overlong_buffer_len
    hit = 0
    for e in experiences:
        over = (e.response_length.to(e.rewards.dtype) - soft_limit).clamp(max=overlong_buffer_len)
        pen = torch.where(over > 0, -over / overlong_buffer_len * overlong_penalty_factor, torch.zeros_like(over))
        e.rewards += pen.to(e.rewards.device)
        hit += int((over > 0).sum())
    return hit


def apply_stop_properly_penalty(experiences, stop_properly_penalty_coef: float) -> int:
    """Truncated samples: reward *= coef for coef in [0,1]; reward = coef for negative coef."""
    c = stop_properly_penalty_coef
    if c >= 0 and not (0 <= c <= 1):
        raise AssertionError(f"stop_properly_penalty_coef must be in [0, 1] or negative, got {c}")
    hit = 0
    for e in experiences:
        if e.truncated is None:
            continue
        t = e.truncated.bool().to(e.rewards.device)
        e.rewards = torch.where(t, torch.full_like(e.rewards, c) if c < 0 else e.rewards * c, e.rewards)
        hit += int(t.sum())
    return hit


def apply_length_penalties(experiences, args) -> None:
    total = sum(len(e.rewards) for e in experiences)
    buf = getattr(args.reward, "overlong_buffer_len", None)
    if buf is not None:
        max_new = getattr(args.rollout, "max_new_tokens", None) or args.data.max_len
        n = apply_overlong_penalty(experiences, max_new, buf, getattr(args.reward, "overlong_penalty_factor", 1.0))
        logger.info("overlong penalty: %d/%d samples penalised (buffer %s)", n, total, buf)
    coef = getattr(args.reward, "stop_properly_penalty_coef", None)
    if coef is not None:
        n = apply_stop_properly_penalty(experiences, coef)
        logger.info("stop-properly penalty: %d/%d samples truncated (coef %s)", n, total, coef)
    for e in experiences:
        if "reward" in e.info:
            e.info["reward"] = e.rewards.clone()
