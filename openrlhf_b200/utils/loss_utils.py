"""Global loss normalisers: one token-mean (or sample-mean) per optimizer step regardless of how its tokens are
spread over micro-batches and data-parallel ranks (reference: openrlhf/utils/loss_utils.py:15-105)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def _get_dp_group(strategy):
    if not _dist_on():
        return None
    getter = getattr(strategy, "dp_group", None)
    if callable(getter):
        return getter()
    mesh = getattr(strategy, "ds_device_mesh", None)
    return mesh["dp"].get_group() if mesh is not None else None


def _count(mask: torch.Tensor):
    m = mask.float()
    return m.sum(), (m.reshape(m.shape[0], -1).sum(-1) > 0).sum().float()


def get_loss_batch_info(strategy, loss_mask: torch.Tensor, *, replay_buffer=None, step: Optional[int] = None,
                        dynamic_batch: bool = False, batch_num_tokens: Optional[float] = None,
                        global_batch_size: Optional[float] = None) -> dict:
    """Normalisers for one micro-batch: explicit values win, then the replay buffer's precomputed per-step totals
    (dynamic batching), else the all-reduced counts of this mask."""
    group = _get_dp_group(strategy)
    dp_size = dist.get_world_size(group=group) if _dist_on() else 1
    if dynamic_batch and replay_buffer is not None and step is not None:
        batch_num_tokens = replay_buffer.dynamic_batch_num_tokens[step]
        global_batch_size = replay_buffer.dynamic_global_batch_size[step]
    tok, smp = _count(loss_mask)
    out = {}
    for name, given, local in (("batch_num_tokens", batch_num_tokens, tok), ("global_batch_size", global_batch_size, smp)):
        if given is None:
            v = local.to(loss_mask.device, dtype=torch.float32)
            if _dist_on():
                dist.all_reduce(v, op=dist.ReduceOp.SUM, group=group)
        else:
            v = torch.as_tensor(given, device=loss_mask.device, dtype=torch.float32)
        out[name] = v
    out["dp_size"] = dp_size
    return out


def _optimizer_step_loss_norm(masks, dp_group, dp_size: int, gas: int) -> dict:
    """Totals over every micro-batch of one optimizer step and every DP rank, divided by `gas` (the engine divides
    each micro-loss by gas again, so the accumulated gradient is that of one global mean)."""
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    tot = torch.zeros(2, dtype=torch.float32, device=device)
    for m in masks:
        t, s = _count(m.to(device))
        tot[0] += t
        tot[1] += s
    if _dist_on():
        dist.all_reduce(tot, op=dist.ReduceOp.SUM, group=dp_group)
    return {"dp_size": dp_size, "batch_num_tokens": tot[0] / gas, "global_batch_size": tot[1] / gas}


def iter_grad_accum_global_norm(data_iter, strategy, accumulated_gradient: int, mask_fn):
    """Yield (item, normalisers); items are grouped into windows of `accumulated_gradient` micro-batches that share
    the same normalisers. A trailing partial window is normalised by its own totals."""
    group = _get_dp_group(strategy)
    dp_size = dist.get_world_size(group=group) if _dist_on() else 1
    gas = max(int(accumulated_gradient), 1)
    pending = []

    def flush():
        info = _optimizer_step_loss_norm([mask_fn(x) for x in pending], group, dp_size, gas)
        for x in pending:
            yield x, info

    for item in data_iter:
        pending.append(item)
        if len(pending) == gas:
            yield from flush()
            pending = []
    if pending:
        yield from flush()
