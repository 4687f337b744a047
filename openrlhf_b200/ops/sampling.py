"""Sampler binding: temperature / top-k / top-p sampling with the log-prob of the drawn token."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def sample(logits: torch.Tensor, temperature: float | torch.Tensor = 1.0, top_k: int = -1, top_p: float = 1.0,
           seed: int = 0, step: int | torch.Tensor = 0, out_tokens: torch.Tensor | None = None,
           out_logprobs: torch.Tensor | None = None, active: torch.Tensor | None = None):
    """logits [B, V] (bf16 or fp32, last dim contiguous). Returns (tokens int64 [B], logprobs fp32 [B]).

    `step` may be a 1-element int64 CUDA tensor so that a captured graph draws fresh noise on every replay.
    """
    if not logits.is_cuda:
        return sample_reference(logits, temperature, top_k, top_p, seed, step)
    B, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    if out_tokens is None:
        out_tokens = torch.empty(B, dtype=torch.int64, device=logits.device)
    if out_logprobs is None:
        out_logprobs = torch.empty(B, dtype=torch.float32, device=logits.device)
    t_ptr, t_scalar = (None, float(temperature)) if not isinstance(temperature, torch.Tensor) else (temperature, 1.0)
    s_ptr, s_scalar = (None, int(step)) if not isinstance(step, torch.Tensor) else (step, 0)
    rc = _lib.lib().b200_sample(
        _lib.ptr(logits), ctypes.c_int(int(logits.dtype == torch.bfloat16)), ctypes.c_int(B), ctypes.c_int(V),
        ctypes.c_int(logits.stride(0)), _lib.ptr(t_ptr), ctypes.c_float(t_scalar), ctypes.c_int(int(top_k)),
        ctypes.c_float(float(top_p)), ctypes.c_ulonglong(int(seed) & (2**64 - 1)), _lib.ptr(s_ptr),
        ctypes.c_longlong(s_scalar), _lib.ptr(out_tokens), _lib.ptr(out_logprobs), _lib.ptr(active), _lib.stream_ptr())
    _lib.check_rc(rc, "sample")
    return out_tokens, out_logprobs


def sample_reference(logits, temperature=1.0, top_k=-1, top_p=1.0, seed=0, step=0):
    """PyTorch restatement (different random stream, same distribution)."""
    z = logits.float()
    if isinstance(temperature, torch.Tensor) or temperature > 1e-6:
        z = z / temperature
    else:
        tok = z.argmax(-1)
        return tok, torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1)
    if top_k and top_k > 0:
        kth = z.topk(min(top_k, z.shape[-1]), -1).values[:, -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p < 1.0:
        sz, si = z.sort(-1, descending=True)
        cp = sz.softmax(-1).cumsum(-1)
        drop = cp - sz.softmax(-1) >= top_p
        sz = sz.masked_fill(drop, float("-inf"))
        z = torch.full_like(z, float("-inf")).scatter(-1, si, sz)
    g = torch.Generator(device=logits.device).manual_seed(int(seed) * 1000003 + int(step))
    tok = torch.multinomial(z.softmax(-1), 1, generator=g).squeeze(-1)
    return tok, torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1)
