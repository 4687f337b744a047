"""Sampler binding: temperature / top-k / top-p sampling with the log-prob of the drawn token."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def sample(logits: torch.Tensor, temperature: float | torch.Tensor = 1.0, top_k: int | torch.Tensor = -1,
           top_p: float | torch.Tensor = 1.0, seed: int = 0, step: int | torch.Tensor = 0,
           out_tokens: torch.Tensor | None = None, out_logprobs: torch.Tensor | None = None,
           active: torch.Tensor | None = None):
    """logits [B, V] (bf16 or fp32, last dim contiguous). Returns (tokens int64 [B], logprobs fp32 [B]).

    `temperature`, `top_k` (int32) and `top_p` (fp32) may be per-row tensors (one value per request); `step` may be a
    1-element int64 CUDA tensor so that a captured graph draws fresh noise on every replay. Rows whose `active` entry is
    0 keep their previous outputs.
    """
    B, V = logits.shape
    if out_tokens is None:
        out_tokens = torch.zeros(B, dtype=torch.int64, device=logits.device)
    if out_logprobs is None:
        out_logprobs = torch.zeros(B, dtype=torch.float32, device=logits.device)
    if not logits.is_cuda:
        tok, lp = sample_reference(logits, temperature, top_k, top_p, seed, step)
        keep = torch.ones(B, dtype=torch.bool) if active is None else active.bool()
        out_tokens.copy_(torch.where(keep, tok, out_tokens))
        out_logprobs.copy_(torch.where(keep, lp, out_logprobs))
        return out_tokens, out_logprobs
    assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
    t_ptr, t_scalar = (None, float(temperature)) if not isinstance(temperature, torch.Tensor) else (temperature, 1.0)
    s_ptr, s_scalar = (None, int(step)) if not isinstance(step, torch.Tensor) else (step, 0)
    k_ptr, k_scalar = (None, int(top_k)) if not isinstance(top_k, torch.Tensor) else (top_k, -1)
    p_ptr, p_scalar = (None, float(top_p)) if not isinstance(top_p, torch.Tensor) else (top_p, 1.0)
    assert k_ptr is None or (k_ptr.dtype == torch.int32 and k_ptr.numel() >= B)
    assert p_ptr is None or (p_ptr.dtype == torch.float32 and p_ptr.numel() >= B)
    rc = _lib.lib().b200_sample(
        _lib.ptr(logits), ctypes.c_int(int(logits.dtype == torch.bfloat16)), ctypes.c_int(B), ctypes.c_int(V),
        ctypes.c_int(logits.stride(0)), _lib.ptr(t_ptr), ctypes.c_float(t_scalar), ctypes.c_int(k_scalar),
        ctypes.c_float(p_scalar), ctypes.c_ulonglong(int(seed) & (2**64 - 1)), _lib.ptr(s_ptr),
        ctypes.c_longlong(s_scalar), _lib.ptr(out_tokens), _lib.ptr(out_logprobs), _lib.ptr(active), _lib.ptr(k_ptr),
        _lib.ptr(p_ptr), _lib.stream_ptr())
    _lib.check_rc(rc, "sample")
    return out_tokens, out_logprobs


def sample_reference(logits, temperature=1.0, top_k=-1, top_p=1.0, seed=0, step=0):
    """PyTorch restatement (different random stream, same distribution). Per-row tensors are accepted for
    temperature / top_k / top_p; rows with temperature <= 1e-6 are greedy and report the log-prob at temperature 1."""
    z0 = logits.float()
    B, V = z0.shape
    dev = logits.device
    temp = torch.as_tensor(temperature, dtype=torch.float32, device=dev).expand(B) if not isinstance(
        temperature, torch.Tensor) else temperature.float().reshape(-1)[:B]
    greedy = temp <= 1e-6
    z = z0 / torch.where(greedy, torch.ones_like(temp), temp)[:, None]
    tk = torch.as_tensor(top_k, device=dev).reshape(-1).expand(B) if not isinstance(top_k, torch.Tensor) \
        else top_k.reshape(-1)[:B]
    tp = torch.as_tensor(top_p, dtype=torch.float32, device=dev).reshape(-1).expand(B) if not isinstance(
        top_p, torch.Tensor) else top_p.float().reshape(-1)[:B]
    sz, si = z.sort(-1, descending=True)
    rank = torch.arange(V, device=dev)[None, :]
    kk = torch.where((tk > 0) & (tk < V), tk, torch.full_like(tk, V)).long()[:, None]
    drop = rank >= kk
    sz = sz.masked_fill(drop, float("-inf"))
    pr = sz.softmax(-1)
    cp = pr.cumsum(-1)
    drop_p = (cp - pr >= tp[:, None]) & (tp[:, None] < 1.0)
    sz = sz.masked_fill(drop_p, float("-inf"))
    zf = torch.full_like(z, float("-inf")).scatter(-1, si, sz)
    zf = torch.where(greedy[:, None], z0, zf)
    step_i = int(step.reshape(-1)[0]) if isinstance(step, torch.Tensor) else int(step)
    g = torch.Generator(device=dev).manual_seed((int(seed) * 1000003 + step_i) % (2 ** 63))
    tok = torch.multinomial(zf.softmax(-1), 1, generator=g).squeeze(-1)
    tok = torch.where(greedy, z0.argmax(-1), tok)
    return tok, torch.log_softmax(zf, -1).gather(-1, tok[:, None]).squeeze(-1)
