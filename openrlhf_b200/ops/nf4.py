"""NF4 block quantisation (QLoRA's 4-bit NormalFloat, blocks of 64 values with one fp32 absmax each).

``--ds.load_in_4bit`` in the reference loads the frozen base weights through bitsandbytes in this format and trains
LoRA adapters on top with bf16 compute (openrlhf/models/actor.py:115-124). Here ``quantize`` / ``dequantize`` are own
kernels (``csrc/quant_nf4.cu``, PyTorch restatement on the CPU), and ``apply_to_model`` gives the projection weights
of a model exactly the values the 4-bit format can represent while keeping them in the bf16 flat buffer the GEMM
kernels read: with 180 GB per GPU the memory saving is not what the flag is needed for, the numerics of QLoRA are.
``pack_model`` / ``unpack_model`` convert between the flat buffer and the compact (codes, absmax) form for storage.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

BLOCK = 64
LEVELS = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])


def quantize(w: torch.Tensor):
    """w: bf16 (or fp32 on the CPU), numel a multiple of 64 -> (codes uint8 [n/2], absmax fp32 [n/64])."""
    n = w.numel()
    assert n % BLOCK == 0, "NF4 blocks hold 64 values"
    if w.is_cuda:
        w = w.contiguous()
        assert w.dtype == torch.bfloat16
        codes = torch.empty(n // 2, dtype=torch.uint8, device=w.device)
        absmax = torch.empty(n // BLOCK, dtype=torch.float32, device=w.device)
        rc = _lib.lib().b200_nf4_quantize(_lib.ptr(w), _lib.ptr(codes), _lib.ptr(absmax), ctypes.c_longlong(n),
                                          _lib.stream_ptr())
        _lib.check_rc(rc, "nf4_quantize")
        return codes, absmax
    x = w.detach().float().reshape(-1, BLOCK)
    absmax = x.abs().amax(dim=1)
    y = x / absmax.clamp_min(1e-30)[:, None]
    y = torch.where(absmax[:, None] > 0, y, torch.zeros_like(y))
    mid = 0.5 * (LEVELS[:-1] + LEVELS[1:])
    idx = (y[..., None] > mid).sum(-1).to(torch.uint8).reshape(-1, 2)
    return (idx[:, 0] << 4 | idx[:, 1]).contiguous(), absmax.contiguous()


def dequantize(codes: torch.Tensor, absmax: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    n = codes.numel() * 2
    if codes.is_cuda:
        out = torch.empty(n, dtype=torch.bfloat16, device=codes.device)
        rc = _lib.lib().b200_nf4_dequantize(_lib.ptr(codes), _lib.ptr(absmax), _lib.ptr(out), ctypes.c_longlong(n),
                                            _lib.stream_ptr())
        _lib.check_rc(rc, "nf4_dequantize")
        return out.to(dtype)
    idx = torch.stack([codes >> 4, codes & 15], dim=1).reshape(-1).long()
    return (LEVELS[idx].reshape(-1, BLOCK) * absmax[:, None]).reshape(-1).to(dtype)


def quantized_names(model) -> list[str]:
    """The frozen projection matrices (what bitsandbytes replaces by 4-bit linears): not embeddings, norms, heads."""
    return [s.name for s in model.specs
            if s.name.startswith("layers.") and len(s.shape) >= 2 and s.numel % BLOCK == 0 and "router" not in s.name]


@torch.no_grad()
def apply_to_model(model) -> int:
    """Round every projection weight to its NF4 value in place. Returns the number of quantised elements."""
    total = 0
    for name in quantized_names(model):
        p = model.p(name)
        flat = p.data.view(-1)
        codes, absmax = quantize(flat if flat.is_cuda else flat.float())
        flat.copy_(dequantize(codes, absmax, flat.dtype))
        total += flat.numel()
    model.nf4 = True
    return total


@torch.no_grad()
def pack_model(model) -> dict:
    """{name: (codes, absmax)} of the projection weights (4.5 bits per weight)."""
    return {n: quantize(model.p(n).data.view(-1) if model.flat.is_cuda else model.p(n).data.view(-1).float())
            for n in quantized_names(model)}


@torch.no_grad()
def unpack_model(model, packed: dict) -> None:
    for n, (codes, absmax) in packed.items():
        p = model.p(n)
        p.data.view(-1).copy_(dequantize(codes.to(p.device), absmax.to(p.device), p.dtype))
