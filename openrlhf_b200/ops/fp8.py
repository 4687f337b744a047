"""fp8 (e4m3) GEMM path: per-tensor quantisation and the tcgen05 ``kind::f8f6f4`` GEMM with fp32 accumulation.

``quantize_e4m3`` returns the quantised tensor (torch.float8_e4m3fn view) and its de-quantisation scale as a device
scalar; ``gemm_e4m3`` multiplies two quantised operands and applies the product of the two scales in the epilogue
(passed as a device pointer, so there is no host read between quantisation and GEMM). ``Fp8Linear`` keeps a weight
quantised once and quantises activations per call: twice the tensor-core rate and half the weight bytes of the bf16
path for large-M rollout work (prefill). The reference reaches fp8 rollout through vLLM's quantisation option
(openrlhf/trainer/ray/vllm_engine.py passes engine kwargs through); scaling here is per tensor, not per block.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def quantize_e4m3(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x bf16 (numel multiple of 8, contiguous) -> (q float8_e4m3fn with x's shape, scale fp32 [1]); x ~ q * scale."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(1, dtype=torch.int32, device=x.device)
    rc = _lib.lib().b200_quantize_e4m3(_lib.ptr(x), ctypes.c_longlong(x.numel()), _lib.ptr(q), _lib.ptr(scale),
                                       _lib.ptr(scratch), _lib.stream_ptr())
    _lib.check_rc(rc, "quantize_e4m3")
    return q.view(torch.float8_e4m3fn), scale


def gemm_e4m3(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
              bias: torch.Tensor | None = None, residual: torch.Tensor | None = None, bn: int = 0) -> torch.Tensor:
    """bf16 C[M,N] = (a_scale * b_scale) * a[M,K] @ b[N,K]^T (+ bias)(+ residual); a, b float8_e4m3fn, K % 16 == 0."""
    assert a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn and a.is_contiguous() and b.is_contiguous()
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and K % 16 == 0
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    alpha = (a_scale * b_scale).float().contiguous()
    rc = _lib.lib().b200_gemm_e4m3(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(residual),
                                   ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(K), ctypes.c_int(K),
                                   ctypes.c_int(N), ctypes.c_float(1.0), _lib.ptr(alpha), ctypes.c_int(bn),
                                   _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_e4m3")
    return out


class Fp8Linear:
    """y = x @ W^T with W quantised once (inference only)."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        self.wq, self.w_scale = quantize_e4m3(weight.detach().contiguous())
        self.bias = bias

    def __call__(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        xq, xs = quantize_e4m3(x.contiguous())
        return gemm_e4m3(xq, xs, self.wq, self.w_scale, self.bias, residual)
