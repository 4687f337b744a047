"""bf16 GEMM on tcgen05 tensor cores and the autograd ``linear`` built from it.

``gemm`` maps one-to-one onto the kernel in ``csrc/gemm_tcgen05.cu``; ``linear`` is what the model code calls in
place of ``nn.Linear`` (the reference's projections are HF ``nn.Linear`` modules: openrlhf/models/actor.py:149-157).
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    out_f32: bool = False,
    accumulate: bool = False,
    k_splits: int = 1,
    alpha: float = 1.0,
    bn: int = 0,
    split_stride: int = 0,
) -> torch.Tensor:
    """C[M,N] (+)= alpha * op(A) @ op(B) with bf16 inputs and fp32 accumulation.

    a_mn=False: ``a`` is [M,K]; a_mn=True: ``a`` is [K,M] (its transpose is used).
    b_mn=False: ``b`` is [N,K]; b_mn=True: ``b`` is [K,N].
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
        if accumulate:
            out.zero_()
    else:
        assert out.stride(-1) == 1
        out_f32 = out.dtype == torch.float32
    if split_stride:
        assert out.dtype == torch.float32 and out.numel() >= k_splits * split_stride
    else:
        assert out.shape == (M, N)
    if M == 0 or N == 0:
        return out
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and not out_f32
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and not out_f32
        assert residual.stride(0) == out.stride(0)
    st = _lib.status_word(a.device)
    if _use_pair_kernel(M, N, K, k_splits, split_stride, bn):
        rc = _lib.lib().b200_gemm2_bf16(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(residual),
            ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(out.stride(0)),
            ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)), ctypes.c_int(int(out_f32)),
            ctypes.c_int(int(accumulate)), ctypes.c_int(int(k_splits)), ctypes.c_float(alpha), ctypes.c_int(256),
            _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "b200_gemm2_bf16")
        return out
    rc = _lib.lib().b200_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(residual),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(N if split_stride else out.stride(0)),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)), ctypes.c_int(int(out_f32)),
        ctypes.c_int(int(accumulate)), ctypes.c_int(int(k_splits)), ctypes.c_longlong(int(split_stride)),
        ctypes.c_float(alpha), ctypes.c_int(bn),
        _lib.ptr(st), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "b200_gemm_bf16")
    return out


PAIR_KERNEL = os.environ.get("OPENRLHF_B200_GEMM2", "1")      # "0": keep every GEMM on the single-CTA kernel


def _use_pair_kernel(M: int, N: int, K: int, k_splits: int, split_stride: int, bn: int) -> bool:
    """The CTA-pair kernel (csrc/gemm2_tcgen05.cu) takes the large training / prefill GEMMs: at least one 256-row
    tile pair per cluster slot, no split-K slabs, caller did not ask for a specific tile width."""
    if PAIR_KERNEL != "1" or split_stride or bn not in (0, 256):
        return False
    return M >= 1024 and N >= 256 and K >= 256 and ((M + 255) // 256) * ((N + 255) // 256) * max(k_splits, 1) >= 74


def gemm_swiglu(x: torch.Tensor, w: torch.Tensor, want_gate_up: bool = False, bn: int = 0):
    """silu(x @ w[:I].T) * (x @ w[I:].T) in one kernel: the gate and up products of the same output columns share a
    tile and the SwiGLU runs in the GEMM epilogue on the fp32 accumulators. x [M, K], w [2I, K] (gate rows, then up
    rows). Returns (y [M, I], gate_up [M, 2I] bf16 or None: the products the backward pass needs)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    I = w.shape[0] // 2
    assert w.shape == (2 * I, K) and swiglu_fusable(I)
    y = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=x.device) if want_gate_up else None
    if M == 0:
        return y, gu
    st = _lib.status_word(x.device)
    if PAIR_KERNEL == "1" and bn in (0, 256) and M >= 1024 and ((M + 255) // 256) * (I // 128) >= 74:
        rc = _lib.lib().b200_gemm2_bf16_swiglu(
            _lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(gu), ctypes.c_int(M), ctypes.c_int(I), ctypes.c_int(K),
            ctypes.c_int(x.stride(0)), ctypes.c_int(w.stride(0)), ctypes.c_int(I), ctypes.c_int(2 * I),
            ctypes.c_int(256), _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "b200_gemm2_bf16_swiglu")
        return y, gu
    rc = _lib.lib().b200_gemm_bf16_swiglu(
        _lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(gu), ctypes.c_int(M), ctypes.c_int(I), ctypes.c_int(K),
        ctypes.c_int(x.stride(0)), ctypes.c_int(w.stride(0)), ctypes.c_int(I), ctypes.c_int(2 * I), ctypes.c_int(bn),
        _lib.ptr(st), _lib.stream_ptr())
    _lib.check_rc(rc, "b200_gemm_bf16_swiglu")
    return y, gu


def swiglu_fusable(intermediate: int) -> bool:
    """The fused kernel pairs 128-row (or 64-row) blocks of the gate and up matrices."""
    return intermediate % 128 == 0


_splitk_ws: dict = {}
_splitk_retired: list = []  # outgrown buffers stay alive: captured CUDA graphs may still point at them


def splitk_workspace(device, numel: int) -> torch.Tensor:
    """fp32 scratch for split-K partial products, grown on demand and reused by every call on the device."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _splitk_ws.get(key)
    if ws is None or ws.numel() < numel:
        if ws is not None:
            _splitk_retired.append(ws)
        ws = torch.empty(max(numel, 1 << 24), dtype=torch.float32, device=device)
        _splitk_ws[key] = ws
    return ws


def gemm_splitk(a: torch.Tensor, b: torch.Tensor, splits: int, bias: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, out: torch.Tensor | None = None, bn: int = 0,
                workspace: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 C = A @ B^T (+bias)(+residual) for small M: K is cut into `splits` slabs so that every SM streams a share
    of the weights; fp32 partial products go to a scratch buffer and a second kernel reduces them."""
    M, K = a.shape
    N = b.shape[0]
    kb_total = (K + 63) // 64
    per = (kb_total + splits - 1) // splits
    splits = (kb_total + per - 1) // per          # no empty K slab
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if splits <= 1:
        return gemm(a, b, bias=bias, residual=residual, out=out, bn=bn)
    ws = workspace if workspace is not None else splitk_workspace(a.device, splits * M * N)
    assert ws.numel() >= splits * M * N
    gemm(a, b, out=ws, k_splits=splits, split_stride=M * N, bn=bn)
    rc = _lib.lib().b200_splitk_reduce(_lib.ptr(ws), ctypes.c_int(splits), _lib.ptr(bias), _lib.ptr(residual),
                                       _lib.ptr(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(out.stride(0)),
                                       _lib.stream_ptr())
    _lib.check_rc(rc, "splitk_reduce")
    return out


# ---------------------------------------------------------------------------------------------- grouped (MoE) GEMMs
def gemm_grouped_rows(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, *, b_mn: bool = False,
                      bn: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Rows of ``a`` [P, K] are sorted by group and every group is padded to a multiple of 128 rows; tile_group int32
    [P/128] names the group of each 128-row tile (< 0: padding tile, left untouched in the output).

    b_mn=False: ``w`` is [G, N, K]; out[rows of g] = a[rows of g] @ w[g].T        (expert forward)
    b_mn=True : ``w`` is [G, K, N]; out[rows of g] = a[rows of g] @ w[g]          (expert input gradient)
    """
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    P, K = a.shape
    G = w.shape[0]
    N = w.shape[2] if b_mn else w.shape[1]
    assert (w.shape[1] if b_mn else w.shape[2]) == K and P % 128 == 0 and tile_group.numel() == P // 128
    if out is None:
        out = torch.zeros(P, N, dtype=torch.bfloat16, device=a.device)
    else:
        assert out.shape == (P, N) and out.is_contiguous() and out.dtype == torch.bfloat16
    rc = _lib.lib().b200_gemm_bf16_grouped(
        _lib.ptr(a), _lib.ptr(w), _lib.ptr(out), ctypes.c_int(P), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(K),
        ctypes.c_int(w.shape[2]), ctypes.c_int(N), ctypes.c_int(1 if b_mn else 0), ctypes.c_int(1), _lib.ptr(tile_group),
        ctypes.c_int(w.shape[1]), None, ctypes.c_int(G), ctypes.c_longlong(0), ctypes.c_int(0), ctypes.c_int(bn),
        _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_grouped_rows")
    return out


def gemm_grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, group_offsets: torch.Tensor, out: torch.Tensor,
                       accumulate: bool = True, bn: int = 0) -> torch.Tensor:
    """out[g] (+)= dy[rows of g].T @ x[rows of g] for every group; dy [P, M], x [P, N] sorted / padded as above,
    group_offsets int32 [G+1] padded row offsets, out fp32 [G, M, N]."""
    assert dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and dy.is_contiguous() and x.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous()
    P, M = dy.shape
    N = x.shape[1]
    G = out.shape[0]
    assert out.shape[1] == M and out.shape[2] == N and group_offsets.numel() == G + 1
    rc = _lib.lib().b200_gemm_bf16_grouped(
        _lib.ptr(dy), _lib.ptr(x), _lib.ptr(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(P), ctypes.c_int(M),
        ctypes.c_int(N), ctypes.c_int(N), ctypes.c_int(1), ctypes.c_int(2), None, ctypes.c_int(0),
        _lib.ptr(group_offsets), ctypes.c_int(G), ctypes.c_longlong(M * N), ctypes.c_int(1 if accumulate else 0),
        ctypes.c_int(bn), _lib.ptr(_lib.status_word(dy.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_grouped_wgrad")
    return out
