"""Mixture-of-experts block of the Qwen3-MoE architecture: top-k softmax router, SwiGLU experts stored as fused 3-D
tensors (gate_up [E, 2I, H], down [E, H, I]) and the load-balancing auxiliary loss.

Behavioural parity target: transformers' Qwen3MoeSparseMoeBlock / load_balancing_loss_func, which the reference
trains through ``output.aux_loss`` (openrlhf/trainer/ray/ppo_actor.py:339-343). Tokens are sorted by expert once and
each expert runs on its contiguous slice of rows, so expert GEMMs see dense [rows_e, H] operands.
"""
from __future__ import annotations

import os

import torch

from ..ops import functional as F
from ..ops.gemm import gemm


class _ExpertLinear(torch.autograd.Function):
    """y = x @ W[e].T for one expert; the weight gradient is accumulated into W.main_grad[e] when present."""

    @staticmethod
    def forward(ctx, x, W, e):
        ctx.save_for_backward(x)
        ctx.W, ctx.e = W, e
        if x.is_cuda and x.shape[0] > 0:
            return gemm(x, W.detach()[e])
        return (x.float() @ W.detach()[e].float().t()).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        W, e = ctx.W, ctx.e
        w = W.detach()[e]
        dy = dy.contiguous()
        if x.is_cuda and x.shape[0] > 0:
            dx = gemm(dy, w, b_mn=True)
        else:
            dx = (dy.float() @ w.float()).to(x.dtype)
        mg = getattr(W, "main_grad", None)
        if mg is not None:
            if x.is_cuda and x.shape[0] > 0:
                gemm(dy, x, a_mn=True, b_mn=True, out=mg[e], accumulate=True)
            else:
                mg[e].add_(dy.float().t() @ x.float())
            return dx, None, None
        dW = torch.zeros_like(W, dtype=torch.float32)
        dW[e] = dy.float().t() @ x.float()
        return dx, dW.to(W.dtype), None


class _ExpertSlice(torch.autograd.Function):
    """W[lo:hi] as a tensor whose weight gradient lands in W.main_grad[lo:hi] (or in a dense zero-padded grad)."""

    @staticmethod
    def forward(ctx, W, lo, hi):
        ctx.W, ctx.lo, ctx.hi = W, lo, hi
        ctx.set_materialize_grads(False)
        out = W.detach()[lo:hi]
        mg = getattr(W, "main_grad", None)
        if mg is not None:
            out.main_grad = mg[lo:hi]
        return out

    @staticmethod
    def backward(ctx, g):
        if g is None or getattr(ctx.W, "main_grad", None) is not None:
            return None, None, None
        full = torch.zeros_like(ctx.W)
        full[ctx.lo:ctx.hi] = g
        return full, None, None


class _RouteFn(torch.autograd.Function):
    """Fused router kernel (softmax + top-k + renormalisation); the backward pass is a handful of [T, E] PyTorch ops."""

    @staticmethod
    def forward(ctx, logits, top_k, norm_topk):
        import ctypes

        from ..ops import _lib

        T, E = logits.shape
        logits = logits.contiguous()
        probs = torch.empty_like(logits)
        w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, top_k, dtype=torch.int64, device=logits.device)
        rc = _lib.lib().b200_moe_route(_lib.ptr(logits), ctypes.c_int(T), ctypes.c_int(E), ctypes.c_int(top_k),
                                       ctypes.c_int(int(norm_topk)), _lib.ptr(probs), _lib.ptr(w), _lib.ptr(idx), None,
                                       None, _lib.stream_ptr())
        _lib.check_rc(rc, "moe_route")
        ctx.save_for_backward(probs, w, idx)
        ctx.norm = norm_topk
        ctx.mark_non_differentiable(idx)
        return w, idx, probs

    @staticmethod
    def backward(ctx, dw, _didx, dprobs):
        probs, w, idx = ctx.saved_tensors
        g = dprobs.clone() if dprobs is not None else torch.zeros_like(probs)
        if dw is not None:
            if ctx.norm:
                s = probs.gather(1, idx).sum(-1, keepdim=True)
                dsel = (dw - (dw * w).sum(-1, keepdim=True)) / s
            else:
                dsel = dw
            g.scatter_add_(1, idx, dsel)
        return probs * (g - (g * probs).sum(-1, keepdim=True)), None, None


def router_topk(x, router_w, top_k: int, norm_topk: bool):
    """Returns (weights [T,k] fp32, experts [T,k] int64, probs [T,E] fp32)."""
    logits = F.linear(x, router_w).float()
    if logits.is_cuda and logits.shape[1] <= 256 and top_k <= 32:
        return _RouteFn.apply(logits, top_k, norm_topk)
    probs = torch.softmax(logits, dim=-1)
    w, idx = probs.topk(top_k, dim=-1)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, probs


def load_balancing_loss(probs: torch.Tensor, idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """E * sum_e mean_tokens(onehot top-k)_e * mean_tokens(softmax)_e for one layer."""
    T, k = idx.shape
    counts = torch.zeros(num_experts, dtype=torch.float32, device=probs.device)
    counts.scatter_add_(0, idx.reshape(-1), torch.ones(T * k, dtype=torch.float32, device=probs.device))
    f = counts / max(T, 1)
    P = probs.mean(0)
    return num_experts * (f * P).sum()


class _GroupedLinear(torch.autograd.Function):
    """y[rows of e] = x[rows of e] @ W[e].T for all experts in one grouped tcgen05 GEMM (rows sorted by expert, each
    expert padded to a multiple of 128 rows). Backward: one grouped GEMM for the input gradient, one grouped
    weight-gradient GEMM accumulating in fp32 into W.main_grad."""

    @staticmethod
    def forward(ctx, x, W, tile_group, offsets):
        from ..ops.gemm import gemm_grouped_rows

        ctx.save_for_backward(x, tile_group, offsets)
        ctx.W = W
        return gemm_grouped_rows(x, W.detach(), tile_group)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm_grouped_rows, gemm_grouped_wgrad

        x, tile_group, offsets = ctx.saved_tensors
        W = ctx.W
        dy = dy.contiguous()
        dx = gemm_grouped_rows(dy, W.detach(), tile_group, b_mn=True)
        mg = getattr(W, "main_grad", None)
        if mg is not None:
            gemm_grouped_wgrad(dy, x, offsets, mg, accumulate=True)
            return dx, None, None, None
        dW = torch.zeros(W.shape, dtype=torch.float32, device=W.device)
        gemm_grouped_wgrad(dy, x, offsets, dW, accumulate=False)
        return dx, dW.to(W.dtype), None, None


def permute_plan(idx: torch.Tensor, num_experts: int):
    """Device-side (no host synchronisation) plan that sorts the T*k routed rows by expert and pads every expert to a
    multiple of 128 rows. Returns (tok [T*k] source token of each sorted row, dest [T*k] row in the padded buffer,
    order [T*k] position in the flattened (token, slot) list, tile_group int32 [P/128], offsets int32 [E+1], P)."""
    T, k = idx.shape
    E = num_experts
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    sorted_e = flat_e[order]
    # scatter_add instead of bincount: no device->host read, so the decode loop can be captured in a CUDA graph
    counts = torch.zeros(E, dtype=torch.long, device=idx.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))
    padded = (counts + 127) // 128 * 128
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    dense_starts = torch.cumsum(counts, 0) - counts
    rank_in_e = torch.arange(T * k, device=idx.device) - dense_starts[sorted_e]
    dest = starts[sorted_e] + rank_in_e
    P = (T * k + E * 127 + 127) // 128 * 128          # static upper bound: no device->host read
    tiles = torch.arange(P // 128, device=idx.device) * 128
    tg = torch.searchsorted(ends, tiles, right=True)
    tile_group = torch.where(tg < E, tg, torch.full_like(tg, -1)).to(torch.int32)
    # a tile past the last used row of its expert cannot exist (experts are padded to whole tiles); tiles past the
    # last expert's end are marked unused above
    offsets = torch.cat([starts[:1] * 0, ends]).to(torch.int32)
    return order // k, dest, order, tile_group, offsets, P


def moe_forward_grouped(x, router_w, gate_up, down, top_k: int, norm_topk: bool):
    """Grouped-GEMM MoE block (CUDA, bf16): router -> sort rows by expert -> gate_up -> SwiGLU -> down -> weighted
    combine. Same results as moe_forward (the per-expert loop) up to bf16 rounding."""
    T, H = x.shape
    E = gate_up.shape[0]
    w, idx, probs = router_topk(x, router_w, top_k, norm_topk)
    aux = load_balancing_loss(probs, idx, E)
    tok, dest, order, tile_group, offsets, P = permute_plan(idx, E)
    xs = torch.zeros(P, H, dtype=x.dtype, device=x.device).index_copy(0, dest, x[tok])
    gu = _GroupedLinear.apply(xs, gate_up, tile_group, offsets)
    a = F.swiglu(gu)
    ys = _GroupedLinear.apply(a, down, tile_group, offsets)
    wk = w.reshape(-1)[order].to(ys.dtype)[:, None]
    y = torch.zeros_like(x)
    y.index_add_(0, tok, ys[dest] * wk)
    return y, aux


def moe_forward(x, router_w, gate_up, down, top_k: int, norm_topk: bool, expert_range: tuple[int, int] | None = None,
                ep=None):
    """x [T,H] -> (y [T,H], aux_loss). `expert_range` restricts computation to local experts (expert parallelism:
    rows routed to other ranks are handled by the caller's dispatch/combine)."""
    T, H = x.shape
    E = gate_up.shape[0]
    if ep is not None and x.is_cuda:
        # expert parallel: this rank computes only its slice of the experts; every rank still holds all expert
        # weights (the slices other ranks own get zero gradient here and their values through the optimizer's
        # parameter all-gather), so the ZeRO engine needs no expert-specific handling
        w, idx, probs = router_topk(x, router_w, top_k, norm_topk)
        aux = load_balancing_loss(probs, idx, E)
        lo, hi = ep.rank * ep.E_loc, (ep.rank + 1) * ep.E_loc
        return ep.moe(x, w, idx, _ExpertSlice.apply(gate_up, lo, hi), _ExpertSlice.apply(down, lo, hi)), aux
    if (x.is_cuda and expert_range is None and x.dtype == torch.bfloat16 and H % 64 == 0
            and gate_up.shape[1] % 128 == 0 and os.environ.get("OPENRLHF_B200_MOE_LOOP", "0") != "1"):
        return moe_forward_grouped(x, router_w, gate_up, down, top_k, norm_topk)
    w, idx, probs = router_topk(x, router_w, top_k, norm_topk)
    aux = load_balancing_loss(probs, idx, E)
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // top_k
    sorted_e = flat_e[order]
    counts = torch.bincount(sorted_e, minlength=E).tolist()
    xs = x[tok]                                   # [T*k, H] rows grouped by expert
    outs = []
    start = 0
    e0, e1 = expert_range if expert_range is not None else (0, E)
    for e in range(E):
        n = counts[e]
        rows = xs[start:start + n]
        if n == 0 or not (e0 <= e < e1):
            outs.append(rows.new_zeros(n, H))
        else:
            gu = _ExpertLinear.apply(rows, gate_up, e)
            a = F.swiglu(gu)
            outs.append(_ExpertLinear.apply(a, down, e))
        start += n
    ys = torch.cat(outs, 0)                        # [T*k, H]
    wk = w.reshape(-1)[order].to(ys.dtype)[:, None]
    y = torch.zeros_like(x)
    y.index_add_(0, tok, ys * wk)
    return y, aux
