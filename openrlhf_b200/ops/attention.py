"""CUDA attention entry points: packed-sequence causal attention for training / prefill and paged-KV decode."""
from __future__ import annotations

import ctypes
import weakref
import os

import torch

from . import _lib

PAGE = 128  # tokens per KV page (one tcgen05 kv tile)


_varlen_impl = None


def _pick_varlen_impl(q, k, v, cu_seqlens, max_seqlen, scale):
    """First working library varlen kernel on this GPU (flash-attn, then torch's varlen_attn)."""
    global _varlen_impl
    errors = []
    try:
        from flash_attn import flash_attn_varlen_func

        def fa(q, k, v, cu, mx, sc):
            return flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, softmax_scale=sc, causal=True)

        with torch.no_grad():
            fa(q[:8].contiguous(), k[:8].contiguous(), v[:8].contiguous(),
               torch.tensor([0, 8], dtype=torch.int32, device=q.device), 8, scale)
            torch.cuda.synchronize()
        _varlen_impl = fa
        return
    except Exception as e:  # noqa: BLE001
        errors.append(f"flash_attn: {e}")
    from torch.nn.attention.varlen import varlen_attn

    def tv(q, k, v, cu, mx, sc):
        rep = q.shape[1] // k.shape[1]
        if rep > 1:
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        return varlen_attn(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, mx, mx, scale=sc,
                           window_size=(-1, 0))

    _varlen_impl = tv


_tile_cache: dict = {}


def _query_tiles_cached(cu_seqlens: torch.Tensor, T: int, n_seqs: int, rows: int):
    """The tile list depends only on cu_seqlens, which every layer of a forward pass shares: keep the last few,
    keyed by tensor identity and in-place version (a weak reference guards against a recycled id)."""
    key = (id(cu_seqlens), cu_seqlens._version, T, rows)
    hit = _tile_cache.get(key)
    if hit is not None and hit[0]() is cu_seqlens:
        return hit[1]
    if len(_tile_cache) >= 8:
        _tile_cache.clear()
    val = _query_tiles(cu_seqlens, T, n_seqs, rows)
    _tile_cache[key] = (weakref.ref(cu_seqlens), val)
    return val


def _query_tiles(cu_seqlens: torch.Tensor, T: int, n_seqs: int, rows: int = 128):
    """Device-side list of `rows`-row query tiles: (tile_seq [n], tile_q0 [n]); n = T//rows + n_seqs is an upper
    bound, surplus entries carry tile_seq = n_seqs (the kernel skips them). No host synchronisation."""
    n = T // rows + n_seqs
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
    per = (lens + rows - 1) // rows
    ends = torch.cumsum(per, 0)
    t = torch.arange(n, device=cu_seqlens.device)
    seq = torch.searchsorted(ends, t, right=True)
    starts = ends - per
    q0 = (t - starts[seq.clamp_max(n_seqs - 1)]) * rows
    return seq.int().contiguous(), q0.int().contiguous(), n


def attn_fwd_tcgen05(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, scale: float,
                     tiles=None):
    """tcgen05 causal varlen forward. q [T,Hq,128], k/v [T,Hkv,128] (views with a common row stride are fine).
    Returns (out [T,Hq,128] bf16, lse [Hq,T] fp32). `tiles` = (tile_seq, tile_q0, n): run only these query tiles
    (rows of other tiles keep whatever `out` held); see attention_with_prefix."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128 and q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == D
    assert k.stride(1) == D and v.stride(1) == D and k.stride(2) == 1 and v.stride(2) == 1
    n_seqs = cu_seqlens.numel() - 1
    rows = 128 if (Hq // Hkv) % 2 == 0 else 256     # two heads per CTA, or two 128-row halves of one head
    tile_seq, tile_q0, n = tiles if tiles is not None else _query_tiles_cached(cu_seqlens, T, n_seqs, rows)
    out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    rc = _lib.lib().b200_attn_fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ctypes.c_int(q.stride(0)), ctypes.c_int(k.stride(0)),
        ctypes.c_int(v.stride(0)), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0), _lib.ptr(cu_seqlens),
        _lib.ptr(tile_seq), _lib.ptr(tile_q0), ctypes.c_int(n), ctypes.c_int(rows), _lib.ptr(out), ctypes.c_int(Hq * D), _lib.ptr(lse),
        ctypes.c_int(n_seqs), ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_float(scale),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "attn_fwd")
    return out, lse


def attn_bwd_tcgen05(q, k, v, out, dout, lse, cu_seqlens, scale, pos=None, rope_table=None):
    """tcgen05 causal varlen backward. q [T,Hq,128], k/v [T,Hkv,128] (the tensors the forward saw: rotated), out /
    dout [T,Hq,128], lse [Hq,T]. Returns dqkv bf16 [T, (Hq+2*Hkv)*128] = [dq | dk | dv]; when pos / rope_table are
    given, dq and dk are rotated back (gradient with respect to the un-rotated projections)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128 and out.is_contiguous()
    dout = dout if (dout.stride(2) == 1 and dout.stride(1) == D and dout.stride(0) % 8 == 0) else dout.contiguous()
    n_seqs = cu_seqlens.numel() - 1
    tile_seq, tile_k0, n = _query_tiles_cached(cu_seqlens, T, n_seqs, 128)
    W = (Hq + 2 * Hkv) * D
    delta = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    acc = torch.empty(T, W, dtype=torch.float32, device=q.device)
    dqkv = torch.empty(T, W, dtype=torch.bfloat16, device=q.device)
    rc = _lib.lib().b200_attn_bwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ctypes.c_int(q.stride(0)), ctypes.c_int(k.stride(0)),
        ctypes.c_int(v.stride(0)), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0), _lib.ptr(out),
        ctypes.c_int(Hq * D), _lib.ptr(dout), ctypes.c_int(dout.stride(0)), _lib.ptr(lse), _lib.ptr(cu_seqlens),
        _lib.ptr(tile_seq), _lib.ptr(tile_k0), ctypes.c_int(n), _lib.ptr(delta), _lib.ptr(acc), _lib.ptr(dqkv),
        _lib.ptr(pos), _lib.ptr(rope_table), ctypes.c_int(rope_table.shape[0] if rope_table is not None else 0),
        ctypes.c_int(n_seqs), ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_float(scale),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "attn_bwd")
    return dqkv


class _AttnVarlen(torch.autograd.Function):
    """Forward and backward on this repository's tcgen05 kernels."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, scale):
        out, lse = attn_fwd_tcgen05(q, k, v, cu_seqlens, scale)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        dqkv = attn_bwd_tcgen05(q, k, v, out, dout, lse, cu, ctx.scale)
        dq = dqkv[:, : Hq * D].view(T, Hq, D)
        dk = dqkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        dv = dqkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        return dq, dk, dv, None, None, None


class _RopeAttn(torch.autograd.Function):
    """Rotary embedding + causal varlen attention on the fused projection output qkv [T, (Hq+2*Hkv)*128]. The rotation
    is applied in place (nothing upstream keeps the projection output for its own backward); the backward returns one
    dqkv tensor in the same fused layout, so no per-slice gradient buffers are assembled."""

    @staticmethod
    def forward(ctx, qkv, pos, table, cu_seqlens, Hq, Hkv, scale):
        from .functional import _rope_inplace

        T, D = qkv.shape[0], 128
        if qkv._is_view() or qkv.is_leaf or not qkv.is_contiguous():
            qkv = qkv.clone()
        else:
            ctx.mark_dirty(qkv)
        _rope_inplace(qkv, pos, table, Hq + Hkv, D, 1.0)
        q = qkv[:, : Hq * D].view(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        out, lse = attn_fwd_tcgen05(q, k, v, cu_seqlens, scale)
        ctx.save_for_backward(qkv, out, lse, cu_seqlens, pos, table)
        ctx.dims = (Hq, Hkv, scale)
        return out.view(T, Hq * D), qkv

    @staticmethod
    def backward(ctx, dout, _dqkv_unused):
        qkv, out, lse, cu, pos, table = ctx.saved_tensors
        Hq, Hkv, scale = ctx.dims
        T, D = qkv.shape[0], 128
        q = qkv[:, : Hq * D].view(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        dqkv = attn_bwd_tcgen05(q, k, v, out, dout.view(T, Hq, D), lse, cu, scale, pos, table)
        return dqkv, None, None, None, None, None, None


def rope_attention(qkv: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, cu_seqlens: torch.Tensor, Hq: int,
                   Hkv: int, scale: float) -> torch.Tensor:
    """Fused rotary embedding + packed causal GQA attention (head_dim 128, bf16, CUDA). Returns [T, Hq*128]."""
    if torch.is_grad_enabled() and qkv.requires_grad:
        return _RopeAttn.apply(qkv, pos, table, cu_seqlens, Hq, Hkv, scale)[0]
    from .functional import _rope_inplace

    T, D = qkv.shape[0], 128
    qkv = qkv if (qkv.is_contiguous() and not qkv.requires_grad) else qkv.detach().clone()
    _rope_inplace(qkv, pos, table, Hq + Hkv, D, 1.0)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    return attn_fwd_tcgen05(q, k, v, cu_seqlens, scale)[0].view(T, Hq * D)


USE_OWN_FWD = os.environ.get("OPENRLHF_B200_ATTN_FWD", "1") == "1"


def _library_varlen(q, k, v, cu_seqlens, max_seqlen, scale):
    if _varlen_impl is None:
        _pick_varlen_impl(q, k, v, cu_seqlens, max_seqlen, scale)
    return _varlen_impl(q, k, v, cu_seqlens, max_seqlen, scale)


def attention_varlen_cuda(q, k, v, cu_seqlens, max_seqlen, scale):
    """Packed causal GQA attention with autograd."""
    if USE_OWN_FWD and q.shape[-1] == 128 and q.dtype == torch.bfloat16 and q.stride(1) == 128 and k.stride(1) == 128 \
            and v.stride(1) == 128:
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
            return _AttnVarlen.apply(q, k, v, cu_seqlens, max_seqlen, scale)
        return attn_fwd_tcgen05(q, k, v, cu_seqlens, scale)[0]
    return _library_varlen(q, k, v, cu_seqlens, max_seqlen, scale)


def query_tile_rows(Hq: int, Hkv: int) -> int:
    """Rows per query tile of the forward kernel: two heads of an even GQA group share 128 rows, otherwise one head
    takes two 128-row halves."""
    return 128 if (Hq // Hkv) % 2 == 0 else 256


def attention_with_prefix(q_new: torch.Tensor, k_all: torch.Tensor, v_all: torch.Tensor, cu_all: list[int],
                          starts: list[int], scale: float) -> torch.Tensor:
    """Causal attention of the NEW tokens of every sequence over its cached prefix plus the new tokens.

    k_all / v_all [Ta, Hkv, D]: keys / values of every sequence in full (prefix rows first), packed with boundaries
    cu_all (host ints). Sequence i has starts[i] prefix rows; q_new [Tn, Hq, D] holds the queries of the remaining rows
    in the same packed order. Used by chunked prefill, prefix-cache hits and the re-prefill of preempted rows.

    On the GPU the forward kernel runs unchanged: the queries are scattered to their global rows of a [Ta] buffer and
    only the query tiles that contain new rows are put on the tile list, so prefix rows cost no attention work."""
    Hq, D = q_new.shape[1], q_new.shape[2]
    Hkv = k_all.shape[1]
    n = len(starts)
    new_rows = torch.cat([torch.arange(cu_all[i] + starts[i], cu_all[i + 1]) for i in range(n)])
    if not q_new.is_cuda:
        rep = Hq // Hkv
        out = torch.empty_like(q_new)
        o = 0
        for i in range(n):
            a, b, s0 = cu_all[i], cu_all[i + 1], starts[i]
            L, m = b - a, b - a - s0
            qs = q_new[o:o + m].float().transpose(0, 1)
            ks = k_all[a:b].float().transpose(0, 1).repeat_interleave(rep, 0)
            vs = v_all[a:b].float().transpose(0, 1).repeat_interleave(rep, 0)
            att = (qs @ ks.transpose(1, 2)) * scale
            keep = torch.arange(L)[None, :] <= (torch.arange(m)[:, None] + s0)
            att = att.masked_fill(~keep, float("-inf")).softmax(-1)
            out[o:o + m] = (att @ vs).transpose(0, 1).to(q_new.dtype)
            o += m
        return out
    dev = q_new.device
    Ta = k_all.shape[0]
    rows = query_tile_rows(Hq, Hkv)
    seq_l, q0_l = [], []
    for i in range(n):
        L = cu_all[i + 1] - cu_all[i]
        for q0 in range(starts[i] // rows * rows, L, rows):
            seq_l.append(i)
            q0_l.append(q0)
    tiles = (torch.tensor(seq_l, dtype=torch.int32, device=dev), torch.tensor(q0_l, dtype=torch.int32, device=dev),
             len(seq_l))
    q_full = torch.zeros(Ta, Hq, D, dtype=q_new.dtype, device=dev)
    idx = new_rows.to(dev)
    q_full.index_copy_(0, idx, q_new)
    cu = torch.tensor(cu_all, dtype=torch.int32, device=dev)
    out, _ = attn_fwd_tcgen05(q_full, k_all.contiguous(), v_all.contiguous(), cu, scale, tiles=tiles)
    return out.index_select(0, idx)


_decode_ws: dict = {}


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, scale: float, out: torch.Tensor | None = None, splits: int = 1,
                 workspace: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """One-token-per-sequence attention over a paged KV cache (tcgen05 kernel).

    q [B, Hq, 128] bf16 contiguous; k_cache / v_cache [num_pages*128, Hkv, 128]; block_table int32 [B, max_pages];
    seq_lens int32 [B] (tokens already in the cache, current one included).
    """
    B, Hq, D = q.shape
    if not q.is_cuda:
        from . import reference

        res = reference.paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, scale, PAGE)
        if out is None:
            return res
        out.copy_(res)
        return out
    assert D == 128 and q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    Hkv = k_cache.shape[1]
    num_pages = k_cache.shape[0] // PAGE
    if out is None:
        out = torch.empty_like(q)
    part_o = part_ml = None
    if splits > 1:
        if workspace is None:
            key = (q.device.index, B, Hq, splits)
            workspace = _decode_ws.get(key)
            if workspace is None:
                workspace = (torch.empty(B * Hq * splits * D, dtype=torch.float32, device=q.device),
                             torch.empty(B * Hq * splits * 2, dtype=torch.float32, device=q.device))
                _decode_ws[key] = workspace
        part_o, part_ml = workspace
    rc = _lib.lib().b200_attn_decode(
        _lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(block_table), _lib.ptr(seq_lens), _lib.ptr(out),
        _lib.ptr(part_o), _lib.ptr(part_ml), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv),
        ctypes.c_int(num_pages), ctypes.c_int(block_table.shape[1]), ctypes.c_int(splits), ctypes.c_float(scale),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "attn_decode")
    return out


def rope_kvwrite(qkv: torch.Tensor, pos: torch.Tensor, slots: torch.Tensor, table: torch.Tensor, q_out: torch.Tensor,
                 k_cache: torch.Tensor, v_cache: torch.Tensor, Hq: int, Hkv: int) -> None:
    """RoPE on q,k of qkv [T, (Hq+2Hkv)*128]; writes roped q to q_out [T,Hq,128] and k,v into cache slot `slots[t]`."""
    T = qkv.shape[0]
    if not qkv.is_cuda:
        from . import reference

        D = q_out.shape[-1]
        r = reference.rope(qkv, pos, table, Hq + Hkv, D)
        q_out.copy_(r[:, : Hq * D].reshape(T, Hq, D))
        k_cache[slots.long()] = r[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
        v_cache[slots.long()] = r[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D].reshape(T, Hkv, D)
        return
    rc = _lib.lib().b200_rope_kvwrite(
        _lib.ptr(qkv), _lib.ptr(pos), _lib.ptr(slots), _lib.ptr(table), _lib.ptr(q_out), _lib.ptr(k_cache),
        _lib.ptr(v_cache), ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(qkv.stride(0)),
        ctypes.c_int(table.shape[0]), _lib.stream_ptr())
    _lib.check_rc(rc, "rope_kvwrite")
