"""CUDA attention entry points: packed-sequence causal attention for training / prefill and paged-KV decode."""
from __future__ import annotations

import ctypes

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


def attention_varlen_cuda(q, k, v, cu_seqlens, max_seqlen, scale):
    """Packed causal GQA attention with autograd, through a library varlen flash-attention kernel."""
    if _varlen_impl is None:
        _pick_varlen_impl(q, k, v, cu_seqlens, max_seqlen, scale)
    return _varlen_impl(q, k, v, cu_seqlens, max_seqlen, scale)


_decode_ws: dict = {}


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, scale: float, out: torch.Tensor | None = None, splits: int = 1,
                 workspace: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """One-token-per-sequence attention over a paged KV cache (tcgen05 kernel).

    q [B, Hq, 128] bf16 contiguous; k_cache / v_cache [num_pages*128, Hkv, 128]; block_table int32 [B, max_pages];
    seq_lens int32 [B] (tokens already in the cache, current one included).
    """
    B, Hq, D = q.shape
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
    rc = _lib.lib().b200_rope_kvwrite(
        _lib.ptr(qkv), _lib.ptr(pos), _lib.ptr(slots), _lib.ptr(table), _lib.ptr(q_out), _lib.ptr(k_cache),
        _lib.ptr(v_cache), ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(qkv.stride(0)),
        ctypes.c_int(table.shape[0]), _lib.stream_ptr())
    _lib.check_rc(rc, "rope_kvwrite")
