"""Autograd-aware operator API used by the model code.

Every op dispatches on the device of its input: CUDA tensors run the sm_100a kernels of ``csrc/``; CPU tensors run
the plain PyTorch restatement in ``ops/reference.py`` (that path exists for the CPU oracle and the unit tests).
Weight gradients are accumulated in fp32 straight into ``param.main_grad`` when the parameter carries that attribute
(set by the ZeRO engine), which fuses gradient accumulation into the wgrad GEMM epilogue.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib, reference
from .gemm import gemm

_c_int = ctypes.c_int
_c_ll = ctypes.c_longlong
_c_f = ctypes.c_float


def _L():
    return _lib.lib()


def _acc_grad(param: torch.Tensor, grad_fn):
    """Accumulate a gradient into param.main_grad (fp32) if present, else return it for autograd."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        grad_fn(mg)
        return None
    buf = torch.zeros(param.shape, dtype=torch.float32, device=param.device)
    grad_fn(buf)
    return buf.to(param.dtype)


# ---------------------------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.bias_ref = bias
        ctx.w_ref = w
        return gemm(x, w, bias=bias, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            T = x.shape[0]
            tiles = ((w.shape[0] + 127) // 128) * ((w.shape[1] + 255) // 256)
            splits = max(1, min(8, 148 // max(tiles, 1), T // 512)) if tiles < 148 else 1
            dw = _acc_grad(ctx.w_ref, lambda buf: gemm(dy, x, a_mn=True, b_mn=True, out=buf, accumulate=True,
                                                      k_splits=splits))
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _acc_grad(ctx.bias_ref, lambda buf: buf.add_(dy.float().sum(0)))
        dres = dy if ctx.has_res and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T (+ bias) (+ residual); x [T, K], w [N, K]."""
    if not x.is_cuda:
        return reference.linear(x, w, bias, residual)
    if w.shape[0] % 8 or w.shape[1] % 8:
        # the TMA tiles want 16-byte rows: a projection with fewer than 8 (or a ragged number of) outputs, such as the
        # router of a model with 4 experts, is too small for the tensor-core kernel to matter
        return reference.linear(x, w, bias, residual)
    return _Linear.apply(x, w, bias, residual)


# ---------------------------------------------------------------------------------------------- RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        T, H = x.shape
        y = torch.empty_like(x)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        rc = _L().b200_rmsnorm_fwd(_lib.ptr(x), None, _lib.ptr(w), _lib.ptr(y), None, _lib.ptr(rstd), _c_int(T),
                                   _c_int(H), _c_int(x.stride(0)), _c_int(y.stride(0)), _c_f(eps), _lib.stream_ptr())
        _lib.check_rc(rc, "rmsnorm_fwd")
        ctx.save_for_backward(x, w, rstd)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        xc = x.contiguous()
        T, H = xc.shape
        dx = torch.empty_like(xc)
        mg = getattr(ctx.w_ref, "main_grad", None)
        dw_buf = mg if mg is not None else torch.zeros(H, dtype=torch.float32, device=x.device)
        rc = _L().b200_rmsnorm_bwd(_lib.ptr(xc), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), None, _lib.ptr(dx),
                                   _lib.ptr(dw_buf), _c_int(T), _c_int(H), _lib.stream_ptr())
        _lib.check_rc(rc, "rmsnorm_bwd")
        return dx, (None if mg is not None else dw_buf.to(w.dtype)), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if not x.is_cuda:
        return reference.rmsnorm(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


# ---------------------------------------------------------------------------------------------- RoPE
_rope_tables: dict = {}


def rope_table(head_dim: int, theta: float, max_pos: int, device) -> torch.Tensor:
    """[max_pos, head_dim/2, 2] fp32 (cos, sin), rounded through bf16 like the HF rotary module's outputs."""
    key = (head_dim, float(theta), int(max_pos), str(device))
    tab = _rope_tables.get(key)
    if tab is None:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
        ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
        tab = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.bfloat16).float().contiguous()
        _rope_tables[key] = tab
    return tab


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, table, n_heads, head_dim):
        out = qkv.clone()
        _rope_inplace(out, pos, table, n_heads, head_dim, 1.0)
        ctx.save_for_backward(pos, table)
        ctx.n_heads, ctx.head_dim = n_heads, head_dim
        return out

    @staticmethod
    def backward(ctx, d):
        pos, table = ctx.saved_tensors
        d = d.clone()
        _rope_inplace(d, pos, table, ctx.n_heads, ctx.head_dim, -1.0)
        return d, None, None, None, None


def _rope_inplace(qkv, pos, table, n_heads, head_dim, sign):
    T = qkv.shape[0]
    rc = _L().b200_rope(_lib.ptr(qkv), _lib.ptr(pos), _lib.ptr(table), _c_int(T), _c_int(n_heads), _c_int(head_dim),
                        _c_int(qkv.stride(0)), _c_f(sign), _c_int(table.shape[0]), _lib.stream_ptr())
    _lib.check_rc(rc, "rope")


def rope(qkv: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """Rotate the first ``n_heads`` heads (q heads then k heads) of every row of qkv [T, *]; pos is int32 [T]."""
    if not qkv.is_cuda:
        return reference.rope(qkv, pos, table, n_heads, head_dim)
    return _Rope.apply(qkv, pos, table, n_heads, head_dim)


# ---------------------------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        T, F2 = gu.shape
        y = torch.empty(T, F2 // 2, dtype=gu.dtype, device=gu.device)
        rc = _L().b200_swiglu_fwd(_lib.ptr(gu), _lib.ptr(y), _c_ll(T), _c_int(F2 // 2), _lib.stream_ptr())
        _lib.check_rc(rc, "swiglu_fwd")
        ctx.save_for_backward(gu)
        return y

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        dy = dy.contiguous()
        dgu = torch.empty_like(gu)
        rc = _L().b200_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dy), _lib.ptr(dgu), _c_ll(gu.shape[0]),
                                  _c_int(gu.shape[1] // 2), _lib.stream_ptr())
        _lib.check_rc(rc, "swiglu_bwd")
        return dgu


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """silu(gu[:, :F]) * gu[:, F:]"""
    if not gu.is_cuda:
        return reference.swiglu(gu)
    return _SwiGLU.apply(gu.contiguous())


class _LinearSwiGLU(torch.autograd.Function):
    """y = swiglu(x @ w.T) with the activation in the GEMM epilogue; the bf16 gate / up products are written next to
    y only when a backward pass will need them."""

    @staticmethod
    def forward(ctx, x, w):
        from .gemm import gemm_swiglu

        need = any(ctx.needs_input_grad)
        y, gu = gemm_swiglu(x, w, want_gate_up=need)
        ctx.save_for_backward(x, w, gu)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, gu = ctx.saved_tensors
        dy = dy.contiguous()
        dgu = torch.empty_like(gu)
        rc = _L().b200_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dy), _lib.ptr(dgu), _c_ll(gu.shape[0]),
                                  _c_int(gu.shape[1] // 2), _lib.stream_ptr())
        _lib.check_rc(rc, "swiglu_bwd")
        dx = gemm(dgu, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            T = x.shape[0]
            tiles = ((w.shape[0] + 127) // 128) * ((w.shape[1] + 255) // 256)
            splits = max(1, min(8, 148 // max(tiles, 1), T // 512)) if tiles < 148 else 1
            dw = _acc_grad(ctx.w_ref, lambda buf: gemm(dgu, x, a_mn=True, b_mn=True, out=buf, accumulate=True,
                                                       k_splits=splits))
        return dx, dw


def linear_swiglu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """swiglu(x @ w.T) for w = [gate rows | up rows]; one kernel on the GPU when the shapes allow it."""
    from .gemm import swiglu_fusable

    if x.is_cuda and x.dtype == torch.bfloat16 and swiglu_fusable(w.shape[0] // 2) and x.stride(1) == 1:
        return _LinearSwiGLU.apply(x, w)
    return swiglu(linear(x, w))


# ---------------------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        T = ids.numel()
        V, H = table.shape
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
        rc = _L().b200_embedding_fwd(_lib.ptr(ids), _lib.ptr(table), _lib.ptr(out), _c_int(T), _c_int(H), _c_int(V),
                                     _lib.stream_ptr())
        _lib.check_rc(rc, "embedding_fwd")
        ctx.save_for_backward(ids)
        ctx.table_ref = table
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        table = ctx.table_ref
        V, H = table.shape
        dout = dout.contiguous()

        def fn(buf):
            rc = _L().b200_embedding_bwd(_lib.ptr(ids), _lib.ptr(dout), _lib.ptr(buf), _c_int(ids.numel()), _c_int(H),
                                         _c_int(V), _lib.stream_ptr())
            _lib.check_rc(rc, "embedding_bwd")

        return None, _acc_grad(table, fn)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not table.is_cuda:
        return reference.embedding(ids, table)
    return _Embedding.apply(ids.contiguous().long(), table)


# ---------------------------------------------------------------------------------------------- attention
def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                     scale: float | None = None) -> torch.Tensor:
    """Causal attention over a packed token stream. q [T,Hq,D], k/v [T,Hkv,D], cu_seqlens int32 [n+1]."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda:
        return reference.attention_varlen(q, k, v, cu_seqlens, scale)
    from .attention import attention_varlen_cuda

    return attention_varlen_cuda(q, k, v, cu_seqlens, max_seqlen, scale)


# ---------------------------------------------------------------------------------------------- LM head -> log-probs
def _lmhead_fusable(h: torch.Tensor, w: torch.Tensor) -> bool:
    return (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and h.stride(1) == 1 and w.stride(1) == 1
            and h.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and w.shape[0] % 8 == 0
            and h.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


class _FusedLogprob(torch.autograd.Function):
    """log p(label) (and optionally entropy) per token from hidden states without ever writing [T, V] logits.

    Forward: one tcgen05 GEMM whose epilogue reduces every 128 x 256 logits tile to per-row softmax partials (32 bytes
    per row and tile instead of 512 bytes of bf16 logits), then a merge kernel over a row's tiles. Backward: the
    logits are recomputed in row chunks by the same GEMM with an epilogue that writes d logits = g/T (onehot -
    softmax) directly as the bf16 operand of the dH and dW GEMMs (no separate pass over the chunk)."""

    @staticmethod
    def forward(ctx, h, w, labels, temperature, want_entropy, chunk):
        T, K = h.shape
        V = w.shape[0]
        dev = h.device
        logp = torch.empty(T, dtype=torch.float32, device=dev)
        ent = torch.empty(T, dtype=torch.float32, device=dev) if want_entropy else None
        lse = torch.empty(T, dtype=torch.float32, device=dev)
        L = _L()
        inv_t = 1.0 / temperature
        if _lmhead_fusable(h, w):
            nb = int(L.b200_lmhead_num_blocks(_c_int(V)))
            rows_max = max(128, min(T, (1 << 28) // (nb * 8)))            # partial buffer of at most 1 GiB
            partial = torch.empty(nb * min(T, rows_max) * 8, dtype=torch.float32, device=dev)
            st = _lib.status_word(dev)
            for s in range(0, T, rows_max):
                e = min(T, s + rows_max)
                rc = L.b200_lmhead_partials(_lib.ptr(h[s:e]), _lib.ptr(w), _lib.ptr(labels[s:e]), _c_f(inv_t),
                                            _c_int(int(want_entropy)), _lib.ptr(partial), _c_int(e - s), _c_int(V),
                                            _c_int(K), _c_int(h.stride(0)), _c_int(w.stride(0)), _lib.ptr(st),
                                            _lib.stream_ptr())
                _lib.check_rc(rc, "lmhead_partials")
                rc = L.b200_lmhead_merge(_lib.ptr(partial), _c_int(nb), _c_int(e - s), _c_f(inv_t), _lib.ptr(logp[s:e]),
                                         _lib.ptr(ent[s:e]) if ent is not None else None, _lib.ptr(lse[s:e]),
                                         _lib.stream_ptr())
                _lib.check_rc(rc, "lmhead_merge")
            ctx.fused = True
        else:
            for s in range(0, T, chunk):
                e = min(T, s + chunk)
                logits = gemm(h[s:e], w)
                rc = L.b200_logprob_rows(_lib.ptr(logits), _c_int(1), _c_int(e - s), _c_int(V), _c_int(logits.stride(0)),
                                         _lib.ptr(labels[s:e]), _c_f(temperature), _lib.ptr(logp[s:e]),
                                         _lib.ptr(ent[s:e]) if ent is not None else None, _lib.ptr(lse[s:e]),
                                         _lib.stream_ptr())
                _lib.check_rc(rc, "logprob_rows")
            ctx.fused = False
        ctx.save_for_backward(h, w, labels, lse)
        ctx.temperature, ctx.chunk, ctx.w_ref = temperature, chunk, w
        ctx.want_entropy = want_entropy
        if want_entropy:
            ctx.mark_non_differentiable(ent)
            return logp, ent
        return logp, None

    @staticmethod
    def backward(ctx, dlogp, _dent):
        h, w, labels, lse = ctx.saved_tensors
        T, V = h.shape[0], w.shape[0]
        K = h.shape[1]
        inv_t = 1.0 / ctx.temperature
        dh = torch.empty_like(h)
        mg = getattr(ctx.w_ref, "main_grad", None)
        dw_buf = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dlogp = dlogp.float().contiguous()
        L = _L()
        st = _lib.status_word(h.device)
        for s in range(0, T, ctx.chunk):
            e = min(T, s + ctx.chunk)
            if ctx.fused:
                dz = torch.empty(e - s, V, dtype=torch.bfloat16, device=h.device)
                from .gemm import PAIR_KERNEL
                # CTA-pair kernel when the chunk has enough 256-row tiles to fill the GPU
                fn = L.b200_lmhead2_dlogits if (PAIR_KERNEL == "1" and e - s >= 1024) else L.b200_lmhead_dlogits
                rc = fn(_lib.ptr(h[s:e]), _lib.ptr(w), _lib.ptr(dz), _lib.ptr(labels[s:e]),
                        _lib.ptr(lse[s:e]), _lib.ptr(dlogp[s:e]), _c_f(inv_t), _c_int(e - s),
                        _c_int(V), _c_int(K), _c_int(h.stride(0)), _c_int(w.stride(0)), _c_int(V),
                        _lib.ptr(st), _lib.stream_ptr())
                _lib.check_rc(rc, "lmhead_dlogits")
            else:
                dz = gemm(h[s:e], w)
                # d logits = g/T * (onehot - softmax(z/T))
                rc = L.b200_logprob_bwd_rows(_lib.ptr(dz), _c_int(e - s), _c_int(V), _c_int(dz.stride(0)),
                                             _lib.ptr(labels[s:e]), _lib.ptr(lse[s:e]), _lib.ptr(dlogp[s:e]),
                                             _c_f(inv_t), _lib.stream_ptr())
                _lib.check_rc(rc, "logprob_bwd_rows")
            gemm(dz, w, b_mn=True, out=dh[s:e])
            gemm(dz, h[s:e], a_mn=True, b_mn=True, out=dw_buf, accumulate=True)
        return dh, (None if mg is not None else dw_buf.to(w.dtype)), None, None, None, None


def fused_logprob(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                  want_entropy: bool = False, chunk: int = 4096):
    """Returns (logp [T] fp32, entropy [T] fp32 or None) for labels [T] given hidden states h [T,H] and lm_head w [V,H].

    Replaces lm_head -> logits.float() -> cross-entropy -> compute_entropy of the reference
    (openrlhf/models/actor.py:265-296, openrlhf/models/utils.py:139-186).
    """
    if not h.is_cuda:
        return reference.fused_logprob(h, w, labels, temperature, want_entropy)
    return _FusedLogprob.apply(h.contiguous(), w, labels.contiguous().long(), float(temperature), want_entropy, chunk)


# ---------------------------------------------------------------------------------------------- vocabulary-parallel LM head
def _vp_combine(stats: torch.Tensor):
    """stats [n, T, 4] per vocabulary shard: (tempered lse, label logit / temperature or 0, untempered lse, untempered
    E[z]). Returns (logp [T], entropy [T], global tempered lse [T])."""
    lse_g = torch.logsumexp(stats[..., 0], dim=0)
    logp = stats[..., 1].sum(0) - lse_g
    lse1_g = torch.logsumexp(stats[..., 2], dim=0)
    w = torch.exp(stats[..., 2] - lse1_g)
    ent = lse1_g - (w * stats[..., 3]).sum(0)
    return logp, ent, lse_g


def _lmhead_stats(h, w, labels, inv_t: float, want_entropy: bool):
    """(log p(label), entropy at temperature 1 or None, log-sum-exp of z / T) per row from the fused LM-head kernels:
    the GEMM epilogue leaves softmax partials, a merge kernel folds them; no logits are written. Labels outside
    [0, rows of w) contribute no label term (vocabulary shards)."""
    T, K = h.shape
    V = w.shape[0]
    dev = h.device
    L = _L()
    logp = torch.empty(T, dtype=torch.float32, device=dev)
    ent = torch.empty(T, dtype=torch.float32, device=dev) if want_entropy else None
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    nb = int(L.b200_lmhead_num_blocks(_c_int(V)))
    rows_max = max(128, min(T, (1 << 28) // (nb * 8)))
    partial = torch.empty(nb * min(T, rows_max) * 8, dtype=torch.float32, device=dev)
    st = _lib.status_word(dev)
    for s in range(0, T, rows_max):
        e = min(T, s + rows_max)
        rc = L.b200_lmhead_partials(_lib.ptr(h[s:e]), _lib.ptr(w), _lib.ptr(labels[s:e]), _c_f(inv_t),
                                    _c_int(int(want_entropy)), _lib.ptr(partial), _c_int(e - s), _c_int(V), _c_int(K),
                                    _c_int(h.stride(0)), _c_int(w.stride(0)), _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "lmhead_partials")
        rc = L.b200_lmhead_merge(_lib.ptr(partial), _c_int(nb), _c_int(e - s), _c_f(inv_t), _lib.ptr(logp[s:e]),
                                 _lib.ptr(ent[s:e]) if ent is not None else None, _lib.ptr(lse[s:e]), _lib.stream_ptr())
        _lib.check_rc(rc, "lmhead_merge")
    return logp, ent, lse


class _VocabParallelLogprob(torch.autograd.Function):
    """Fused log-prob over an lm_head whose rows (vocabulary) are split across a group: every rank streams its own
    V/n columns of the logits, 16 bytes of statistics per token and rank are exchanged, and the backward pass needs one
    all-reduce of dh. No rank ever holds [T, V] logits."""

    @staticmethod
    def forward(ctx, h, w, labels, vocab_start, group, temperature, want_entropy, chunk):
        import torch.distributed as dist

        T, Vl = h.shape[0], w.shape[0]
        lab = labels.long() - vocab_start
        inr = (lab >= 0) & (lab < Vl)
        stats = torch.zeros(T, 4, dtype=torch.float32, device=h.device)
        ctx.fused = bool(h.is_cuda and _lmhead_fusable(h, w))
        if ctx.fused:
            lab = lab.contiguous()
            logp, ent, lse = _lmhead_stats(h, w, lab, 1.0 / temperature, want_entropy)
            stats[:, 0] = lse
            stats[:, 1] = torch.where(inr, logp + lse, torch.zeros_like(logp))
            if want_entropy:
                lse1 = lse if temperature == 1.0 else _lmhead_stats(h, w, lab, 1.0, False)[2]
                stats[:, 2], stats[:, 3] = lse1, lse1 - ent
        elif h.is_cuda:
            logp = torch.empty(T, dtype=torch.float32, device=h.device)
            lse = torch.empty_like(logp)
            ent = torch.empty_like(logp)
            lse1 = torch.empty_like(logp)
            scratch = torch.empty_like(logp)
            for s in range(0, T, chunk):
                e = min(T, s + chunk)
                logits = gemm(h[s:e], w)
                args = (_lib.ptr(logits), _c_int(1), _c_int(e - s), _c_int(Vl), _c_int(logits.stride(0)), _lib.ptr(lab[s:e]))
                _lib.check_rc(_L().b200_logprob_rows(*args, _c_f(temperature), _lib.ptr(logp[s:e]),
                                                    _lib.ptr(ent[s:e]) if want_entropy else None, _lib.ptr(lse[s:e]),
                                                    _lib.stream_ptr()), "logprob_rows")
                if want_entropy:
                    if temperature == 1.0:
                        lse1[s:e] = lse[s:e]
                    else:
                        _lib.check_rc(_L().b200_logprob_rows(*args, _c_f(1.0), _lib.ptr(scratch[s:e]), None,
                                                            _lib.ptr(lse1[s:e]), _lib.stream_ptr()), "logprob_rows")
            stats[:, 0] = lse
            stats[:, 1] = torch.where(inr, logp + lse, torch.zeros_like(logp))
            if want_entropy:
                stats[:, 2], stats[:, 3] = lse1, lse1 - ent
        else:
            z = h.float() @ w.float().t()
            stats[:, 0] = torch.logsumexp(z / temperature, -1)
            stats[:, 1] = torch.where(inr, z.gather(1, lab.clamp(0, Vl - 1)[:, None]).squeeze(1) / temperature,
                                      torch.zeros(T))
            stats[:, 2] = torch.logsumexp(z, -1)
            stats[:, 3] = (torch.softmax(z, -1) * z).sum(-1)
        n = dist.get_world_size(group)
        allst = torch.empty(n * T, 4, dtype=torch.float32, device=h.device)
        dist.all_gather_into_tensor(allst, stats, group=group)
        logp_g, ent_g, lse_g = _vp_combine(allst.view(n, T, 4))
        ctx.save_for_backward(h, w, lab, lse_g)
        ctx.group, ctx.temperature, ctx.chunk, ctx.w_ref = group, temperature, chunk, w
        if want_entropy:
            ctx.mark_non_differentiable(ent_g)
            return logp_g, ent_g
        return logp_g, None

    @staticmethod
    def backward(ctx, dlogp, _dent):
        import torch.distributed as dist

        h, w, lab, lse_g = ctx.saved_tensors
        T, Vl = h.shape[0], w.shape[0]
        inv_t = 1.0 / ctx.temperature
        dlogp = dlogp.float().contiguous()
        mg = getattr(ctx.w_ref, "main_grad", None)
        if h.is_cuda:
            dh = torch.empty_like(h)
            dw_buf = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            st = _lib.status_word(h.device)
            for s in range(0, T, ctx.chunk):
                e = min(T, s + ctx.chunk)
                if ctx.fused:
                    # the recomputed logits leave the GEMM epilogue as d logits (global log-sum-exp; the one-hot term
                    # only on the rank whose shard holds the label)
                    logits = torch.empty(e - s, Vl, dtype=torch.bfloat16, device=h.device)
                    rc = _L().b200_lmhead_dlogits(_lib.ptr(h[s:e]), _lib.ptr(w), _lib.ptr(logits), _lib.ptr(lab[s:e]),
                                                  _lib.ptr(lse_g[s:e]), _lib.ptr(dlogp[s:e]), _c_f(inv_t), _c_int(e - s),
                                                  _c_int(Vl), _c_int(h.shape[1]), _c_int(h.stride(0)),
                                                  _c_int(w.stride(0)), _c_int(Vl), _lib.ptr(st), _lib.stream_ptr())
                    _lib.check_rc(rc, "lmhead_dlogits")
                else:
                    logits = gemm(h[s:e], w)
                    rc = _L().b200_logprob_bwd_rows(_lib.ptr(logits), _c_int(e - s), _c_int(Vl),
                                                    _c_int(logits.stride(0)), _lib.ptr(lab[s:e]), _lib.ptr(lse_g[s:e]),
                                                    _lib.ptr(dlogp[s:e]), _c_f(inv_t), _lib.stream_ptr())
                    _lib.check_rc(rc, "logprob_bwd_rows")
                gemm(logits, w, b_mn=True, out=dh[s:e])
                gemm(logits, h[s:e], a_mn=True, b_mn=True, out=dw_buf, accumulate=True)
            dw = None if mg is not None else dw_buf.to(w.dtype)
        else:
            z = h.float() @ w.float().t()
            p = torch.exp(z * inv_t - lse_g[:, None])
            onehot = torch.zeros_like(p)
            inr = (lab >= 0) & (lab < Vl)
            onehot[inr, lab[inr]] = 1.0
            dz = dlogp[:, None] * inv_t * (onehot - p)
            dh = (dz @ w.float()).to(h.dtype)
            dw = (dz.t() @ h.float()).to(w.dtype)
            if mg is not None:
                mg.add_(dw.float())
                dw = None
        dist.all_reduce(dh, group=ctx.group)      # every vocabulary shard contributes to dh
        return dh, dw, None, None, None, None, None, None


def vocab_parallel_logprob(h: torch.Tensor, w_local: torch.Tensor, labels: torch.Tensor, vocab_start: int, group,
                           temperature: float = 1.0, want_entropy: bool = False, chunk: int = 4096):
    """fused_logprob with the lm_head rows [vocab_start, vocab_start + w_local.shape[0]) on this rank. All ranks of
    `group` pass the same h and labels; returns the same (logp, entropy) on every rank."""
    return _VocabParallelLogprob.apply(h.contiguous(), w_local, labels.contiguous(), int(vocab_start), group,
                                       float(temperature), want_entropy, chunk)


# ---------------------------------------------------------------------------------------------- value head
def value_head(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """[T,H] x [1,H] -> [T] fp32 (tiny GEMV; fp32 accumulate)."""
    return (h.float() @ w.float().t()).squeeze(-1)
