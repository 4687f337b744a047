"""Plain PyTorch restatements of every operator (fp32 math where the kernels use fp32). Used on CPU by the oracle and
as the comparison target of the kernel tests; never on the GPU production path."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def linear(x, w, bias=None, residual=None):
    y = (x.float() @ w.float().t())
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def rmsnorm(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y.to(x.dtype).float() * w.float()).to(x.dtype)


def rope(qkv, pos, table, n_heads, head_dim):
    """table [max_pos, head_dim/2, 2]; rotate-half layout on the first n_heads heads of each row."""
    T = qkv.shape[0]
    half = head_dim // 2
    cs = table[pos.long().clamp(0, table.shape[0] - 1)]  # [T, half, 2]
    cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
    x = qkv[:, : n_heads * head_dim].reshape(T, n_heads, head_dim).float()
    lo, hi = x[..., :half], x[..., half:]
    out = torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1).to(qkv.dtype)
    return torch.cat([out.reshape(T, n_heads * head_dim), qkv[:, n_heads * head_dim:]], dim=1)


def swiglu(gu):
    Fh = gu.shape[1] // 2
    g, u = gu[:, :Fh].float(), gu[:, Fh:].float()
    return (F.silu(g) * u).to(gu.dtype)


def embedding(ids, table):
    return table[ids.long()]


def attention_varlen(q, k, v, cu_seqlens, scale):
    """Causal attention per document of a packed stream. q [T,Hq,D], k/v [T,Hkv,D]."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        qs = q[s:e].float().transpose(0, 1)                      # [Hq, L, D]
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        att = (qs @ ks.transpose(1, 2)) * scale
        L = e - s
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        out[s:e] = (att @ vs).transpose(0, 1).to(q.dtype)
    return out


def fused_logprob(h, w, labels, temperature=1.0, want_entropy=False):
    logits = h.float() @ w.float().t()
    ent = None
    if want_entropy:
        lse0 = torch.logsumexp(logits, -1)
        p = torch.softmax(logits, -1)
        ent = lse0 - (p * logits).sum(-1)
    z = logits / temperature
    logp = z.gather(-1, labels.long()[:, None]).squeeze(-1) - torch.logsumexp(z, -1)
    return logp, ent


def paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, scale, page=128):
    """q [B,Hq,D]; caches [num_pages*page, Hkv, D]."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    rep = Hq // Hkv
    out = torch.empty_like(q)
    for b in range(B):
        L = int(seq_lens[b])
        n = (L + page - 1) // page
        idx = torch.cat([torch.arange(page, device=q.device) + int(block_table[b, i]) * page for i in range(n)])[:L]
        ks = k_cache[idx].float().transpose(0, 1).repeat_interleave(rep, 0)  # [Hq, L, D]
        vs = v_cache[idx].float().transpose(0, 1).repeat_interleave(rep, 0)
        att = torch.einsum("hd,hld->hl", q[b].float(), ks) * scale
        out[b] = torch.einsum("hl,hld->hd", att.softmax(-1), vs).to(q.dtype)
    return out
