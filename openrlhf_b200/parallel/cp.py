"""Context (sequence) parallelism for attention over NVLink peer memory.

The packed token stream is cut into ``world`` contiguous chunks of ``T_loc`` rows (a multiple of 128); documents are
padded to multiples of 128 tokens so that no 128-row K/V tile straddles two ranks. Every layer then runs

    forward :  rope (in place)  ->  copy of the fused qkv rows into a symmetric buffer  ->  barrier
               ->  ONE launch: gather CTAs pull the K/V rows this rank needs from their owners into a local buffer
                   (each remote byte crosses NVLink once) and publish a flag per tile; the attention CTAs of the same
                   launch consume tiles as they land
    backward:  barrier  ->  local query rows against the gathered K/V: dq local, dk/dv partial sums at global rows
               ->  barrier  ->  owner pulls and adds the peers' dk/dv partials (one pass)  ->  rope^-1 + cast

which is what the reference gets from ring-flash-attn's llama3 variant (all-gather of K/V per head stride, FA2 on the
local queries, reduce-scatter of dK/dV in backward; openrlhf/models/ring_attn_utils.py:9-41 sets it up,
openrlhf/models/actor.py:216-240 slices the inputs) with NCCL collectives between separate kernels.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.attention import _query_tiles_cached
from .symm import _ptr_array


class CPContext:
    def __init__(self, group, T_loc: int, Hq: int, Hkv: int, device, n_copy_y: int = 3):
        import torch.distributed._symmetric_memory as symm_mem

        assert T_loc % 128 == 0, "context-parallel chunks are multiples of 128 rows"
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.T_loc, self.Hq, self.Hkv = T_loc, Hq, Hkv
        self.W = (Hq + 2 * Hkv) * 128
        self.kv_cols = 2 * Hkv * 128
        self.T_total = T_loc * self.world
        self.n_copy_y = n_copy_y
        self.qkv = [symm_mem.empty(T_loc * self.W, dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        self._hq = [symm_mem.rendezvous(b, self.group) for b in self.qkv]
        self.qkv_ptrs = [_ptr_array(h.buffer_ptrs) for h in self._hq]
        self.dkv_g = symm_mem.empty(self.T_total * self.kv_cols, dtype=torch.float32, device=self.device)
        self._hd = symm_mem.rendezvous(self.dkv_g, self.group)
        self.dkv_ptrs = _ptr_array(self._hd.buffer_ptrs)
        self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self._hs = symm_mem.rendezvous(self.pad, self.group)
        self.pad_ptrs = _ptr_array(self._hs.buffer_ptrs)
        self.flags = torch.zeros(self.T_total // 128, dtype=torch.int32, device=self.device)
        self.flag_epoch = 0
        self.bar_epoch = 0
        self.parity = 0
        self.wait_limit_s = float(os.environ.get("OPENRLHF_B200_WAIT_LIMIT_S", "60"))
        self._lo_cache: dict = {}
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # ------------------------------------------------------------------------------------------------ helpers
    def barrier(self):
        self.bar_epoch += 1
        rc = _lib.lib().b200_symm_barrier(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                          ctypes.c_int(0), ctypes.c_uint(self.bar_epoch),
                                          ctypes.c_double(self.wait_limit_s), _lib.ptr(_lib.status_word(self.device)),
                                          _lib.stream_ptr())
        _lib.check_rc(rc, "symm_barrier")

    def kv_tile_lo(self, cu_seqlens: torch.Tensor, cu_cpu=None) -> int:
        """First 128-row K/V tile this rank needs: the start of the document that holds its first row."""
        key = (id(cu_seqlens), cu_seqlens._version)
        hit = self._lo_cache.get(key)
        if hit is not None:
            return hit
        cu = (cu_cpu if cu_cpu is not None else cu_seqlens.cpu()).tolist()
        first = self.rank * self.T_loc
        start = 0
        for a, b in zip(cu[:-1], cu[1:]):
            if a <= first < b:
                start = a
                break
        else:
            start = first        # past the last document (pure padding)
        if len(self._lo_cache) > 8:
            self._lo_cache.clear()
        self._lo_cache[key] = start // 128
        return start // 128

    def attention(self, qkv: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, cu_seqlens: torch.Tensor,
                  scale: float | None = None, cu_cpu=None) -> torch.Tensor:
        """qkv [T_loc, W] bf16 (this rank's rows of the fused projection output, not yet rotated), pos int32 [T_loc],
        cu_seqlens int32 [n+1] over the GLOBAL stream (all boundaries multiples of 128). Returns [T_loc, Hq*128]."""
        scale = scale if scale is not None else 1.0 / math.sqrt(128)
        lo = self.kv_tile_lo(cu_seqlens, cu_cpu)
        if torch.is_grad_enabled() and qkv.requires_grad:
            return _CPAttn.apply(qkv, pos, table, cu_seqlens, self, lo, scale)[0]
        return _cp_forward(self, qkv.detach(), pos, table, cu_seqlens, lo, scale)[0]


def _cp_forward(cp: CPContext, qkv, pos, table, cu, lo, scale):
    from ..ops.functional import _rope_inplace

    T_loc, W = qkv.shape
    assert T_loc == cp.T_loc and W == cp.W and qkv.is_contiguous()
    Hq, Hkv = cp.Hq, cp.Hkv
    _rope_inplace(qkv, pos, table, Hq + Hkv, 128, 1.0)
    buf = cp.qkv[cp.parity]
    ptrs = cp.qkv_ptrs[cp.parity]
    cp.parity ^= 1
    buf.view(T_loc, W).copy_(qkv)
    cp.barrier()                       # every rank's rows are in place (and the previous use of this buffer is over)
    cp.flag_epoch += 1
    n_seqs = cu.numel() - 1
    rows = 128 if (Hq // Hkv) % 2 == 0 else 256
    tile_seq, tile_q0, n = _query_tiles_cached(cu, cp.T_total, n_seqs, rows)
    kv_g = torch.empty(cp.T_total, cp.kv_cols, dtype=torch.bfloat16, device=qkv.device)
    out = torch.empty(T_loc, Hq * 128, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(Hq, T_loc, dtype=torch.float32, device=qkv.device)
    rc = _lib.lib().b200_attn_fwd_cp(
        _lib.ptr(qkv), ptrs, ctypes.c_int(cp.world), ctypes.c_int(cp.rank), ctypes.c_int(T_loc), _lib.ptr(kv_g),
        _lib.ptr(cp.flags), ctypes.c_int(cp.flag_epoch), ctypes.c_int(lo), ctypes.c_int(cp.n_copy_y), _lib.ptr(cu),
        _lib.ptr(tile_seq), _lib.ptr(tile_q0), ctypes.c_int(n), ctypes.c_int(rows), _lib.ptr(out), _lib.ptr(lse),
        ctypes.c_int(n_seqs), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_float(scale),
        _lib.ptr(_lib.status_word(qkv.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "attn_fwd_cp")
    return out, lse, kv_g


class _CPAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, table, cu, cp: CPContext, lo: int, scale: float):
        if qkv._is_view() or qkv.is_leaf or not qkv.is_contiguous():
            qkv = qkv.clone()
        else:
            ctx.mark_dirty(qkv)
        out, lse, kv_g = _cp_forward(cp, qkv, pos, table, cu, lo, scale)
        ctx.save_for_backward(qkv, out, lse, kv_g, cu, pos, table)
        ctx.cp, ctx.lo, ctx.scale = cp, lo, scale
        return out, qkv

    @staticmethod
    def backward(ctx, dout, _unused):
        qkv, out, lse, kv_g, cu, pos, table = ctx.saved_tensors
        cp: CPContext = ctx.cp
        L = _lib.lib()
        T_loc, Hq, Hkv = cp.T_loc, cp.Hq, cp.Hkv
        dout = dout if (dout.stride(1) == 1 and dout.stride(0) % 8 == 0) else dout.contiguous()
        n_seqs = cu.numel() - 1
        tile_seq, tile_k0, n = _query_tiles_cached(cu, cp.T_total, n_seqs, 128)
        delta = torch.empty(Hq, T_loc, dtype=torch.float32, device=qkv.device)
        acc = torch.empty(T_loc, cp.W, dtype=torch.float32, device=qkv.device)
        dqkv = torch.empty(T_loc, cp.W, dtype=torch.bfloat16, device=qkv.device)
        st = _lib.ptr(_lib.status_word(qkv.device))
        cp.barrier()                   # peers are done reading my dk/dv partials of the previous layer
        rc = L.b200_attn_bwd_cp(
            _lib.ptr(qkv), _lib.ptr(kv_g), ctypes.c_int(cp.world), ctypes.c_int(cp.rank), ctypes.c_int(T_loc),
            ctypes.c_int(ctx.lo), _lib.ptr(out), _lib.ptr(dout), ctypes.c_int(dout.stride(0)), _lib.ptr(lse),
            _lib.ptr(cu), _lib.ptr(tile_seq), _lib.ptr(tile_k0), ctypes.c_int(n), _lib.ptr(delta), _lib.ptr(acc),
            _lib.ptr(cp.dkv_g), ctypes.c_int(n_seqs), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_float(ctx.scale),
            st, _lib.stream_ptr())
        _lib.check_rc(rc, "attn_bwd_cp")
        cp.barrier()                   # every rank's partial sums are complete
        rc = L.b200_cp_dkv_reduce(cp.dkv_ptrs, ctypes.c_int(cp.world), ctypes.c_int(cp.rank), ctypes.c_int(T_loc),
                                  ctypes.c_int(cp.kv_cols), _lib.ptr(acc), ctypes.c_int(cp.W), ctypes.c_int(Hq * 128),
                                  _lib.stream_ptr())
        _lib.check_rc(rc, "cp_dkv_reduce")
        rc = L.b200_attn_bwd_finalize(_lib.ptr(acc), _lib.ptr(dqkv), _lib.ptr(pos), _lib.ptr(table),
                                      ctypes.c_int(table.shape[0]), ctypes.c_int(T_loc), ctypes.c_int(Hq),
                                      ctypes.c_int(Hkv), _lib.stream_ptr())
        _lib.check_rc(rc, "attn_bwd_finalize")
        return dqkv, None, None, None, None, None, None


class _GatherTokens(torch.autograd.Function):
    """All-gather of a per-token vector across the context-parallel group. Every rank then computes the same loss on
    the gathered vector, so the sum over ranks of the slice gradients (what an autograd-aware all-gather would
    reduce-scatter; openrlhf/models/ring_attn_utils.py:177-181) is ``size`` times the local slice gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = torch.empty(world * x.numel(), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        world, rank = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        n = g.numel() // world
        return g[rank * n:(rank + 1) * n] * world, None


class ContextParallel:
    """Model-level glue: takes the packed batch every rank of the group holds, re-packs it with 128-aligned documents,
    runs this rank's rows through the model with context-parallel attention and returns per-token results in the
    original packed order (Actor.forward_packed calls forward_logprobs)."""

    def __init__(self, group):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._ctx: dict = {}

    def _context(self, T_loc, cfg, device) -> CPContext:
        key = (T_loc, cfg.num_attention_heads, cfg.num_key_value_heads)
        c = self._ctx.get(key)
        if c is None:
            if len(self._ctx) >= 2:       # symmetric buffers are sized per chunk length: keep only recent shapes
                self._ctx.clear()
            c = CPContext(self.group, T_loc, cfg.num_attention_heads, cfg.num_key_value_heads, device)
            self._ctx[key] = c
        return c

    def _run(self, model, pb):
        """This rank's rows through the decoder stack; returns (hidden [T_loc, H], aux, local labels, index that maps
        the gathered context-parallel stream back to pb's packed order)."""
        from ..models.packing import cp_slice, pack_lists_cp

        cu = pb.cu_seqlens.tolist()
        seqs = [pb.input_ids[a:b] for a, b in zip(cu[:-1], cu[1:])]
        pb_cp, _ = pack_lists_cp(seqs, self.size, device=pb.input_ids.device)
        ids, labels, pos = cp_slice(pb_cp, self.rank, self.size)
        ctx = self._context(ids.numel(), model.cfg, ids.device)
        model.cp = ctx
        try:
            h, aux = model(ids, pos, pb_cp.cu_seqlens, pb_cp.max_seqlen)
        finally:
            model.cp = None
        cu_cp = pb_cp.cu_seqlens.tolist()
        idx = torch.cat([torch.arange(b - a) + c for a, b, c in zip(cu[:-1], cu[1:], cu_cp[:-1])]).to(ids.device)
        return h, aux, labels, idx

    def forward_values(self, model, pb):
        """Per-token values of a reward / critic model over the packed batch (context-parallel attention)."""
        h, aux, _, idx = self._run(model, pb)
        v = model.values(h)
        return _GatherTokens.apply(v, self.group)[idx], aux

    def forward_logprobs(self, model, pb, temperature: float = 1.0, return_entropy: bool = False):
        from ..models.packing import cp_slice, pack_lists_cp

        cu = pb.cu_seqlens.tolist()
        seqs = [pb.input_ids[a:b] for a, b in zip(cu[:-1], cu[1:])]
        pb_cp, _ = pack_lists_cp(seqs, self.size, device=pb.input_ids.device)
        ids, labels, pos = cp_slice(pb_cp, self.rank, self.size)
        ctx = self._context(ids.numel(), model.cfg, ids.device)
        model.cp = ctx
        try:
            h, aux = model(ids, pos, pb_cp.cu_seqlens, pb_cp.max_seqlen)
        finally:
            model.cp = None
        logp, ent = model.logprobs(h, labels, temperature, return_entropy)
        cu_cp = pb_cp.cu_seqlens.tolist()
        idx = torch.cat([torch.arange(b - a) + c for a, b, c in zip(cu[:-1], cu[1:], cu_cp[:-1])]).to(ids.device)
        logp = _GatherTokens.apply(logp, self.group)[idx]
        if ent is not None:
            ent = _GatherTokens.apply(ent, self.group)[idx]
        return logp, ent, aux
