"""Expert parallelism for mixture-of-experts layers over NVLink peer memory.

The experts are cut into ``world`` contiguous ranges (rank r owns experts [r*E_loc, (r+1)*E_loc)). One MoE layer is

    route (local)  ->  all-gather of the per-expert counts (E ints per rank, the only NCCL call)
    dispatch   : every routed token row is stored straight into its expert owner's receive buffer at its final,
                 expert-sorted and 128-row-padded position (peer stores; positions follow from the count matrix, so no
                 second exchange and no re-sort on the receiver)
    experts    : grouped tcgen05 GEMMs over the receive buffer (gate_up -> SwiGLU -> down)
    combine    : every token pulls its k expert outputs back from the owners' output buffers and adds them with its
                 routing weights (peer loads, fixed order: deterministic)

with device-side barriers between the phases; the backward pass mirrors it (scaled scatter of dy, grouped input /
weight gradients, pull of dx). The reference has no expert parallelism: HF's expert loop / grouped_mm runs under
ZeRO-3 on every rank (openrlhf/models/actor.py:95-110 only marks the MoE block as a ZeRO-3 leaf).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import gemm_grouped_rows, gemm_grouped_wgrad
from .symm import _ptr_array


class EPContext:
    def __init__(self, group, max_tokens: int, top_k: int, hidden: int, num_experts: int, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        assert num_experts % self.world == 0
        self.E, self.E_loc, self.k, self.H = num_experts, num_experts // self.world, top_k, hidden
        self.device = torch.device(device)
        # worst case: every routed row of every rank lands on one rank, plus 127 padding rows per local expert
        self.cap = (self.world * max_tokens * top_k + self.E_loc * 127 + 127) // 128 * 128
        self.max_tokens = max_tokens

        def buf():
            t = symm_mem.empty(self.cap * hidden, dtype=torch.bfloat16, device=self.device)
            h = symm_mem.rendezvous(t, self.group)
            return t.view(self.cap, hidden), _ptr_array(h.buffer_ptrs), h

        self.recv, self.recv_ptrs, self._h0 = buf()      # dispatched activations (forward) / pulled dx source (backward)
        self.outb, self.out_ptrs, self._h1 = buf()       # expert outputs (forward) / dispatched dy (backward)
        self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self._hs = symm_mem.rendezvous(self.pad, self.group)
        self.pad_ptrs = _ptr_array(self._hs.buffer_ptrs)
        self.bar_epoch = 0
        self.wait_limit_s = float(os.environ.get("OPENRLHF_B200_WAIT_LIMIT_S", "60"))
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self):
        self.bar_epoch += 1
        rc = _lib.lib().b200_symm_barrier(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                          ctypes.c_int(0), ctypes.c_uint(self.bar_epoch),
                                          ctypes.c_double(self.wait_limit_s), _lib.ptr(_lib.status_word(self.device)),
                                          _lib.stream_ptr())
        _lib.check_rc(rc, "symm_barrier")

    # ------------------------------------------------------------------------------------------------ routing plan
    def plan(self, idx: torch.Tensor):
        """idx int64 [T, k] (global expert ids). Returns (dest_rank int32 [T*k], dest_row int32 [T*k], tile_group int32
        [cap/128], offsets int32 [E_loc+1]) - everything on the device, no host read."""
        T, k = idx.shape
        E, E_loc, W = self.E, self.E_loc, self.world
        flat_e = idx.reshape(-1)
        counts = torch.zeros(E, dtype=torch.long, device=idx.device).scatter_add_(
            0, flat_e, torch.ones_like(flat_e)).to(torch.int32)
        allc = torch.empty(W, E, dtype=torch.int32, device=idx.device)
        dist.all_gather_into_tensor(allc, counts, group=self.group)
        allc = allc.long()
        tot = allc.sum(0)                                        # rows per expert over all sources
        padded = (tot + 127) // 128 * 128
        padded_r = padded.view(W, E_loc)
        ends_r = torch.cumsum(padded_r, 1)                       # per owner rank: padded end of each local expert
        starts = (ends_r - padded_r).reshape(-1)                 # [E] start row inside the owner's buffer
        before_me = allc[: self.rank].sum(0)                     # rows of earlier source ranks, per expert
        order = torch.argsort(flat_e, stable=True)
        sorted_e = flat_e[order]
        dense_starts = torch.cumsum(counts.long(), 0) - counts.long()
        rank_in_e = torch.arange(T * k, device=idx.device) - dense_starts[sorted_e]
        row_sorted = starts[sorted_e] + before_me[sorted_e] + rank_in_e
        dest_row = torch.empty(T * k, dtype=torch.int32, device=idx.device)
        dest_row[order] = row_sorted.to(torch.int32)
        dest_rank = (flat_e // E_loc).to(torch.int32)
        my_ends = ends_r[self.rank]
        tiles = torch.arange(self.cap // 128, device=idx.device) * 128
        tg = torch.searchsorted(my_ends, tiles, right=True)
        tile_group = torch.where(tg < E_loc, tg, torch.full_like(tg, -1)).to(torch.int32)
        offsets = torch.cat([my_ends[:1] * 0, my_ends]).to(torch.int32)
        return dest_rank, dest_row, tile_group, offsets

    def moe(self, x, weights, idx, gate_up_local, down_local):
        """x [T, H] bf16, weights fp32 [T, k] (routing weights, differentiable), idx int64 [T, k], gate_up_local
        [E_loc, 2I, H], down_local [E_loc, H, I]: this rank's experts. Returns y [T, H]."""
        assert x.shape[0] <= self.max_tokens and x.shape[1] == self.H and idx.shape[1] == self.k
        dest_rank, dest_row, tile_group, offsets = self.plan(idx)
        return _EPMoE.apply(x, weights, gate_up_local, down_local, self, dest_rank, dest_row, tile_group, offsets)


def _scatter(ep: EPContext, x, dest_rank, dest_row, scale, ptrs):
    rc = _lib.lib().b200_ep_scatter(_lib.ptr(x), _lib.ptr(dest_rank), _lib.ptr(dest_row), _lib.ptr(scale), ptrs,
                                    ctypes.c_int(ep.world), ctypes.c_int(dest_rank.numel()), ctypes.c_int(ep.k),
                                    ctypes.c_int(ep.H), _lib.stream_ptr())
    _lib.check_rc(rc, "ep_scatter")


def _gather(ep: EPContext, ptrs, dest_rank, dest_row, w, out, rows_out, dy, dots, T):
    rc = _lib.lib().b200_ep_gather(ptrs, ctypes.c_int(ep.world), _lib.ptr(dest_rank), _lib.ptr(dest_row), _lib.ptr(w),
                                   _lib.ptr(out), _lib.ptr(rows_out), _lib.ptr(dy), _lib.ptr(dots), ctypes.c_int(T),
                                   ctypes.c_int(ep.k), ctypes.c_int(ep.H), _lib.stream_ptr())
    _lib.check_rc(rc, "ep_gather")


class _EPMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, gate_up, down, ep: EPContext, dest_rank, dest_row, tile_group, offsets):
        L = _lib.lib()
        T, H = x.shape
        x = x.contiguous()
        wflat = weights.reshape(-1).float().contiguous()
        ep.recv.zero_()
        ep.barrier()                                   # every receive buffer is cleared (and its last readers are done)
        _scatter(ep, x, dest_rank, dest_row, None, ep.recv_ptrs)
        ep.barrier()                                   # all rows have landed
        gu = gemm_grouped_rows(ep.recv, gate_up.detach(), tile_group)
        a = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=gu.dtype, device=gu.device)
        _lib.check_rc(L.b200_swiglu_fwd(_lib.ptr(gu), _lib.ptr(a), ctypes.c_longlong(gu.shape[0]),
                                        ctypes.c_int(gu.shape[1] // 2), _lib.stream_ptr()), "swiglu_fwd")
        gemm_grouped_rows(a, down.detach(), tile_group, out=ep.outb)
        ep.barrier()                                   # expert outputs are complete everywhere
        y = torch.empty_like(x)
        rows = torch.empty(T * ep.k, H, dtype=x.dtype, device=x.device)
        _gather(ep, ep.out_ptrs, dest_rank, dest_row, wflat, y, rows, None, None, T)
        ctx.save_for_backward(ep.recv.clone(), gu, a, rows, wflat, dest_rank, dest_row, tile_group, offsets)
        ctx.ep, ctx.gate_up, ctx.down, ctx.wshape = ep, gate_up, down, weights.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        L = _lib.lib()
        recv, gu, a, rows, wflat, dest_rank, dest_row, tile_group, offsets = ctx.saved_tensors
        ep: EPContext = ctx.ep
        gate_up, down = ctx.gate_up, ctx.down
        dy = dy.contiguous()
        T, H = dy.shape
        # gradient of the routing weights: <dy[t], expert output row> (the rows were pulled in the forward pass)
        dw = torch.einsum("tkh,th->tk", rows.view(T, ep.k, H).float(), dy.float())
        ep.outb.zero_()
        ep.barrier()
        _scatter(ep, dy, dest_rank, dest_row, wflat, ep.out_ptrs)          # d(expert output rows) = w * dy
        ep.barrier()
        d_a = gemm_grouped_rows(ep.outb, down.detach(), tile_group, b_mn=True)
        g_dn = _acc_wgrad(down, ep.outb, a, offsets)
        d_gu = torch.empty_like(gu)
        _lib.check_rc(L.b200_swiglu_bwd(_lib.ptr(gu), _lib.ptr(d_a), _lib.ptr(d_gu), ctypes.c_longlong(gu.shape[0]),
                                        ctypes.c_int(gu.shape[1] // 2), _lib.stream_ptr()), "swiglu_bwd")
        gemm_grouped_rows(d_gu, gate_up.detach(), tile_group, b_mn=True, out=ep.recv)
        g_gu = _acc_wgrad(gate_up, d_gu, recv, offsets)
        ep.barrier()                                   # every rank's d(receive buffer) is complete
        dx = torch.empty_like(dy)
        _gather(ep, ep.recv_ptrs, dest_rank, dest_row, None, dx, None, None, None, T)
        ep.barrier()                                   # pulls are done before anyone clears the buffers again
        return dx, dw.view(ctx.wshape), g_gu, g_dn, None, None, None, None, None


def _acc_wgrad(W, dy, x, offsets):
    """W.main_grad += per-expert dy^T x when the ZeRO engine owns a gradient buffer (returns None), else returns the
    dense gradient for autograd."""
    mg = getattr(W, "main_grad", None)
    if mg is not None:
        gemm_grouped_wgrad(dy, x, offsets, mg, accumulate=True)
        return None
    dW = torch.zeros(W.shape, dtype=torch.float32, device=W.device)
    gemm_grouped_wgrad(dy, x, offsets, dW, accumulate=False)
    return dW.to(W.dtype)
