"""Symmetric (peer-mapped) buffers and the fused NVLink optimizer step built on them.

``SymmBuffers`` allocates the bf16 parameter buffer, the fp32 gradient buffer and a small flag pad in symmetric
memory (``torch.distributed._symmetric_memory``: every rank can address every peer's copy, and an NVSwitch multicast
address exists when the fabric supports it). ``step`` then runs the whole ZeRO optimizer step as three launches of
this repository's kernels instead of NCCL reduce-scatter + FusedAdam + all-gather:

    barrier (all backward passes done)
    zero_reduce        pull my shard of every peer's gradients, sum, scale, write locally, partial grad-norm
    all-reduce of one float (grad norm^2)       <- the only NCCL call, 4 bytes
    clip coefficient on device
    zero_adam_gather   AdamW on my master shard, bf16 result stored into every peer's parameter buffer
    barrier (all parameter stores landed)
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])
    return arr


class SymmBuffers:
    def __init__(self, group, padded_numel: int, device, use_nvls: bool | None = None, with_grad: bool = True):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.padded = padded_numel
        self.param = symm_mem.empty(padded_numel, dtype=torch.bfloat16, device=self.device)
        self.param.zero_()
        self._hp = symm_mem.rendezvous(self.param, self.group)
        self.grad = None
        self._hg = None
        if with_grad:
            self.grad = symm_mem.empty(padded_numel, dtype=torch.float32, device=self.device)
            self.grad.zero_()
            self._hg = symm_mem.rendezvous(self.grad, self.group)
        self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self._hs = symm_mem.rendezvous(self.pad, self.group)
        self.param_ptrs = _ptr_array(self._hp.buffer_ptrs)
        self.grad_ptrs = _ptr_array(self._hg.buffer_ptrs) if self._hg is not None else None
        self.pad_ptrs = _ptr_array(self._hs.buffer_ptrs)
        if use_nvls is None:
            use_nvls = os.environ.get("OPENRLHF_B200_NVLS", "0") == "1"
        self.mc_param = self.mc_grad = 0
        if use_nvls and int(getattr(self._hp, 'multicast_ptr', 0) or 0) != 0:
            self.mc_param = int(self._hp.multicast_ptr)
            self.mc_grad = int(self._hg.multicast_ptr) if self._hg is not None else 0
        self.epoch = 0
        self.wait_limit_s = float(os.environ.get("OPENRLHF_B200_WAIT_LIMIT_S", "60"))
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self, channel: int = 0):
        """Device-side barrier across the group on the current stream; a peer that never arrives produces a
        KernelError at the next status check instead of a hang."""
        self.epoch += 1
        st = _lib.status_word(self.device)
        rc = _lib.lib().b200_symm_barrier(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                          ctypes.c_int(channel), ctypes.c_uint(self.epoch),
                                          ctypes.c_double(self.wait_limit_s), _lib.ptr(st), _lib.stream_ptr())
        _lib.check_rc(rc, "symm_barrier")

    @torch.no_grad()
    def step(self, eng, lr: float, grad_scale: float):
        L = _lib.lib()
        lo, n = eng.lo, eng.shard_size
        if getattr(eng, "_reduced", None) is None:
            eng._reduced = torch.empty(n, dtype=torch.float32, device=self.device)
        eng.scalars.zero_()
        # ranks reach the optimizer step with whatever skew generation and the backward passes left them; a 4-byte NCCL
        # all-reduce absorbs it (NCCL waits without a deadline of its own), so that the bounded device-side barrier
        # below only ever sees microseconds of skew and its limit can stay a failure detector
        if getattr(self, "_skew", None) is None:
            self._skew = torch.zeros(1, dtype=torch.float32, device=self.device)
        dist.all_reduce(self._skew, group=self.group)
        self.barrier(0)
        rc = L.b200_zero_reduce(self.grad_ptrs, ctypes.c_void_p(self.mc_grad), ctypes.c_int(self.world),
                                ctypes.c_longlong(lo), ctypes.c_longlong(n), ctypes.c_float(1.0 / self.world),
                                _lib.ptr(eng._reduced), _lib.ptr(eng.scalars), ctypes.c_int(0), _lib.stream_ptr())
        _lib.check_rc(rc, "zero_reduce")
        dist.all_reduce(eng.scalars[:1], group=self.group)
        _lib.check_rc(L.b200_clip_coef(_lib.ptr(eng.scalars), ctypes.c_float(eng.max_norm or 0.0),
                                       ctypes.c_float(grad_scale), _lib.stream_ptr()), "clip_coef")
        mask = eng.decay_mask
        rc = L.b200_zero_adam_gather(_lib.ptr(eng.master), _lib.ptr(eng.exp_avg), _lib.ptr(eng.exp_avg_sq),
                                     _lib.ptr(eng._reduced), self.param_ptrs, ctypes.c_void_p(self.mc_param),
                                     ctypes.c_int(self.world), ctypes.c_longlong(lo), ctypes.c_longlong(n),
                                     _lib.ptr(eng.scalars), ctypes.c_float(lr), ctypes.c_float(eng.betas[0]),
                                     ctypes.c_float(eng.betas[1]), ctypes.c_float(eng.eps), ctypes.c_float(eng.wd),
                                     ctypes.c_int(eng.opt_step),
                                     _lib.ptr(mask.view(torch.uint8)) if mask is not None else None, ctypes.c_int(0),
                                     _lib.stream_ptr())
        _lib.check_rc(rc, "zero_adam_gather")
        self.grad.zero_()          # safe: every peer finished reading it before the all-reduce above completed
        self.barrier(1)
        eng.last_grad_norm = eng.scalars[1]
