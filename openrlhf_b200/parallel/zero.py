"""ZeRO-style training engine over the model's flat parameter buffer.

Takes the place of the DeepSpeed engine the reference builds in ``DeepspeedStrategy.prepare``
(openrlhf/utils/deepspeed/deepspeed.py:295-429: ZeRO stage, AdamW, bf16 with fp32 master weights, gradient clipping
by global norm, HF LR schedule). Layout:

* bf16 parameters: ``model.flat`` (every rank holds the full buffer during compute);
* fp32 gradients: one flat buffer of the same layout; each parameter's ``main_grad`` is a view into it, so wgrad
  GEMMs accumulate micro-batches in fp32 in their epilogue;
* fp32 master weights and Adam moments: only this rank's contiguous shard ``[lo, hi)`` of the flat index space.

``step()`` = gradient reduce-scatter -> global grad norm -> clip coefficient (device scalar, no host sync) -> fused
AdamW on the shard writing the bf16 parameters -> parameter all-gather. With more than one rank the reduce-scatter,
the update and the all-gather run as peer-memory kernels over NVLink (``parallel/symm.py``); NCCL is the fallback
and the baseline they are tested against.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.distributed as dist

from ..ops import _lib


def cosine_with_min_lr(step: int, total: int, warmup: int, min_ratio: float) -> float:
    """HF ``cosine_with_min_lr``: linear warm-up, then 0.5(1+cos(pi*progress))(1-r)+r."""
    if step < warmup:
        return float(step) / float(max(1, warmup))
    progress = float(step - warmup) / float(max(1, total - warmup))
    f = 0.5 * (1.0 + math.cos(math.pi * min(progress, 1.0)))
    return f * (1 - min_ratio) + min_ratio


class LRScheduler:
    def __init__(self, base_lr: float, total_steps: int, warmup_ratio: float = 0.03, min_lr_ratio: float = 0.1,
                 kind: str = "cosine_with_min_lr"):
        self.base_lr, self.total, self.kind = base_lr, max(1, total_steps), kind
        self.warmup = math.ceil(warmup_ratio * self.total)
        self.min_ratio = min_lr_ratio
        self.step_idx = 0

    def get_lr(self) -> float:
        if self.kind == "constant":
            return self.base_lr
        if self.kind == "constant_with_warmup":
            return self.base_lr * min(1.0, self.step_idx / max(1, self.warmup))
        if self.kind == "linear":
            if self.step_idx < self.warmup:
                return self.base_lr * self.step_idx / max(1, self.warmup)
            return self.base_lr * max(0.0, (self.total - self.step_idx) / max(1, self.total - self.warmup))
        return self.base_lr * cosine_with_min_lr(self.step_idx, self.total, self.warmup, self.min_ratio)

    def get_last_lr(self):
        return [self.get_lr()]

    def step(self):
        self.step_idx += 1

    def state_dict(self):
        return {"step_idx": self.step_idx}

    def load_state_dict(self, d):
        self.step_idx = int(d["step_idx"])


class ZeroEngine:
    def __init__(self, model, lr: float = 1e-6, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_norm: float = 1.0, zero_stage: int = 2, group=None, scheduler: LRScheduler | None = None,
                 train: bool = True, use_symm: bool | None = None, symm=None, adam_offload: bool = False):
        """use_symm: run the multi-rank optimizer step with the peer-memory kernels of ``parallel/symm.py``. None picks
        them whenever they apply (CUDA, more than one rank, all ranks on this node, no tensor-parallel shard); the
        model's flat buffer is then moved into symmetric memory and every parameter re-bound to it, so build the
        engine before anything that keeps views of the parameters. ``OPENRLHF_B200_SYMM=0`` selects NCCL.
        adam_offload: keep master weights and moments in pinned host memory between optimizer steps
        (``--ds.adam_offload``, openrlhf/utils/deepspeed/deepspeed_utils.py:24-28)."""
        self.model = model
        self.adam_offload = bool(adam_offload) and train
        self.flat = model.flat
        self.device = self.flat.device
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.zero_stage = zero_stage
        self.lr, self.betas, self.eps, self.wd, self.max_norm = lr, betas, eps, weight_decay, max_norm
        self.scheduler = scheduler
        self.opt_step = 0
        self.micro_steps = 0
        self.last_grad_norm = None
        self.trainable = train
        n = model.total_numel
        # shard boundaries on 256-element multiples so every shard starts 16-byte aligned in every dtype
        per = ((n + self.world - 1) // self.world + 255) // 256 * 256
        self.shard_size = per
        self.padded = per * self.world
        if self.flat.numel() < self.padded:
            raise ValueError("model.flat must be allocated with room for shard padding; use alloc_flat()")
        self.lo = per * self.rank if zero_stage >= 1 else 0
        self.hi = self.lo + per if zero_stage >= 1 else self.padded
        self.symm = None
        # tensor-parallel shard (parallel/tp_train.py): replicated parameters are averaged over the TP group before
        # the step and count once in the clipping norm
        self.tp = getattr(model, "tp_train", None)
        self.tp_rep_mask = None
        if not train:
            return
        if self.tp is not None:
            assert symm is None, "the peer-memory optimizer step is not combined with tensor-parallel training"
            self.tp_rep_mask = self.tp.replicated_mask(model, self.lo, self.hi, self.device)
        on_gpu = self.flat.is_cuda
        self.symm = symm if (symm is not None and on_gpu and self.world > 1) else None
        if self.symm is None and self._want_symm(use_symm, on_gpu):
            self.symm = self._move_to_symmetric_memory()
        if self.symm is not None:
            assert self.symm.param.data_ptr() == self.flat.data_ptr(), "the model must be built on symm.param"
            self.grad_flat = self.symm.grad
        else:
            self.grad_flat = torch.zeros(self.padded, dtype=torch.float32, device=self.device)
        for s, p in model.named_specs():
            p.main_grad = self.grad_flat[s.offset:s.offset + s.numel].view(s.shape)
        sl = slice(self.lo, self.hi)
        self.master = self.flat[sl].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.scalars = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.decay_mask = None
        if weight_decay != 0.0:
            mask = torch.zeros(self.padded, dtype=torch.bool, device=self.device)
            for s in model.specs:
                if s.decay and model.p(s.name).requires_grad:      # frozen parameters (no gradient) must not decay
                    mask[s.offset:s.offset + s.numel] = True
            self.decay_mask = mask[sl].clone()
        if self.adam_offload:
            self.offload_states()

    # ------------------------------------------------------------------ allocation helpers
    def _want_symm(self, use_symm, on_gpu: bool) -> bool:
        import os

        if not on_gpu or self.world == 1 or self.tp is not None or self.zero_stage < 1:
            if use_symm:
                raise ValueError("the peer-memory optimizer step needs CUDA, more than one rank, ZeRO stage >= 1 and no "
                                 "tensor-parallel shard")
            return False
        if use_symm is None:
            local = int(os.environ.get("LOCAL_WORLD_SIZE", dist.get_world_size()))
            use_symm = os.environ.get("OPENRLHF_B200_SYMM", "1") == "1" and local >= dist.get_world_size()
        return bool(use_symm)

    def _move_to_symmetric_memory(self):
        """Re-home the flat parameter buffer in symmetric memory (peers can then address it) and re-bind the views."""
        from .symm import SymmBuffers

        symm = SymmBuffers(self.group, self.padded, self.device)
        n = min(self.flat.numel(), self.padded)
        symm.param[:n].copy_(self.flat[:n])
        for s_, p in self.model.named_specs():
            p.data = symm.param[s_.offset:s_.offset + s_.numel].view(s_.shape)
        self.model.flat = symm.param
        self.flat = symm.param
        return symm

    @staticmethod
    def padded_numel(total_numel: int, world: int) -> int:
        per = ((total_numel + world - 1) // world + 255) // 256 * 256
        return per * world

    # ------------------------------------------------------------------ training API
    def backward(self, loss: torch.Tensor):
        loss.backward()
        self.micro_steps += 1
        # gradients that arrived through plain autograd (CPU restatements, small torch ops such as the value head)
        # are folded into the fp32 flat buffer next to the ones the kernels accumulated there directly
        with torch.no_grad():
            for _, p in self.model.named_specs():
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None

    def zero_grad(self):
        self.grad_flat.zero_()

    def current_lr(self) -> float:
        return self.scheduler.get_lr() if self.scheduler is not None else self.lr

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        """One optimizer step. `grad_scale` multiplies the accumulated gradient (1 / accumulation steps)."""
        self.opt_step += 1
        lr = self.current_lr()
        if self.adam_offload:
            self.reload_states()
        if self.tp is not None:
            self.tp.sync_replicated_grads(self.model)
        if self.symm is not None:
            self.symm.step(self, lr, grad_scale)
        elif self.flat.is_cuda:
            self._step_cuda(lr, grad_scale)
        else:
            self._step_reference(lr, grad_scale)
        if self.scheduler is not None:
            self.scheduler.step()
        if self.adam_offload:
            self.offload_states()

    def _reduce_grads(self) -> torch.Tensor:
        """Mean of gradients over data-parallel ranks; returns this rank's fp32 shard."""
        if self.world == 1:
            return self.grad_flat[self.lo:self.hi]
        if self.zero_stage >= 1:
            out = torch.empty(self.shard_size, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(out, self.grad_flat, op=dist.ReduceOp.AVG if self.flat.is_cuda else dist.ReduceOp.SUM,
                                       group=self.group)
            if not self.flat.is_cuda:
                out /= self.world
            return out
        dist.all_reduce(self.grad_flat, group=self.group)
        self.grad_flat /= self.world
        return self.grad_flat

    def _tp_norm_fix(self, g: torch.Tensor, sq: torch.Tensor):
        """sq holds sum(g^2) of this rank's slice; the TP-wide sum that follows would count replicated parameters
        tp times: keep 1/tp of their share here."""
        mask = self.tp_rep_mask if g.numel() == self.tp_rep_mask.numel() else \
            self.tp.replicated_mask(self.model, 0, g.numel(), g.device)
        rep = (torch.where(mask, g, torch.zeros((), dtype=g.dtype, device=g.device)).double() ** 2).sum().float()
        sq -= rep * (1.0 - 1.0 / self.tp.size)

    def _gather_params(self):
        if self.world > 1 and self.zero_stage >= 1:
            dist.all_gather_into_tensor(self.flat[: self.padded], self.flat[self.lo:self.hi].clone(), group=self.group)

    def _step_cuda(self, lr, grad_scale):
        L = _lib.lib()
        g = self._reduce_grads()
        n = g.numel()
        st = _lib.stream_ptr()
        self.scalars.zero_()
        _lib.check_rc(L.b200_sumsq(_lib.ptr(g), ctypes.c_longlong(n), _lib.ptr(self.scalars), st), "sumsq")
        if self.tp is not None:
            self._tp_norm_fix(g, self.scalars[:1])
        if self.world > 1 and self.zero_stage >= 1:
            dist.all_reduce(self.scalars[:1], group=self.group)
        if self.tp is not None:
            dist.all_reduce(self.scalars[:1], group=self.tp.group)
        _lib.check_rc(L.b200_clip_coef(_lib.ptr(self.scalars), ctypes.c_float(self.max_norm or 0.0),
                                       ctypes.c_float(grad_scale), st), "clip_coef")
        self._adam_cuda(g, lr, zero_grad=self.world == 1)
        self.last_grad_norm = self.scalars[1]
        if self.world > 1:
            self.grad_flat.zero_()
            self._gather_params()

    def _adam_cuda(self, g, lr, zero_grad):
        L = _lib.lib()
        n = g.numel()
        pbf = self.flat[self.lo:self.hi]
        scale_ptr = ctypes.c_void_p(self.scalars.data_ptr() + 8)
        if self.decay_mask is None:
            _lib.check_rc(L.b200_adamw(_lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq),
                                       _lib.ptr(g), _lib.ptr(pbf), ctypes.c_longlong(n), scale_ptr, ctypes.c_float(lr),
                                       ctypes.c_float(self.betas[0]), ctypes.c_float(self.betas[1]),
                                       ctypes.c_float(self.eps), ctypes.c_float(0.0), ctypes.c_int(self.opt_step),
                                       ctypes.c_int(int(zero_grad)), _lib.stream_ptr()), "adamw")
        else:
            # decoupled weight decay only on matrices: pre-scale the masked master weights, then plain Adam
            self.master.mul_(torch.where(self.decay_mask.bool(), 1.0 - lr * self.wd, 1.0))
            _lib.check_rc(L.b200_adamw(_lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq),
                                       _lib.ptr(g), _lib.ptr(pbf), ctypes.c_longlong(n), scale_ptr, ctypes.c_float(lr),
                                       ctypes.c_float(self.betas[0]), ctypes.c_float(self.betas[1]),
                                       ctypes.c_float(self.eps), ctypes.c_float(0.0), ctypes.c_int(self.opt_step),
                                       ctypes.c_int(int(zero_grad)), _lib.stream_ptr()), "adamw")

    def _step_reference(self, lr, grad_scale):
        """PyTorch restatement (CPU ranks / gloo): same arithmetic as the kernels."""
        g = self._reduce_grads()
        sq = (g.double() ** 2).sum().float().reshape(1)
        if self.tp is not None:
            self._tp_norm_fix(g, sq)
        if self.world > 1 and self.zero_stage >= 1:
            dist.all_reduce(sq, group=self.group)
        if self.tp is not None:
            dist.all_reduce(sq, group=self.tp.group)
        norm = sq.sqrt().item() * grad_scale
        coef = 1.0
        if self.max_norm and norm > self.max_norm:
            coef = self.max_norm / (norm + 1e-6)
        self.last_grad_norm = torch.tensor(norm)
        gg = g * (coef * grad_scale)
        b1, b2 = self.betas
        self.exp_avg.mul_(b1).add_(gg, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(gg, gg, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.opt_step, 1 - b2 ** self.opt_step
        if self.decay_mask is not None:
            self.master.mul_(torch.where(self.decay_mask.bool(), 1.0 - lr * self.wd, 1.0))
        denom = (self.exp_avg_sq / bc2).sqrt_().add_(self.eps)
        self.master.addcdiv_(self.exp_avg / bc1, denom, value=-lr)
        self.flat[self.lo:self.hi].copy_(self.master.to(self.flat.dtype))
        self.grad_flat.zero_()
        self._gather_params()

    def grad_norm(self) -> float:
        return float(self.last_grad_norm) if self.last_grad_norm is not None else 0.0

    # ------------------------------------------------------------------ hybrid-engine sleep
    def offload_states(self):
        """Move optimizer shards to pinned host memory (hybrid-engine sleep: openrlhf/utils/deepspeed/deepspeed_utils.py:151-211)."""
        if not self.trainable or getattr(self, "_offloaded", False):
            return
        keep = getattr(self, "_host_bufs", None)
        if keep is None:
            keep = self._host_bufs = [torch.empty(t.shape, dtype=t.dtype, device="cpu",
                                                  pin_memory=t.is_cuda) for t in (self.master, self.exp_avg, self.exp_avg_sq)]
        for h, t in zip(keep, (self.master, self.exp_avg, self.exp_avg_sq)):
            h.copy_(t, non_blocking=False)
        self._host = keep
        self.master = self.exp_avg = self.exp_avg_sq = None
        self._offloaded = True
        if self.flat.is_cuda and not self.adam_offload:
            torch.cuda.empty_cache()

    def reload_states(self):
        if not getattr(self, "_offloaded", False):
            return
        self.master, self.exp_avg, self.exp_avg_sq = [t.to(self.device, non_blocking=True) for t in self._host]
        self._host = None
        self._offloaded = False

    # ------------------------------------------------------------------ state for checkpoints
    def shard_state(self) -> dict:
        if getattr(self, "_offloaded", False):
            m, a, b = self._host
            return {"master": m, "exp_avg": a, "exp_avg_sq": b, "lo": self.lo, "hi": self.hi,
                    "opt_step": self.opt_step, "world": self.world, "total_numel": self.model.total_numel,
                    "shard_size": self.shard_size}
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "lo": self.lo, "hi": self.hi, "opt_step": self.opt_step, "world": self.world,
                "total_numel": self.model.total_numel, "shard_size": self.shard_size}

    def load_shard_state(self, master, exp_avg, exp_avg_sq, opt_step):
        was_off = getattr(self, "_offloaded", False)
        if was_off:
            self.reload_states()
        self._load_shard_state(master, exp_avg, exp_avg_sq, opt_step)
        if was_off:
            self.offload_states()

    def _load_shard_state(self, master, exp_avg, exp_avg_sq, opt_step):
        self.master.copy_(master)
        self.exp_avg.copy_(exp_avg)
        self.exp_avg_sq.copy_(exp_avg_sq)
        self.opt_step = int(opt_step)
        self.flat[self.lo:self.hi].copy_(self.master.to(self.flat.dtype))
        self._gather_params()
