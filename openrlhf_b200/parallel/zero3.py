"""ZeRO stage 3: bf16 parameters, fp32 gradients, fp32 master weights and Adam moments are all sharded.

Layout. The model's logical flat parameter buffer (models/transformer.py) is cut into ``world`` equal contiguous
slices; rank r permanently holds only slice r of the bf16 parameters (in symmetric memory, so peers can read it), of the
fp32 gradient accumulator, of the master weights and of the Adam moments. For compute, a small working buffer replaces
the full one:

    [ resident parameters: embedding, final norm, lm_head, value head ] [ layer slot 0 ] [ layer slot 1 ]

Layer i's parameters are (permanently) views into slot i % 2 at their offsets inside the layer, so the model code and
every kernel see ordinary tensors. Before layer i runs, its parameters are pulled from their owners into the slot by
ONE copy kernel over peer memory (K-ZERO-AG: ``reshard_copy`` with a per-layer plan); a hook on the layer's output
gradient does the same before the layer's backward pass. Weight gradients accumulate in fp32 into a gradient slot of
the same shape (symmetric memory); when layer i's backward is complete, each rank pulls the part of that layer it owns
from every peer's slot, sums it and adds it to its gradient slice (K-ZERO-RS per layer, one device-side barrier per
layer). The optimizer step is then purely local: AdamW on the slice, bf16 result into the rank's parameter slice.

The reference gets this from DeepSpeed stage 3 (per-module all-gather with prefetch, reduce-scatter in buckets:
openrlhf/utils/deepspeed/deepspeed_utils.py:7-75, used by the 8B+ recipes).
CPU / gloo ranks run the same control flow with torch.distributed collectives in place of the peer-memory kernels.
"""
from __future__ import annotations

import ctypes
import os
import math

import torch
import torch.distributed as dist

from ..models.transformer import ALIGN, ParamSpec, TransformerLM
from ..ops import _lib
from .reshard import CopyEntry, ReshardPlan
from .zero import LRScheduler


# Block budget of the copy / reduction kernels that run on side streams under the compute stream's GEMMs (0: fill the
# GPU). Measured on 2 GPUs with the Qwen2.5-7B architecture, budgets of one or two blocks per SM were not faster than
# full launches (training phase 4.85 / 4.62 s against 4.55 s), so the default is 0.
OVERLAP_CTAS = int(os.environ.get("OPENRLHF_B200_OVERLAP_CTAS", "0"))
# "0": run the layer gathers and gradient reductions on the compute stream (no overlap; for measurements)
OVERLAP = os.environ.get("OPENRLHF_B200_ZERO3_OVERLAP", "1") != "0"
GRAD_SLOTS = int(os.environ.get("OPENRLHF_B200_ZERO3_GRAD_SLOTS", "4"))


def _round(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class Zero3Engine:
    def __init__(self, model: TransformerLM, lr: float = 1e-6, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_norm: float = 1.0, group=None, scheduler: LRScheduler | None = None,
                 expert_range: tuple[int, int] | None = None, train: bool = True):
        """train=False: a frozen model (reference policy, reward model). Only the bf16 parameter slice and the working
        buffer with its two layer slots exist; forward passes gather layer by layer exactly as in training (the
        reference shards its frozen models the same way with a stage-3 inference engine,
        openrlhf/utils/deepspeed/deepspeed.py:460-487)."""
        self.model = model
        self.trainable = train
        # expert parallelism: this rank only computes experts [lo, hi) of every MoE layer, so only those are gathered
        self.expert_range = expert_range
        initialised = dist.is_available() and dist.is_initialized()
        self.group = group if group is not None else (dist.group.WORLD if initialised else None)
        self.world = dist.get_world_size(self.group) if initialised else 1
        self.rank = dist.get_rank(self.group) if self.world > 1 else 0
        self.device = model.flat.device
        self.on_gpu = self.device.type == "cuda"
        self.lr, self.betas, self.eps, self.wd, self.max_norm, self.scheduler = lr, betas, eps, weight_decay, max_norm, scheduler
        self.opt_step = self.micro_steps = 0
        self.last_grad_norm = None
        cfg = model.cfg
        L = cfg.num_hidden_layers
        specs = model.specs                                      # logical layout
        total = model.total_numel
        self.per = _round((total + self.world - 1) // self.world, 256)
        self.padded = self.per * self.world
        self.lo, self.hi = self.per * self.rank, self.per * (self.rank + 1)

        # ---- groups of the logical layout
        def layer_of(name):
            return int(name.split(".")[1]) if name.startswith("layers.") else -1

        self.layer_rng = []
        for i in range(L):
            ss = [s for s in specs if layer_of(s.name) == i]
            self.layer_rng.append((ss[0].offset, _round(ss[-1].offset + ss[-1].numel, ALIGN)))
        res = [s for s in specs if layer_of(s.name) < 0]
        slot = max(b - a for a, b in self.layer_rng)
        self.res_map, off = {}, 0
        for s in res:
            self.res_map[s.name] = off
            off += _round(s.numel, ALIGN)
        self.res_size = off
        # parameter slots: two rotating ones, or one per layer when the gathered copy may stay (see _want_persist): a
        # layer is then gathered once per optimizer step (once ever for a frozen model) instead of twice per
        # micro-batch; parameters at rest stay sharded either way
        self.gslots = max(2, min(GRAD_SLOTS, L)) if train else 2
        self.pslots = L if self._want_persist(L, slot, train) else 2
        self.slot_base = [self.res_size + k * slot for k in range(self.pslots)]
        self.work_size = self.res_size + self.pslots * slot
        # gradient slots: layer i accumulates into slot i % G. More slots than parameter slots, so that a layer's
        # reduction (two cross-rank barriers around a pull over NVLink) has G - 1 layers of backward compute to finish
        # in before its slot is needed again; with two slots every rank would run in lockstep with the slowest one
        # at a granularity of one layer.
        self.gslot_base = [self.res_size + k * slot for k in range(self.gslots)]
        self.slot_width = slot
        self.gwork_size = self.res_size + self.gslots * slot

        # ---- this rank's slices (taken from the full buffer the model was built on)
        full = model.flat
        if full.numel() < self.padded:
            full = torch.cat([full, full.new_zeros(self.padded - full.numel())])
        self.symm = None
        if self.on_gpu and self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            from .symm import _ptr_array

            self.param_shard = symm_mem.empty(self.per, dtype=torch.bfloat16, device=self.device)
            self._hp = symm_mem.rendezvous(self.param_shard, self.group)
            self.param_ptrs = list(self._hp.buffer_ptrs)
            self.grad_work = self.grad_ptrs = None
            if train:
                self.grad_work = symm_mem.empty(self.gwork_size, dtype=torch.float32, device=self.device)
                self._hg = symm_mem.rendezvous(self.grad_work, self.group)
                self.grad_ptrs = list(self._hg.buffer_ptrs)
            self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
            self.pad.zero_()
            self._hs = symm_mem.rendezvous(self.pad, self.group)
            self.pad_ptrs = _ptr_array(self._hs.buffer_ptrs)
            self.bar_epochs = [0, 0]
        else:
            self.param_shard = torch.empty(self.per, dtype=full.dtype, device=self.device)
            self.grad_work = torch.zeros(self.gwork_size, dtype=torch.float32, device=self.device) if train else None
        self.param_shard.copy_(full[self.lo:self.hi])
        self.master = self.exp_avg = self.exp_avg_sq = self.grad_shard = None
        if train:
            self.grad_work.zero_()
            self.master = self.param_shard.float().clone()
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
            self.grad_shard = torch.zeros_like(self.master)
        self.scalars = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.decay_mask = None
        if train and weight_decay != 0.0:
            mask = torch.zeros(self.padded, dtype=torch.bool, device=self.device)
            for s in specs:
                if s.decay:
                    mask[s.offset:s.offset + s.numel] = True
            self.decay_mask = mask[self.lo:self.hi].clone()

        # ---- working buffer; re-bind every parameter to it and drop the full buffer
        self.work = torch.zeros(self.work_size, dtype=full.dtype, device=self.device)
        self.work_off = {}
        for s, p in model.named_specs():
            i = layer_of(s.name)
            w_off = (self.res_map[s.name] if i < 0 else
                     self.slot_base[i % self.pslots] + (s.offset - self.layer_rng[i][0]))
            self.work_off[s.name] = w_off
            p.data = self.work[w_off:w_off + s.numel].view(s.shape)
            if train:
                g_off = w_off if i < 0 else self.gslot_base[i % self.gslots] + (s.offset - self.layer_rng[i][0])
                p.main_grad = self.grad_work[g_off:g_off + s.numel].view(s.shape)
        model.flat = self.work          # the logical flat buffer no longer exists on this rank
        model.z3 = self
        del full
        self.slot_layer = [-1] * self.pslots   # which layer's parameters each slot holds (or is being filled with)
        self._inflight: dict = {}       # layer -> event of its gather on the side stream
        self._side = None
        self._plans: dict = {}
        self._tmp = torch.empty(min(self.per, _round(slot, 256)) if train else 0, dtype=torch.float32,
                                device=self.device)
        self._pending_zero = -1
        self._rs_stream = None                    # side stream of the per-layer gradient reductions
        self._slot_reduced = [None] * self.gslots  # event: the gradient slot has been reduced and cleared
        self._sync()
        self.gather_resident()

    # ------------------------------------------------------------------------------------------------ plumbing
    def _want_persist(self, L: int, slot: int, train: bool) -> bool:
        """Keep every layer's gathered parameters (one slot per layer) instead of rotating two slots? Yes when asked
        (OPENRLHF_B200_ZERO3_PERSIST=1), never with one rank or when told not to (=0); otherwise on a GPU when what is
        already allocated plus this engine's own state plus the full bf16 copy stays below 40 % of the device memory
        (the rest is for activations, the rollout engine and the other models)."""
        env = os.environ.get("OPENRLHF_B200_ZERO3_PERSIST", "auto")
        if env == "0" or self.world == 1:
            return False
        if env == "1":
            return True
        if not self.on_gpu:
            return False
        free, total = torch.cuda.mem_get_info(self.device)
        own = self.per * (18 if train else 2) + (self.res_size + max(2, min(GRAD_SLOTS, L)) * slot) * (4 if train else 0)
        return (total - free) + own + (self.res_size + L * slot) * 2 < 0.4 * total

    def _sync(self, channel: int = 0):
        """All ranks' parameter slices (or gradient slots) are in a consistent state. Barriers issued on the side
        stream of the gradient reductions use their own flag channel and epoch counter: they may execute out of order
        with the compute stream's barriers, and one channel's epochs must only ever grow."""
        if self.world == 1:
            return
        if self.on_gpu:
            self.bar_epochs[channel] += 1
            rc = _lib.lib().b200_symm_barrier(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                              ctypes.c_int(channel), ctypes.c_uint(self.bar_epochs[channel]),
                                              ctypes.c_double(60.0),
                                              _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
            _lib.check_rc(rc, "symm_barrier")
        else:
            dist.barrier(self.group)

    def _ranges(self, a: int, b: int):
        """Cut the logical range [a, b) at slice boundaries: (owner, offset inside its slice, offset from a, length)."""
        out = []
        while a < b:
            r = a // self.per
            n = min(b, (r + 1) * self.per) - a
            out.append((r, a - r * self.per, a, n))
            a += n
        return out

    def _gather_range(self, key, pieces, max_ctas: int = 0):
        """pieces: list of (logical lo, logical hi, working offset). One copy kernel over peer memory per call.
        max_ctas: block budget of a copy that runs under compute kernels of another stream (0: fill the GPU)."""
        if self.world == 1:
            for a, b, w in pieces:
                self.work.data[w:w + (b - a)].copy_(self.param_shard[a:b])
            return
        if self.on_gpu:
            plan = self._plans.get(key)
            if plan is None:
                entries = []
                for a, b, w in pieces:
                    for r, so, la, n in self._ranges(a, b):
                        entries.append(CopyEntry(so, w + (la - a), 1, n, n, n, r))
                plan = self._plans[key] = ReshardPlan(entries, self.device)
            plan.run(self.param_ptrs, self.work, max_ctas)
            return
        full = torch.empty(self.padded, dtype=self.param_shard.dtype)
        dist.all_gather_into_tensor(full, self.param_shard, group=self.group)
        for a, b, w in pieces:
            self.work.data[w:w + (b - a)].copy_(full[a:b])   # .data: saved activations' version checks stay valid

    def gather_resident(self):
        pieces = []
        for s in self.model.specs:
            if s.name in self.res_map:
                pieces.append((s.offset, s.offset + _round(s.numel, ALIGN), self.res_map[s.name]))
        self._gather_range("resident", pieces)

    def _start_gather(self, i: int):
        """Begin pulling layer i into its slot. On a GPU the copy kernel runs on a side stream, after everything that
        is already enqueued on the compute stream (which includes the last user of that slot), so it overlaps with
        the layer that is about to run."""
        if self.slot_layer[i % self.pslots] == i:
            return
        a, b = self.layer_rng[i]
        pieces = [(a, b, self.slot_base[i % self.pslots])]
        if self.expert_range is not None:
            pieces = []
            e0, e1 = self.expert_range
            for sp in self.model.specs:
                if not sp.name.startswith(f"layers.{i}."):
                    continue
                w = self.slot_base[i % self.pslots] + (sp.offset - a)
                if len(sp.shape) == 3:                       # [experts, rows, cols]: the local experts' block only
                    per_e = sp.shape[1] * sp.shape[2]
                    pieces.append((sp.offset + e0 * per_e, sp.offset + e1 * per_e, w + e0 * per_e))
                else:
                    n = _round(sp.numel, ALIGN)
                    pieces.append((sp.offset, sp.offset + n, w))
        if self.on_gpu and self.world > 1 and OVERLAP:
            if self._side is None:
                # high priority: the copy's blocks are placed as soon as slots free up instead of queueing behind the
                # waves of the compute stream's kernels
                self._side = torch.cuda.Stream(device=self.device, priority=-1)
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                self._side.wait_event(ready)
                self._gather_range(("layer", i), pieces, OVERLAP_CTAS)
                done = torch.cuda.Event()
                done.record(self._side)
            self._inflight[i] = done
        else:
            self._gather_range(("layer", i), pieces)
        self.slot_layer[i % self.pslots] = i

    def gather_layer(self, i: int):
        """Layer i's parameters are in their slot for everything enqueued on the compute stream after this call."""
        self._start_gather(i)
        done = self._inflight.pop(i, None)
        if done is not None:
            torch.cuda.current_stream(self.device).wait_event(done)

    def _reduce_range(self, a: int, b: int, w_off: int, max_ctas: int = 0):
        """grad_shard[my part of logical [a, b)] += mean over ranks of the working gradients at w_off + (x - a)."""
        lo, hi = max(a, self.lo), min(b, self.hi)
        if self.world == 1:
            self.grad_shard[a:b].add_(self.grad_work[w_off:w_off + (b - a)])
            return
        if not self.on_gpu:
            buf = self.grad_work[w_off:w_off + (b - a)].clone()
            dist.all_reduce(buf, group=self.group)
            if lo < hi:
                self.grad_shard[lo - self.lo:hi - self.lo].add_(buf[lo - a:hi - a] / self.world)
            return
        if lo >= hi:
            return
        ptrs = (ctypes.c_void_p * self.world)(*[ctypes.c_void_p(int(p)) for p in self.grad_ptrs])
        step = self._tmp.numel()
        for c0 in range(lo, hi, step):
            n = min(step, hi - c0)
            tmp = self._tmp[:n]
            rc = _lib.lib().b200_zero_reduce(ptrs, None, ctypes.c_int(self.world), ctypes.c_longlong(w_off + (c0 - a)),
                                             ctypes.c_longlong(n), ctypes.c_float(1.0 / self.world), _lib.ptr(tmp),
                                             _lib.ptr(self.scalars), ctypes.c_int(max_ctas), _lib.stream_ptr())
            _lib.check_rc(rc, "zero_reduce")
            self.grad_shard[c0 - self.lo:c0 - self.lo + n].add_(tmp)

    # ------------------------------------------------------------------------------------------------ model hooks
    def before_layer_forward(self, i: int):
        self.gather_layer(i)
        if i + 1 < len(self.layer_rng):
            self._start_gather(i + 1)          # prefetch: overlaps with layer i's compute

    def pre_backward_hook(self, i: int):
        def hook(grad):
            ev = self._slot_reduced[i % self.gslots]
            if ev is not None:
                # layer i's weight gradients go into the gradient slot that layer i + G used: its reduction (which ran
                # on the side stream under the backward passes of the layers in between) must have emptied the slot
                torch.cuda.current_stream(self.device).wait_event(ev)
                self._slot_reduced[i % self.gslots] = None
            self.gather_layer(i)
            if i > 0:
                self._start_gather(i - 1)      # prefetch for the next layer of the backward pass
            return grad
        return hook

    def post_backward_hook(self, i: int):
        def hook(grad):
            self._layer_backward_done(i)
            return grad
        return hook

    def _layer_backward_done(self, i: int):
        """Layer i's weight gradients are complete on this rank: reduce them into the owners' gradient slices and empty
        the slot. With more than one rank this runs on a side stream, under the backward pass of layer i - 1:
        barrier (every rank finished layer i) -> pull-reduce -> barrier (every rank finished pulling) -> clear."""
        if not self.on_gpu:
            return                                     # CPU ranks reduce after loss.backward() (see backward)
        a, b = self.layer_rng[i]
        slot = self.gslot_base[i % self.gslots]
        width = self.slot_width
        if self.world == 1:
            self._reduce_range(a, b, slot)
            self.grad_work[slot:slot + width].zero_()
            return
        if not OVERLAP:
            self._sync(1)
            self._reduce_range(a, b, slot)
            self._sync(1)
            self.grad_work[slot:slot + width].zero_()
            return
        if self._rs_stream is None:
            self._rs_stream = torch.cuda.Stream(device=self.device, priority=-1)
        cur = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        with torch.cuda.stream(self._rs_stream):
            self._rs_stream.wait_event(ready)
            self._sync(1)
            self._reduce_range(a, b, slot, OVERLAP_CTAS)
            self._sync(1)
            self.grad_work[slot:slot + width].zero_()
            done = torch.cuda.Event()
            done.record(self._rs_stream)
        self._slot_reduced[i % self.gslots] = done

    def _finish_backward(self):
        """Resident parameters' gradients; joins the per-layer reductions still running on the side stream."""
        if self.on_gpu:
            cur = torch.cuda.current_stream(self.device)
            for k in range(self.gslots):
                if self._slot_reduced[k] is not None:
                    cur.wait_event(self._slot_reduced[k])
                    self._slot_reduced[k] = None
        self._sync()
        for s in self.model.specs:
            if s.name in self.res_map:
                self._reduce_range(s.offset, s.offset + _round(s.numel, ALIGN), self.res_map[s.name])
        self._sync()
        self.grad_work.zero_()
        self._pending_zero = -1

    # ------------------------------------------------------------------------------------------------ training API
    def backward(self, loss: torch.Tensor):
        assert self.trainable, "this engine holds a frozen model"
        loss.backward()
        self.micro_steps += 1
        if not self.on_gpu:
            # CPU restatements deliver gradients through autograd (.grad): run the per-layer reductions now, layer by
            # layer through the slots, in the order the GPU hooks would have
            with torch.no_grad():
                named = dict((s.name, p) for s, p in self.model.named_specs())
                L = self.model.cfg.num_hidden_layers
                self.grad_work.zero_()
                for i in reversed(range(L)):
                    for s in self.model.specs:
                        if s.name.startswith(f"layers.{i}.") and named[s.name].grad is not None:
                            named[s.name].main_grad.add_(named[s.name].grad.float())
                    a, b = self.layer_rng[i]
                    base = self.gslot_base[i % self.gslots]
                    self._reduce_range(a, b, base)
                    self.grad_work[base:base + self.slot_width].zero_()
                for s in self.model.specs:
                    if s.name in self.res_map and named[s.name].grad is not None:
                        named[s.name].main_grad.add_(named[s.name].grad.float())
                for p in named.values():
                    p.grad = None
        else:
            with torch.no_grad():
                for s, p in self.model.named_specs():
                    if p.grad is not None:          # resident parameters touched by plain torch ops
                        if s.name in self.res_map:
                            p.main_grad.add_(p.grad.float())
                        p.grad = None
        with torch.no_grad():
            self._finish_backward()

    def zero_grad(self):
        self.grad_shard.zero_()

    def current_lr(self) -> float:
        return self.scheduler.get_lr() if self.scheduler is not None else self.lr

    def grad_norm(self) -> float:
        return float(self.last_grad_norm) if self.last_grad_norm is not None else 0.0

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        assert self.trainable, "this engine holds a frozen model"
        self.opt_step += 1
        lr = self.current_lr()
        g = self.grad_shard
        sq = (g.double() ** 2).sum().float().reshape(1)
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        norm = sq.sqrt() * grad_scale
        self.last_grad_norm = norm[0]
        coef = torch.ones_like(norm)
        if self.max_norm:
            coef = torch.clamp(self.max_norm / (norm + 1e-6), max=1.0)
        scale = (coef * grad_scale)
        b1, b2 = self.betas
        if self.on_gpu:
            self.scalars[2:3] = scale
            L = _lib.lib()
            if self.decay_mask is not None:
                self.master.mul_(torch.where(self.decay_mask, 1.0 - lr * self.wd, 1.0))
            _lib.check_rc(L.b200_adamw(_lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq),
                                       _lib.ptr(g), _lib.ptr(self.param_shard), ctypes.c_longlong(g.numel()),
                                       ctypes.c_void_p(self.scalars.data_ptr() + 8), ctypes.c_float(lr),
                                       ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(self.eps),
                                       ctypes.c_float(0.0), ctypes.c_int(self.opt_step), ctypes.c_int(1),
                                       _lib.stream_ptr()), "adamw")
        else:
            gg = g * scale
            self.exp_avg.mul_(b1).add_(gg, alpha=1 - b1)
            self.exp_avg_sq.mul_(b2).addcmul_(gg, gg, value=1 - b2)
            bc1, bc2 = 1 - b1 ** self.opt_step, 1 - b2 ** self.opt_step
            if self.decay_mask is not None:
                self.master.mul_(torch.where(self.decay_mask, 1.0 - lr * self.wd, 1.0))
            self.master.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt_().add_(self.eps), value=-lr)
            self.param_shard.copy_(self.master.to(self.param_shard.dtype))
            self.grad_shard.zero_()
        self._sync()                       # every rank's new parameter slice is visible
        for ev in self._inflight.values():
            torch.cuda.current_stream(self.device).wait_event(ev)
        self._inflight.clear()
        self.slot_layer = [-1] * self.pslots
        self.gather_resident()
        if self.scheduler is not None:
            self.scheduler.step()

    # ------------------------------------------------------------------------------------------------ sleep
    def offload_states(self):
        """Optimizer slices (master weights, moments, gradient slice) to pinned host memory: --ds.enable_sleep."""
        if not self.trainable or getattr(self, "_host", None) is not None:
            return
        names = ("master", "exp_avg", "exp_avg_sq", "grad_shard")
        self._host = {}
        for n in names:
            t = getattr(self, n)
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)
            h.copy_(t)
            self._host[n] = h
            setattr(self, n, None)
        if self.on_gpu:
            torch.cuda.empty_cache()

    def reload_states(self):
        host = getattr(self, "_host", None)
        if host is None:
            return
        for n, h in host.items():
            setattr(self, n, h.to(self.device, non_blocking=True))
        self._host = None

    # ------------------------------------------------------------------------------------------------ full views
    @torch.no_grad()
    def gather_full(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """The whole logical flat parameter buffer (weight sync to a rollout engine, checkpoints)."""
        if out is None:
            out = torch.empty(self.padded, dtype=self.param_shard.dtype, device=self.device)
        if self.world == 1:
            out[: self.per].copy_(self.param_shard)
        elif self.on_gpu:
            key = ("full", out.data_ptr())
            plan = self._plans.get("full")
            if plan is None:
                plan = self._plans["full"] = ReshardPlan(
                    [CopyEntry(0, r * self.per, 1, self.per, self.per, self.per, r) for r in range(self.world)],
                    self.device)
            del key
            plan.run(self.param_ptrs, out)
        else:
            dist.all_gather_into_tensor(out, self.param_shard, group=self.group)
        return out

    # ------------------------------------------------------------------------------------------------ checkpoints
    # (same interface as ZeroEngine: utils/checkpoint.py writes one slice per rank and can re-slice on load)
    def shard_state(self) -> dict:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "lo": self.lo,
                "hi": self.hi, "opt_step": self.opt_step, "world": self.world,
                "total_numel": self.model.total_numel, "shard_size": self.per}

    @torch.no_grad()
    def load_shard_state(self, master, exp_avg, exp_avg_sq, opt_step) -> None:
        self.master.copy_(master)
        self.exp_avg.copy_(exp_avg)
        self.exp_avg_sq.copy_(exp_avg_sq)
        self.opt_step = int(opt_step)
        self.param_shard.copy_(self.master.to(self.param_shard.dtype))
        self._sync()
        self.slot_layer = [-1] * self.pslots
        self.gather_resident()
