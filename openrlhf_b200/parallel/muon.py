"""Muon optimizer engine: momentum + Newton-Schulz orthogonalisation for the 2-D hidden matrices, AdamW for the rest
(embeddings, lm_head, norms, biases, router).

Same training interface as ZeroEngine (``backward`` / ``step`` / ``zero_grad`` / ``current_lr``). Sharding is by whole
tensor instead of by flat slice, because the Newton-Schulz iteration needs a matrix in one piece: gradients are
averaged over the data-parallel group, every tensor has one owner rank (greedy by size) that keeps its fp32 master
weights and optimizer state and computes the update, and owners broadcast their bf16 results. The five Newton-Schulz
iterations run on the tcgen05 GEMM (``X X^T``, ``A A``, ``B X`` in bf16 with fp32 accumulation).

Reference: DeepSpeed's Muon as configured by openrlhf/utils/deepspeed/deepspeed.py:305-356 (muon group: lr, momentum,
weight_decay; aux AdamW group: lr, betas, eps, weight_decay; ns_steps = 5 and nesterov = True are fixed there).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def _mm(a: torch.Tensor, b: torch.Tensor, b_mn: bool) -> torch.Tensor:
    """a [M,K] @ (b [N,K]^T or b [K,N]); own GEMM when the shapes allow TMA (strides multiples of 8), else torch."""
    if a.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.shape[0] % 8 == 0 \
            and b.shape[0] % 8 == 0:
        from ..ops.gemm import gemm

        return gemm(a.contiguous(), b.contiguous(), b_mn=b_mn)
    return (a.float() @ (b.float() if b_mn else b.float().t())).to(a.dtype)


def newton_schulz5(g: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate orthogonalisation U V^T of g = U S V^T (quintic Newton-Schulz, bf16 matmuls). Returns fp32."""
    a, b, c = NS_COEFFS
    x = g.float()
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = (x / (x.norm() + 1e-7)).to(torch.bfloat16).contiguous()
    for _ in range(steps):
        A = _mm(x, x, False)                    # X X^T
        B = (b * A.float() + c * _mm(A, A, False).float()).to(torch.bfloat16)   # A is symmetric: A A^T = A A
        x = (a * x.float() + _mm(B, x, True).float()).to(torch.bfloat16)
    x = x.float()
    return x.t() if transposed else x


def is_muon_param(name: str, shape) -> bool:
    if len(shape) < 2 or "layers." not in name:
        return False
    return not any(k in name for k in ("router", "norm", "embed", "lm_head", "value_head"))


class MuonEngine:
    def __init__(self, model, muon_lr: float = 2e-2, momentum: float = 0.95, adam_lr: float = 1e-6, betas=(0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.0, max_norm: float = 0.0, group=None, scheduler=None,
                 ns_steps: int = 5, nesterov: bool = True):
        self.model, self.flat, self.device, self.group = model, model.flat, model.flat.device, group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.muon_lr, self.momentum, self.adam_lr, self.betas, self.eps = muon_lr, momentum, adam_lr, betas, eps
        self.wd, self.max_norm, self.scheduler = weight_decay, max_norm, scheduler
        self.ns_steps, self.nesterov = ns_steps, nesterov
        self.opt_step = self.micro_steps = 0
        self.last_grad_norm = None
        n = model.specs[-1].offset + model.specs[-1].numel
        self.grad_flat = torch.zeros(n, dtype=torch.float32, device=self.device)
        load = [0] * self.world
        self.owner, self.state = {}, {}
        for s, p in sorted(model.named_specs(), key=lambda sp: -sp[0].numel):
            r = min(range(self.world), key=lambda i: load[i])
            load[r] += s.numel
            self.owner[s.name] = r
        for s, p in model.named_specs():
            p.main_grad = self.grad_flat[s.offset:s.offset + s.numel].view(s.shape)
            if self.owner[s.name] == self.rank:
                st = {"master": p.detach().float().clone()}
                if is_muon_param(s.name, s.shape):
                    st["buf"] = torch.zeros_like(st["master"])
                else:
                    st["m"], st["v"] = torch.zeros_like(st["master"]), torch.zeros_like(st["master"])
                self.state[s.name] = st

    # ------------------------------------------------------------------ training API (mirrors ZeroEngine)
    def backward(self, loss: torch.Tensor):
        loss.backward()
        self.micro_steps += 1
        with torch.no_grad():
            for _, p in self.model.named_specs():
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None

    def zero_grad(self):
        self.grad_flat.zero_()

    def current_lr(self) -> float:
        return self.scheduler.get_lr() if self.scheduler is not None else self.adam_lr

    def grad_norm(self) -> float:
        return float(self.last_grad_norm) if self.last_grad_norm is not None else 0.0

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        self.opt_step += 1
        ratio = 1.0
        if self.scheduler is not None:          # one schedule drives both groups through its ratio to the base lr
            ratio = self.scheduler.get_lr() / max(self.scheduler.base_lr, 1e-30)
        if self.world > 1:
            dist.all_reduce(self.grad_flat, group=self.group)
            self.grad_flat /= self.world
        if grad_scale != 1.0:
            self.grad_flat *= grad_scale
        norm = self.grad_flat.norm()
        self.last_grad_norm = norm
        if self.max_norm and self.max_norm > 0:
            self.grad_flat *= torch.clamp(self.max_norm / (norm + 1e-6), max=1.0)
        b1, b2 = self.betas
        for s, p in self.model.named_specs():
            if self.owner[s.name] != self.rank:
                continue
            st, g = self.state[s.name], p.main_grad
            w = st["master"]
            if "buf" in st:
                lr = self.muon_lr * ratio
                st["buf"].mul_(self.momentum).add_(g)
                u = g.add(st["buf"], alpha=self.momentum) if self.nesterov else st["buf"]
                mats = u.reshape(-1, *u.shape[-2:])
                o = torch.stack([newton_schulz5(m, self.ns_steps) for m in mats]).reshape(u.shape)
                scale = max(1.0, u.shape[-2] / u.shape[-1]) ** 0.5
                w.mul_(1.0 - lr * self.wd).add_(o, alpha=-lr * scale)
            else:
                lr = self.adam_lr * ratio
                st["m"].mul_(b1).add_(g, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** self.opt_step, 1 - b2 ** self.opt_step
                if s.decay:
                    w.mul_(1.0 - lr * self.wd)
                w.addcdiv_(st["m"] / bc1, (st["v"] / bc2).sqrt_().add_(self.eps), value=-lr)
            p.data.copy_(w.to(p.dtype))
        if self.world > 1:
            works = [dist.broadcast(p.data, src=dist.get_global_rank(self.group, self.owner[s.name])
                                    if self.group is not None else self.owner[s.name], group=self.group, async_op=True)
                     for s, p in self.model.named_specs()]
            for wk in works:
                wk.wait()
        self.grad_flat.zero_()
        if self.scheduler is not None:
            self.scheduler.step()
