"""Tensor parallelism for training: every rank of a TP group holds 1/tp of each projection and the same activations.

* qkv and gate_up are column-parallel (a rank owns Hq/tp query heads, Hkv/tp kv heads and I/tp FFN columns), o_proj and
  down_proj are row-parallel; an lm_head that is a matrix of its own is split by vocabulary rows (the log-prob kernel
  exchanges 16 bytes of softmax statistics per token); embeddings, norms and the value head are replicated. The
  per-rank model is an ordinary ``TransformerLM`` built from the local head / FFN counts, so every kernel (fused RoPE + attention, SwiGLU
  GEMM epilogue, fused log-prob head) runs unchanged on the shard.
* Two autograd-aware collectives stitch the shards together: the input of a column-parallel projection is an identity
  whose backward sums the input gradients over the group, the output of a row-parallel projection is a sum over the
  group whose backward is an identity. Residual stream, norms and the loss are computed redundantly on every rank.
* TP ranks read the same batches (the sampler shards by the data-parallel index only); gradients of the shards are
  reduced over the data-parallel group by the ZeRO engine; gradients of replicated parameters are additionally
  averaged over the TP group before the step (they agree up to atomic summation order, the average keeps the replicas
  bit-identical), and the clipping norm counts replicated parameters once.
* Checkpoints: HF export gathers the shards back into the full fused layout with the inverse of the weight-sync copy
  plan (parallel/reshard.py); optimizer shards are saved per (tp, dp) rank.

The reference gets this from DeepSpeed AutoTP (``--ds.tensor_parallel_size``: openrlhf/utils/deepspeed/deepspeed.py:389-398,
466-473; weights gathered with ``GatherReplacedLayerParams`` for export and weight sync, openrlhf/trainer/ray/ppo_actor.py:469-470).
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.transformer import TransformerLM, build_param_specs
from .reshard import ReshardPlan, _tp_row_ranges, build_plan, run_plan_reference


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, group):
        y = y.contiguous()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _RowParallelFused(torch.autograd.Function):
    """Row-parallel projection whose all-reduce rides on the GEMM: the epilogue adds every output tile into the fp32
    accumulation buffer of all TP ranks over NVLink (parallel/tp.py::TPContext.row_parallel, one kernel plus two flag
    barriers). Backward is local: dx = dy @ w, dw += dy^T x."""

    @staticmethod
    def forward(ctx, x, w, tpt):
        from ..ops import functional as F

        acc = tpt.fused_context(x.shape[0], w.shape[0]).row_parallel(x.contiguous(), w)
        ctx.save_for_backward(x, w)
        ctx.w_ref = w
        ctx.F = F
        return acc.to(torch.bfloat16)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm

        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            T = x.shape[0]
            tiles = ((w.shape[0] + 127) // 128) * ((w.shape[1] + 255) // 256)
            splits = max(1, min(8, 148 // max(tiles, 1), T // 512)) if tiles < 148 else 1
            dw = ctx.F._acc_grad(ctx.w_ref, lambda buf: gemm(dy, x, a_mn=True, b_mn=True, out=buf, accumulate=True,
                                                             k_splits=splits))
        return dx, dw, None


def vocab_parallel_head(cfg: ModelConfig, tp: int, with_lm_head: bool) -> bool:
    """The lm_head is split by vocabulary rows when it is a matrix of its own (no tied embeddings) and its rows divide
    evenly into shards that the GEMM accepts (multiples of 8); OPENRLHF_B200_TP_VOCAB_PARALLEL=0 keeps it replicated."""
    import os

    return (with_lm_head and not cfg.tie_word_embeddings and cfg.vocab_size % (8 * tp) == 0
            and os.environ.get("OPENRLHF_B200_TP_VOCAB_PARALLEL", "1") != "0")


def local_config(cfg: ModelConfig, tp: int, vocab_parallel: bool = False) -> ModelConfig:
    assert cfg.num_experts == 0, "tensor-parallel training covers dense models (MoE layers use expert parallelism)"
    assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0 and cfg.intermediate_size % tp == 0, \
        "attention heads, kv heads and the FFN width must be divisible by the tensor-parallel size"
    return dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // tp,
                               num_key_value_heads=cfg.num_key_value_heads // tp,
                               intermediate_size=cfg.intermediate_size // tp, head_dim=cfg.head_dim,
                               lm_head_vocab=cfg.vocab_size // tp if vocab_parallel else 0)


class TPTrain:
    """Attached to a shard model as ``model.tp_train``."""

    def __init__(self, full_cfg: ModelConfig, group, with_lm_head: bool, with_value_head: bool):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.full_cfg = full_cfg
        self.with_lm_head, self.with_value_head = with_lm_head, with_value_head
        # vocabulary-parallel head: this rank's rows [vocab_start, vocab_start + vocab_size / tp) of lm_head.weight
        self.vocab_parallel = vocab_parallel_head(full_cfg, self.size, with_lm_head)
        self.vocab_start = self.rank * (full_cfg.vocab_size // self.size) if self.vocab_parallel else 0
        self.entries, self.shard_numel = build_plan(full_cfg, self.rank, self.size, with_lm_head=with_lm_head,
                                                    with_value_head=with_value_head,
                                                    vocab_parallel=self.vocab_parallel)
        # GEMM + all-reduce in one kernel for the row-parallel projections of the forward pass (GPU, bf16);
        # OPENRLHF_B200_TP_FUSED=0 falls back to a GEMM followed by an NCCL all-reduce
        import os

        self.fused = os.environ.get("OPENRLHF_B200_TP_FUSED", "1") != "0"
        self._fctx = None
        self.device = None

    # ---- collectives used by TransformerLM
    def copy_in(self, x):
        return _CopyToTP.apply(x, self.group) if torch.is_grad_enabled() and x.requires_grad else x

    def reduce_out(self, y):
        return _ReduceFromTP.apply(y, self.group)

    def row_parallel_linear(self, x, w):
        """sum over the TP group of x @ w.T for a row-parallel weight shard w [N, K/tp]."""
        from ..ops import functional as F

        if self.fused and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] > 0:
            return _RowParallelFused.apply(x, w, self)
        return self.reduce_out(F.linear(x, w))

    def fused_context(self, rows: int, cols: int):
        """Symmetric accumulation buffers of the fused GEMM + all-reduce, grown (collectively: every TP rank sees the
        same shapes) when a larger micro-batch arrives."""
        from .tp import TPContext

        need = rows * cols
        if self._fctx is None or need > self._fctx.max_rows * self._fctx.max_cols:
            cap_rows = max(rows, 4096)
            cap_rows = (cap_rows + 1023) // 1024 * 1024
            self._fctx = TPContext(self.group, cap_rows, cols, 8, self.device)
        return self._fctx

    # ---- parameter classes
    def replicated_specs(self, model: TransformerLM):
        """Specs of the shard model whose tensor is the whole parameter (identical on every TP rank)."""
        full = {s.name: s for s in build_param_specs(self.full_cfg, self.with_lm_head, self.with_value_head)}
        return [s for s in model.specs if s.numel == full[s.name].numel]

    def replicated_mask(self, model: TransformerLM, lo: int, hi: int, device) -> torch.Tensor:
        m = torch.zeros(hi - lo, dtype=torch.bool, device=device)
        for s in self.replicated_specs(model):
            a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
            if a < b:
                m[a - lo:b - lo] = True
        return m

    @torch.no_grad()
    def sync_replicated_grads(self, model: TransformerLM):
        """Average the gradients of replicated parameters over the TP group (fp32 main_grad, else .grad)."""
        for s in self.replicated_specs(model):
            p = model.p(s.name)
            g = getattr(p, "main_grad", None)
            if g is None:
                g = p.grad
            if g is None:
                continue
            dist.all_reduce(g, group=self.group)
            g.div_(self.size)

    # ---- layout conversion
    @torch.no_grad()
    def load_from_full(self, full_flat: torch.Tensor, model: TransformerLM):
        """Fill this rank's shard from a full flat buffer on the same device."""
        if full_flat.is_cuda:
            ReshardPlan(self.entries, full_flat.device).run([full_flat.data_ptr()], model.flat)
        else:
            run_plan_reference(self.entries, [full_flat], model.flat)

    @torch.no_grad()
    def gather_full(self, model: TransformerLM) -> torch.Tensor:
        """The full flat parameter buffer (trainer layout), rebuilt on every rank from all shards."""
        specs = build_param_specs(self.full_cfg, self.with_lm_head, self.with_value_head)
        total = specs[-1].offset + specs[-1].numel
        full = torch.zeros(total, dtype=model.flat.dtype, device=model.flat.device)
        n = model.flat.numel()
        shards = [torch.empty_like(model.flat) for _ in range(self.size)]
        dist.all_gather(shards, model.flat.contiguous(), group=self.group)
        for r in range(self.size):
            entries, _ = build_plan(self.full_cfg, r, self.size, with_lm_head=self.with_lm_head,
                                    with_value_head=self.with_value_head, vocab_parallel=self.vocab_parallel)
            for e in entries:            # inverse of full -> shard: destination and source swap roles
                dst = full.as_strided((e.rows, e.row_elems), (e.src_ld, 1), e.src_off)
                src = shards[r].as_strided((e.rows, e.row_elems), (e.dst_ld, 1), e.dst_off)
                dst.copy_(src)
        assert n >= self.shard_numel
        return full


def shard_for_training(full: TransformerLM, group, shard_world: int = 1) -> TransformerLM:
    """This rank's tensor-parallel shard of `full` (same device, same dtype), ready for the optimizer engine.
    shard_world: size of the data-parallel group whose ZeRO engine will slice the shard's flat buffer."""
    tp = dist.get_world_size(group)
    assert getattr(full, "lora", None) is None, "tensor-parallel training does not cover LoRA adapters"
    assert not full.cfg.is_vlm, "tensor-parallel training does not cover vision-language models"
    ctx = TPTrain(full.cfg, group, full.with_lm_head, full.with_value_head)
    shard = TransformerLM(local_config(full.cfg, tp, ctx.vocab_parallel), device=full.flat.device,
                          dtype=full.flat.dtype,
                          with_lm_head=full.with_lm_head, with_value_head=full.with_value_head, seed=None,
                          shard_world=shard_world)
    assert shard.total_numel <= ctx.shard_numel + 128
    ctx.load_from_full(full.flat, shard)
    ctx.device = full.flat.device
    shard.tp_train = ctx
    shard.gradient_checkpointing = full.gradient_checkpointing
    shard.train(full.training)
    return shard
