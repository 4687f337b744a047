"""Own decoder-only transformer definition for the Llama-3, Qwen2.5 and Qwen3(-MoE) architectures.

The reference never defines a model: it instantiates HF ``AutoModelForCausalLM`` classes (openrlhf/models/actor.py:98-157,
openrlhf/models/model.py:77-118). This module owns the architecture so that every op runs on this framework's kernels:
the packed token stream ``[T]`` is the only input layout (no padding anywhere), q/k/v and gate/up projections are
stored fused (the layout the rollout engine uses as well, so trainer and rollout can share one weight buffer), and all
parameters are views into one flat bf16 buffer (the unit of ZeRO sharding, weight sync and checkpointing).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.utils.checkpoint

from ..ops import functional as F
from .config import ModelConfig

ALIGN = 128  # every parameter starts on a 256-byte boundary of the flat buffer (TMA needs 16 B; shards like 256 B)


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    offset: int
    numel: int
    decay: bool       # subject to weight decay (matrices) or exempt (norms, biases)
    init: str         # normal | ones | zeros


def build_param_specs(cfg: ModelConfig, with_lm_head: bool = True, with_value_head: bool = False) -> list[ParamSpec]:
    specs: list[ParamSpec] = []
    off = 0

    def add(name, shape, decay=True, init="normal"):
        nonlocal off
        n = math.prod(shape)
        specs.append(ParamSpec(name, tuple(shape), off, n, decay, init))
        off += (n + ALIGN - 1) // ALIGN * ALIGN

    H = cfg.hidden_size
    add("embed.weight", (cfg.vocab_size, H))
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        add(p + "norm1.weight", (H,), False, "ones")
        add(p + "qkv.weight", (cfg.qkv_size, H))
        if cfg.attention_bias:
            add(p + "qkv.bias", (cfg.qkv_size,), False, "zeros")
        if cfg.qk_norm:
            add(p + "q_norm.weight", (cfg.head_dim,), False, "ones")
            add(p + "k_norm.weight", (cfg.head_dim,), False, "ones")
        add(p + "o.weight", (H, cfg.q_size))
        add(p + "norm2.weight", (H,), False, "ones")
        if cfg.is_moe_layer(i):
            I = cfg.moe_intermediate_size
            add(p + "router.weight", (cfg.num_experts, H))
            add(p + "experts.gate_up", (cfg.num_experts, 2 * I, H))
            add(p + "experts.down", (cfg.num_experts, H, I))
        else:
            add(p + "gate_up.weight", (2 * cfg.intermediate_size, H))
            add(p + "down.weight", (H, cfg.intermediate_size))
    add("norm.weight", (H,), False, "ones")
    if with_lm_head and not cfg.tie_word_embeddings:
        add("lm_head.weight", (cfg.lm_head_vocab or cfg.vocab_size, H))
    if with_value_head:
        add("value_head.weight", (1, H))
    if cfg.vision is not None:
        from .vision import vision_param_shapes

        for name, shape, decay, init in vision_param_shapes(cfg.vision_config()):
            add(name, shape, decay, init)
    return specs


class TransformerLM(nn.Module):
    """Decoder stack over a packed token stream. ``forward`` returns the final-norm hidden states [T, H]."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype=torch.bfloat16, with_lm_head=True, with_value_head=False,
                 init_std: float = 0.02, seed: int | None = 0, flat: torch.Tensor | None = None,
                 shard_world: int = 1):
        super().__init__()
        self.cfg = cfg
        self.specs = build_param_specs(cfg, with_lm_head, with_value_head)
        self.with_lm_head, self.with_value_head = with_lm_head, with_value_head
        total = self.specs[-1].offset + (self.specs[-1].numel + ALIGN - 1) // ALIGN * ALIGN
        if flat is None:
            # room for the padding that makes the flat index space divisible into `shard_world` aligned shards
            per = ((total + shard_world - 1) // shard_world + 255) // 256 * 256
            flat = torch.zeros(per * shard_world, dtype=dtype, device=device)
        assert flat.numel() >= total
        self.flat = flat                      # not a Parameter: parameters are views into it
        self.total_numel = total
        self._params: dict[str, nn.Parameter] = {}
        for s in self.specs:
            view = flat[s.offset:s.offset + s.numel].view(s.shape)
            p = nn.Parameter(view, requires_grad=True)
            self._params[s.name] = p
            self.register_parameter(s.name.replace(".", "__"), p)
        self.gradient_checkpointing = False
        self.tp_group = None   # set on a tensor-parallel shard of the model (rollout/tp_engine.py)
        self.tp_train = None   # parallel.tp_train.TPTrain: this model is one rank's shard of a TP-trained model
        self.ep = None   # parallel.ep.EPContext: MoE layers run expert-parallel over its group
        self.cp = None   # parallel.cp.CPContext: attention over a context-parallel group (inputs are this rank's rows)
        self.lora = None                      # optional LoraAdapters (models/lora.py)
        self.max_pos = min(cfg.max_position_embeddings, 1 << 17)
        if seed is not None:
            self.reset_parameters(init_std, seed)

    # ------------------------------------------------------------------ parameters
    def p(self, name: str) -> nn.Parameter:
        return self._params[name]

    def named_specs(self):
        return [(s, self._params[s.name]) for s in self.specs]

    @torch.no_grad()
    def reset_parameters(self, std: float = 0.02, seed: int = 0):
        g = torch.Generator(device=self.flat.device).manual_seed(seed)
        for s, p in self.named_specs():
            if s.init == "ones":
                p.fill_(1.0)
            elif s.init == "zeros":
                p.zero_()
            elif s.name == "value_head.weight":
                # N(0, 1/(hidden+1)) as in openrlhf/models/model.py:164-172
                p.copy_(torch.randn(s.shape, generator=g, device=p.device, dtype=torch.float32)
                        * (1.0 / math.sqrt(self.cfg.hidden_size + 1)))
            else:
                # chunked to bound the fp32 temporary for large embeddings
                flat = p.view(-1)
                step = 1 << 26
                for a in range(0, flat.numel(), step):
                    b = min(flat.numel(), a + step)
                    flat[a:b].copy_(torch.randn(b - a, generator=g, device=p.device, dtype=torch.float32) * std)

    def lm_head_weight(self) -> torch.Tensor:
        return self.p("embed.weight") if self.cfg.tie_word_embeddings else self.p("lm_head.weight")

    def rope(self, device) -> torch.Tensor:
        return F.rope_table(self.cfg.head_dim, self.cfg.rope_theta, self.max_pos, device)

    # ------------------------------------------------------------------ forward
    def _lin(self, i: int, target: str, x, bias=None, residual=None):
        """Projection `target` of layer i, plus its low-rank adapter when adapters are attached."""
        if self.tp_group is not None and target in ("o", "down"):
            # row-parallel shard (rollout engine with tensor parallelism, prefill path): partial product, sum over the
            # TP group, then the residual once
            import torch.distributed as dist

            y = F.linear(x, self.p(f"layers.{i}.{target}.weight"), bias, None)
            dist.all_reduce(y, group=self.tp_group)
            return y if residual is None else y + residual
        if self.tp_train is not None and target in ("o", "down"):
            # row-parallel shard in training: the sum over the group is differentiable (identity backwards)
            assert bias is None
            y = self.tp_train.row_parallel_linear(x, self.p(f"layers.{i}.{target}.weight"))
            return y if residual is None else y + residual
        y = F.linear(x, self.p(f"layers.{i}.{target}.weight"), bias, residual)
        if self.lora is not None:
            d = self.lora.delta(i, target, x)
            if d is not None:
                y = y + d.to(y.dtype)
        return y

    def _attention_block(self, i: int, h, pos, cu_seqlens, max_seqlen, attn_fn=None):
        cfg = self.cfg
        pre = f"layers.{i}."
        rope_tab = None
        if isinstance(pos, tuple):          # (row index, per-token rotary rows): multimodal positions
            pos, rope_tab = pos
        x = F.rmsnorm(h, self.p(pre + "norm1.weight"), cfg.rms_norm_eps)
        if self.tp_train is not None:
            x = self.tp_train.copy_in(x)        # column-parallel input: gradients are summed over the group
        qkv = self._lin(i, "qkv", x, self._params.get(pre + "qkv.bias"))
        if rope_tab is None:
            rope_tab = self.rope(qkv.device)
        T = qkv.shape[0]
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if cfg.qk_norm:
            qk = qkv[:, : (Hq + Hkv) * D].reshape(T, Hq + Hkv, D)
            qn = F.rmsnorm(qk[:, :Hq].reshape(-1, D), self.p(pre + "q_norm.weight"), cfg.rms_norm_eps).view(T, Hq * D)
            kn = F.rmsnorm(qk[:, Hq:].reshape(-1, D), self.p(pre + "k_norm.weight"), cfg.rms_norm_eps).view(T, Hkv * D)
            qkv = torch.cat([qn, kn, qkv[:, (Hq + Hkv) * D:]], dim=1)
        if self.cp is not None and attn_fn is None:
            a = self.cp.attention(qkv, pos, rope_tab, cu_seqlens, 1.0 / math.sqrt(D))
            return self._lin(i, "o", a, None, h)
        if attn_fn is None and qkv.is_cuda and D == 128 and qkv.dtype == torch.bfloat16:
            from ..ops.attention import rope_attention

            a = rope_attention(qkv, pos, rope_tab, cu_seqlens, Hq, Hkv, 1.0 / math.sqrt(D))
            return self._lin(i, "o", a, None, h)
        qkv = F.rope(qkv, pos, rope_tab, Hq + Hkv, D)
        q = qkv[:, : Hq * D].view(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        if attn_fn is not None:
            a = attn_fn(i, q, k, v)
        else:
            a = F.attention_varlen(q, k, v, cu_seqlens, max_seqlen)
        return self._lin(i, "o", a.reshape(T, Hq * D), None, h)

    def _mlp_block(self, i: int, h):
        cfg = self.cfg
        pre = f"layers.{i}."
        x = F.rmsnorm(h, self.p(pre + "norm2.weight"), cfg.rms_norm_eps)
        if self.tp_train is not None:
            x = self.tp_train.copy_in(x)
        if cfg.is_moe_layer(i):
            from .moe import moe_forward

            y, aux = moe_forward(x, self.p(pre + "router.weight"), self.p(pre + "experts.gate_up"),
                                 self.p(pre + "experts.down"), cfg.num_experts_per_tok, cfg.norm_topk_prob, ep=self.ep)
            return h + y, aux
        if self.lora is None:
            a = F.linear_swiglu(x, self.p(pre + "gate_up.weight"))      # activation fused into the GEMM epilogue
        else:
            a = F.swiglu(self._lin(i, "gate_up", x))
        return self._lin(i, "down", a, None, h), None

    def _layer(self, i, h, pos, cu_seqlens, max_seqlen, attn_fn=None):
        h = self._attention_block(i, h, pos, cu_seqlens, max_seqlen, attn_fn)
        h, aux = self._mlp_block(i, h)
        if aux is None:
            aux = h.new_zeros((), dtype=torch.float32)
        return h, aux

    def image_embeds(self, pixel_values: torch.Tensor, image_grid_thw: torch.Tensor) -> torch.Tensor:
        """Vision tower: the processor's flattened patches -> one embedding per image placeholder token."""
        from .vision import vision_forward

        return vision_forward(self.p, self.cfg.vision_config(), pixel_values, image_grid_thw)

    def multimodal_inputs(self, input_ids, cu_list, pixel_values, image_grid_thw):
        """Embeddings with the image placeholders filled in, and per-token M-RoPE rows for the packed stream.
        cu_list: document boundaries as Python ints. Returns (embeds [T, H], (row index [T], rows [T, D/2, 2]))."""
        from .vision import image_runs, mrope_positions, mrope_rows, scatter_image_embeds

        cfg = self.cfg
        merge = cfg.vision_config().spatial_merge_size
        embeds = F.embedding(input_ids, self.p("embed.weight"))
        grids = [tuple(g) for g in image_grid_thw.tolist()] if image_grid_thw is not None else []
        ids = input_ids.tolist()
        pos3, where, gi = [], [], 0
        for a, b in zip(cu_list[:-1], cu_list[1:]):
            doc = ids[a:b]
            runs = image_runs(doc, grids[gi:], cfg.image_token_id, merge, cfg.video_token_id)
            mine = [r[2] for r in runs]
            p3, _ = mrope_positions(doc, mine, cfg.image_token_id, merge, cfg.video_token_id)
            for start, cnt, _g in runs:
                where.append(torch.arange(a + start, a + start + cnt))
            gi += len(runs)
            pos3.append(p3)
        assert gi == len(grids), f"{len(grids)} images were passed but the token stream holds {gi} complete image runs"
        if pixel_values is not None and len(grids):
            embeds = scatter_image_embeds(embeds, torch.cat(where), self.image_embeds(pixel_values, image_grid_thw))
        pos3 = torch.cat(pos3, dim=1)
        rows = mrope_rows(self.rope(input_ids.device), pos3, cfg.mrope_section or (cfg.head_dim // 2,))
        return embeds, (torch.arange(input_ids.numel(), dtype=torch.int32, device=input_ids.device), rows)

    def forward(self, input_ids: torch.Tensor, position_ids, cu_seqlens: torch.Tensor, max_seqlen: int,
                attn_fn=None, inputs_embeds: torch.Tensor | None = None):
        """input_ids int64 [T], position_ids int32 [T] (restart at 0 per document), cu_seqlens int32 [n+1].
        Vision-language batches pass `inputs_embeds` and `position_ids = (row index, rotary rows)` from
        `multimodal_inputs`.

        Returns (hidden [T,H] after the final norm, aux_loss scalar: sum of the MoE load-balancing terms)."""
        h = inputs_embeds if inputs_embeds is not None else F.embedding(input_ids, self.p("embed.weight"))
        aux_total = h.new_zeros((), dtype=torch.float32)
        z3 = getattr(self, "z3", None)      # parallel.zero3.Zero3Engine: layer parameters live in two shared slots
        for i in range(self.cfg.num_hidden_layers):
            if z3 is not None:
                z3.before_layer_forward(i)
                if h.requires_grad and torch.is_grad_enabled():
                    h.register_hook(z3.post_backward_hook(i))      # fires once layer i's backward is complete
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                h, aux = torch.utils.checkpoint.checkpoint(self._layer, i, h, position_ids, cu_seqlens, max_seqlen,
                                                           attn_fn, use_reentrant=False)
            else:
                h, aux = self._layer(i, h, position_ids, cu_seqlens, max_seqlen, attn_fn)
            if z3 is not None and h.requires_grad and torch.is_grad_enabled():
                h.register_hook(z3.pre_backward_hook(i))           # fires before layer i's backward starts
            aux_total = aux_total + aux
        h = F.rmsnorm(h, self.p("norm.weight"), self.cfg.rms_norm_eps)
        return h, aux_total

    # ------------------------------------------------------------------ heads
    def logprobs(self, hidden, labels, temperature=1.0, want_entropy=False, chunk=4096):
        tpt = self.tp_train
        if tpt is not None and tpt.vocab_parallel:
            # this rank holds vocab_size / tp rows of the head: every rank streams its own columns of the logits and
            # the ranks exchange 16 bytes of softmax statistics per token
            return F.vocab_parallel_logprob(hidden, self.lm_head_weight(), labels, tpt.vocab_start, tpt.group,
                                            temperature, want_entropy, chunk)
        return F.fused_logprob(hidden, self.lm_head_weight(), labels, temperature, want_entropy, chunk)

    def logits(self, hidden):
        tpt = self.tp_train
        if tpt is not None and tpt.vocab_parallel:
            import torch.distributed as dist

            assert not (torch.is_grad_enabled() and hidden.requires_grad), \
                "full logits of a vocabulary-parallel head are for evaluation; train through logprobs()"
            local = F.linear(hidden, self.lm_head_weight())
            parts = [torch.empty_like(local) for _ in range(tpt.size)]
            dist.all_gather(parts, local.contiguous(), group=tpt.group)
            return torch.cat(parts, dim=1)
        return F.linear(hidden, self.lm_head_weight())

    def values(self, hidden):
        return F.value_head(hidden, self.p("value_head.weight"))
