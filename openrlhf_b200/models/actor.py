"""Policy / reference model wrapper with the reference's ``Actor.forward`` contract
(openrlhf/models/actor.py:221-296): padded ``sequences (B,T)`` + ``action_mask (B,A)`` + ``attention_mask (B,T)`` in,
per-action log-probs ``(B,A)`` out, with optional entropy. Internally the batch is always packed (no padding reaches
a kernel) and the LM head is fused with the log-softmax so ``[T,V]`` logits are never materialised.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .config import ModelConfig
from .packing import PackedBatch, pack_padded, unpack_to_padded
from .transformer import TransformerLM


@dataclass
class ActorOutput:
    logits: torch.Tensor | None = None
    aux_loss: torch.Tensor | None = None
    entropy: torch.Tensor | None = None
    log_probs: torch.Tensor | None = None

    def __contains__(self, key) -> bool:
        return getattr(self, key, None) is not None

    def __getitem__(self, key):
        return getattr(self, key)


class Actor(nn.Module):
    def __init__(self, pretrain_or_model, device="cuda", temperature: float = 1.0, packing_samples: bool = True,
                 shard_world: int = 1, seed: int = 0, lora_rank: int = 0, lora_alpha: float = 16,
                 target_modules="all-linear", lora_dropout: float = 0.0, freeze_visual_encoder: bool = False,
                 load_in_4bit: bool = False, **_unused):
        super().__init__()
        if isinstance(pretrain_or_model, TransformerLM):
            self.model = pretrain_or_model
        else:
            from .hf_io import load_pretrained

            self.model = load_pretrained(pretrain_or_model, device=device, shard_world=shard_world, seed=seed)
        self.cfg: ModelConfig = self.model.cfg
        self.lora = None
        if lora_rank and lora_rank > 0:
            from .lora import LoraAdapters

            self.lora = LoraAdapters(self.model, lora_rank, lora_alpha, target_modules, lora_dropout, seed)
            self.lora._cfg = self.cfg
        if load_in_4bit:
            # QLoRA: the frozen projection weights take their NF4 values (ops/nf4.py); adapters train in bf16
            from ..ops.nf4 import apply_to_model

            apply_to_model(self.model)
        self.temperature = temperature
        self.packing_samples = packing_samples
        self.is_vlm = self.cfg.is_vlm
        if self.is_vlm and freeze_visual_encoder:
            # only the language model trains (and only it changes between weight syncs);
            # openrlhf/models/actor.py:167-175
            for s, p in self.model.named_specs():
                if s.name.startswith("visual."):
                    p.requires_grad_(False)

    def gradient_checkpointing_enable(self, **_kw):
        self.model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.model.gradient_checkpointing = False

    def print_trainable_parameters(self):
        """One line with the trainable and total parameter counts (LoRA adapters included), like the PEFT helper the
        reference forwards to (openrlhf/models/actor.py:304-305). Returns (trainable, total)."""
        total = trainable = 0
        for _, p in self.model.named_specs():
            total += p.numel()
            trainable += p.numel() if p.requires_grad else 0
        lora = getattr(self.model, "lora", None)
        if lora is not None:
            n = sum(p.numel() for p in lora.parameters())
            total += n
            trainable += sum(p.numel() for p in lora.parameters() if p.requires_grad)
        print(f"trainable params: {trainable:,} || all params: {total:,} || trainable%: "
              f"{100.0 * trainable / max(total, 1):.4f}")
        return trainable, total

    # ------------------------------------------------------------------ native packed API
    def forward_packed(self, pb: PackedBatch, return_entropy: bool = False, context_parallel=None,
                       pixel_values=None, image_grid_thw=None):
        """Per-token log-prob of the next token over the packed stream: returns (logp [T], entropy [T] | None, aux).
        pixel_values / image_grid_thw: the image processor's outputs for the images of the batch, in batch order."""
        if context_parallel is not None and context_parallel.size > 1:
            assert pixel_values is None, "context parallelism does not cover image inputs"
            return context_parallel.forward_logprobs(self.model, pb, self.temperature, return_entropy)
        if self.is_vlm and pixel_values is not None:
            cu_list = pb.cu_list if pb.cu_list is not None else pb.cu_seqlens.tolist()
            dev = pb.input_ids.device
            emb, pos = self.model.multimodal_inputs(pb.input_ids, cu_list, pixel_values.to(dev), image_grid_thw)
            h, aux = self.model(pb.input_ids, pos, pb.cu_seqlens, pb.max_seqlen, inputs_embeds=emb)
        else:
            h, aux = self.model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        logp, ent = self.model.logprobs(h, pb.labels, self.temperature, return_entropy)
        return logp, ent, aux

    # ------------------------------------------------------------------ reference-compatible padded API
    def forward(self, sequences: torch.LongTensor, action_mask: torch.Tensor | None = None,
                attention_mask: torch.Tensor | None = None, return_output: bool = False,
                allgather_logits: bool = False, return_logprobs: bool = False, ring_attn_group=None,
                packed_seq_lens=None, return_entropy: bool = False, context_parallel=None,
                pixel_values=None, image_grid_thw=None, **_mm_unused):
        if attention_mask is None:
            attention_mask = torch.ones_like(sequences)
        pb = pack_padded(sequences, attention_mask)
        if context_parallel is None and ring_attn_group is not None and sequences.is_cuda:
            if getattr(self, "_cp", None) is None or self._cp.group is not ring_attn_group:
                from ..parallel.cp import ContextParallel

                self._cp = ContextParallel(ring_attn_group)
            context_parallel = self._cp
        logp_t, ent_t, aux = self.forward_packed(pb, return_entropy, context_parallel, pixel_values, image_grid_thw)
        log_probs = unpack_to_padded(logp_t, pb)[:, :-1]
        out = ActorOutput(aux_loss=aux)
        if return_entropy:
            out.entropy = unpack_to_padded(ent_t, pb)[:, :-1]
        if action_mask is None:
            out.log_probs = log_probs
            return (log_probs, out) if return_output else log_probs
        A = action_mask.shape[1]
        action_log_probs = log_probs[:, -A:] * action_mask.float()
        out.log_probs = action_log_probs
        if return_entropy and out.entropy is not None:
            out.entropy = out.entropy[:, -A:]
        return (action_log_probs, out) if return_output else action_log_probs
