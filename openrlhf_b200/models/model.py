"""Reward and critic models: the decoder stack with a scalar value head, with the forward contracts of the
reference (openrlhf/models/model.py:204-240 reward, :272-317 critic). The head is stored as
``<value_head_prefix>.weight`` ([1, H], default prefix ``score``) and ``mean`` / ``std`` / ``normalize_reward`` live
in ``config.json`` so HF ``AutoModelForSequenceClassification`` can read the checkpoint.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .config import ModelConfig
from .hf_io import load_pretrained
from .packing import pack_padded, unpack_to_padded
from .transformer import TransformerLM


class _ValueModel(nn.Module):
    def __init__(self, model: TransformerLM, normalize_reward: bool = False, packing_samples: bool = True):
        super().__init__()
        assert model.with_value_head
        self.model = model
        self.cfg: ModelConfig = model.cfg
        self.normalize_reward = normalize_reward or self.cfg.normalize_reward
        self.packing_samples = packing_samples
        self.value_head_prefix = self.cfg.value_head_prefix
        self.register_buffer("mean", torch.tensor([float(self.cfg.mean)]), persistent=False)
        self.register_buffer("std", torch.tensor([float(self.cfg.std)]), persistent=False)

    @property
    def config(self):
        return self.cfg

    def gradient_checkpointing_enable(self, **_kw):
        self.model.gradient_checkpointing = True

    def _token_values(self, input_ids, attention_mask, ring_attn_group=None):
        pb = pack_padded(input_ids, attention_mask)
        if ring_attn_group is not None and input_ids.is_cuda:
            # context parallel: this rank runs its rows of the re-packed stream, values are gathered per token
            if getattr(self, "_cp", None) is None or self._cp.group is not ring_attn_group:
                from ..parallel.cp import ContextParallel

                self._cp = ContextParallel(ring_attn_group)
            v, _ = self._cp.forward_values(self.model, pb)
            return unpack_to_padded(v, pb), None, pb
        h, _ = self.model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        v = self.model.values(h)
        return unpack_to_padded(v, pb), h, pb


class RewardModel(_ValueModel):
    """Scalar reward = value at the last attended token (works for left- and right-padded batches)."""

    def forward(self, input_ids: torch.LongTensor = None, attention_mask: Optional[torch.Tensor] = None,
                return_output: bool = False, ring_attn_group=None, pad_sequence: bool = False, packed_seq_lens=None):
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        last = attention_mask.size(1) - 1 - attention_mask.long().fliplr().argmax(dim=1, keepdim=True)
        values, h, _ = self._token_values(input_ids, attention_mask, ring_attn_group)
        reward = values.gather(1, last).squeeze(1)
        if not self.training and self.normalize_reward:
            reward = (reward - self.mean.to(reward.device)) / self.std.to(reward.device)
        return (reward, {"last_hidden_state": h}) if return_output else reward


class CriticModel(_ValueModel):
    """Per-action values: values[:, :-1], last A columns, times the action mask."""

    def forward(self, input_ids: torch.LongTensor = None, action_mask: Optional[torch.Tensor] = None,
                attention_mask: Optional[torch.Tensor] = None, return_output: bool = False, ring_attn_group=None,
                packed_seq_lens=None):
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        values, h, _ = self._token_values(input_ids, attention_mask, ring_attn_group)
        if action_mask is None:
            assert return_output
            return {"last_hidden_state": h}
        values = values[:, :-1]
        if self.normalize_reward:
            values = (values - self.mean.to(values.device)) / self.std.to(values.device)
        out = values[:, -action_mask.shape[1]:] * action_mask.float()
        return (out, {"last_hidden_state": h}) if return_output else out


def get_llm_for_sequence_regression(model_name_or_path: str, model_type: str, *, param_dtype: str = "bf16",
                                    normalize_reward: bool = False, init_value_head: bool = False,
                                    value_head_prefix: str = "score", device="cuda", packing_samples: bool = True,
                                    shard_world: int = 1, seed: int = 0, load_in_4bit: bool = False,
                                    **_unused) -> nn.Module:
    """Build a reward (``model_type='reward'``) or critic (``'critic'``) model from an HF checkpoint or a preset."""
    if model_type not in ("reward", "critic"):
        raise AssertionError(f"invalid model_type: {model_type}, should be critic or reward.")
    base = load_pretrained(model_name_or_path, device=device, with_lm_head=False, with_value_head=True,
                           shard_world=shard_world, seed=seed, init_value_head=init_value_head,
                           value_head_prefix=value_head_prefix)
    if load_in_4bit:
        from ..ops.nf4 import apply_to_model

        apply_to_model(base)           # projection weights take their NF4 values (openrlhf/models/model.py:96-105)
    cls = RewardModel if model_type == "reward" else CriticModel
    return cls(base, normalize_reward=normalize_reward, packing_samples=packing_samples)
