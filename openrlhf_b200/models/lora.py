"""Low-rank adapters on the fused projections of this framework's model (the reference uses PEFT:
openrlhf/models/actor.py:176-198; adapter-only saving at openrlhf/utils/deepspeed/deepspeed.py:564-574).

``y = x W^T + (alpha / r) * (x A^T) B^T`` with A [r, in] ~ N(0, 1/r-scaled Kaiming), B [out, r] = 0. Adapters live in
their own small flat buffer (so the ZeRO engine can own them while the base weights stay frozen), are saved in the
PEFT file layout (``adapter_model.safetensors`` + ``adapter_config.json``) and can be merged into the base weights.
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.nn as nn

from ..ops import functional as F

TARGETS = {"q_proj": "qkv", "k_proj": "qkv", "v_proj": "qkv", "o_proj": "o", "gate_proj": "gate_up",
           "up_proj": "gate_up", "down_proj": "down"}


class LoraAdapters(nn.Module):
    def __init__(self, model, rank: int, alpha: float = 16, target_modules="all-linear", dropout: float = 0.0,
                 seed: int = 0):
        super().__init__()
        self.rank, self.alpha, self.dropout = rank, alpha, dropout
        self.scale = alpha / rank
        cfg = model.cfg
        if target_modules in ("all-linear", ["all-linear"], None):
            fused = {"qkv", "o", "gate_up", "down"}
        else:
            fused = {TARGETS.get(t, t) for t in target_modules}
        self.targets = sorted(fused)
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.A, self.B = nn.ParameterDict(), nn.ParameterDict()
        dev, dt = model.flat.device, model.flat.dtype
        for i in range(cfg.num_hidden_layers):
            for t in self.targets:
                name = f"layers.{i}.{t}.weight"
                if name not in model._params:
                    continue
                out_f, in_f = model.p(name).shape
                key = f"{i}_{t}"
                a = torch.randn(rank, in_f, generator=g) * (1.0 / math.sqrt(in_f))
                self.A[key] = nn.Parameter(a.to(dev, dt))
                self.B[key] = nn.Parameter(torch.zeros(out_f, rank, device=dev, dtype=dt))
        for p in model.parameters():
            p.requires_grad_(False)
        model.lora = self

    def delta(self, layer: int, target: str, x: torch.Tensor):
        key = f"{layer}_{target}"
        if key not in self.A:
            return None
        if self.dropout and self.training:
            x = torch.nn.functional.dropout(x, self.dropout)
        return (x @ self.A[key].t()) @ self.B[key].t() * self.scale

    @torch.no_grad()
    def merge_into(self, model, sign: float = 1.0):
        """W += sign * scale * B A for every adapted matrix (sign = -1 un-merges)."""
        for key in self.A:
            i, t = key.split("_", 1)
            w = model.p(f"layers.{i}.{t}.weight")
            w.add_((self.B[key].float() @ self.A[key].float() * (sign * self.scale)).to(w.dtype))

    def peft_state_dict(self, cfg) -> dict:
        """PEFT key names on the HF module names (fused matrices are split back into q/k/v and gate/up rows)."""
        sd = {}
        q, kv, Fi = cfg.q_size, cfg.kv_size, cfg.intermediate_size
        rows = {"qkv": [("self_attn.q_proj", 0, q), ("self_attn.k_proj", q, q + kv), ("self_attn.v_proj", q + kv, q + 2 * kv)],
                "o": [("self_attn.o_proj", None, None)], "down": [("mlp.down_proj", None, None)],
                "gate_up": [("mlp.gate_proj", 0, Fi), ("mlp.up_proj", Fi, 2 * Fi)]}
        for key in self.A:
            i, t = key.split("_", 1)
            for mod, a, b in rows[t]:
                base = f"base_model.model.model.layers.{i}.{mod}"
                sd[base + ".lora_A.weight"] = self.A[key].detach().cpu().clone().contiguous()
                Bm = self.B[key].detach()
                sd[base + ".lora_B.weight"] = (Bm if a is None else Bm[a:b]).cpu().clone().contiguous()
        return sd

    def save_adapter(self, path: str):
        from safetensors.torch import save_file

        os.makedirs(path, exist_ok=True)
        cfg = getattr(self, "_cfg", None)
        save_file(self.peft_state_dict(cfg), os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
        tm = sorted({m for t in self.targets for m, v in TARGETS.items() if v == t})
        with open(os.path.join(path, "adapter_config.json"), "w") as f:
            json.dump({"peft_type": "LORA", "r": self.rank, "lora_alpha": self.alpha, "lora_dropout": self.dropout,
                       "target_modules": tm, "bias": "none", "task_type": "CAUSAL_LM"}, f, indent=2)


def load_adapter(model, path: str) -> LoraAdapters:
    from safetensors.torch import load_file

    with open(os.path.join(path, "adapter_config.json")) as f:
        c = json.load(f)
    ad = LoraAdapters(model, c["r"], c["lora_alpha"], c["target_modules"], c.get("lora_dropout", 0.0))
    ad._cfg = model.cfg
    sd = load_file(os.path.join(path, "adapter_model.safetensors"))
    cfg = model.cfg
    for key in ad.A:
        i, t = key.split("_", 1)
        first = {"qkv": "self_attn.q_proj", "o": "self_attn.o_proj", "down": "mlp.down_proj", "gate_up": "mlp.gate_proj"}[t]
        base = f"base_model.model.model.layers.{i}."
        ad.A[key].data.copy_(sd[base + first + ".lora_A.weight"].to(ad.A[key].dtype))
        parts = {"qkv": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], "o": ["self_attn.o_proj"],
                 "down": ["mlp.down_proj"], "gate_up": ["mlp.gate_proj", "mlp.up_proj"]}[t]
        ad.B[key].data.copy_(torch.cat([sd[base + m + ".lora_B.weight"] for m in parts], 0).to(ad.B[key].dtype))
    return ad
