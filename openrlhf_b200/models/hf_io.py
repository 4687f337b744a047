"""HF-format checkpoint I/O for this framework's own model definition.

On disk: standard HF safetensors shards + ``model.safetensors.index.json`` + ``config.json`` with the HF parameter
names (separate q/k/v and gate/up projections, per-expert MoE tensors, ``lm_head.weight`` omitted when tied,
``<value_head_prefix>.weight`` for reward / critic models), so checkpoints load in ``transformers`` and vice versa.
In memory: fused ``qkv`` / ``gate_up`` views of one flat buffer. This module converts between the two.
It covers what ``DeepspeedStrategy.save_model`` does in the reference (openrlhf/utils/deepspeed/deepspeed.py:533-591)
and the value-head conventions of openrlhf/models/model.py:70-82,183-198.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Iterator

import torch

from .config import PRESETS, ModelConfig
from .transformer import TransformerLM

MAX_SHARD_BYTES = 5 * 1024 ** 3


def hf_names_for(cfg: ModelConfig, name: str) -> list[tuple[str, tuple | None]]:
    """Internal parameter name -> [(hf_name, row slice or expert selector)].

    A selector is None (whole tensor), ("rows", a, b) for a row range of a fused matrix / bias, or
    ("expert", e, a, b) for rows [a, b) of expert e of a fused 3-D tensor.
    """
    if name.startswith("visual."):
        # vision tower (Qwen2-VL): same names under "model."; the patch embedding is stored as a Conv3d kernel
        if name == "visual.patch_embed.weight":
            v = cfg.vision_config()
            return [("model.visual.patch_embed.proj.weight",
                     ("view", (v.embed_dim, v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)))]
        return [("model." + name, None)]
    if cfg.is_vlm and name not in ("lm_head.weight", "value_head.weight"):
        # the language model of a vision-language checkpoint lives under "model.language_model."
        plain = dataclasses.replace(cfg, vision=None)
        return [(("model.language_model." + n[len("model."):]) if n.startswith("model.") else n, sel)
                for n, sel in hf_names_for(plain, name)]
    if name == "embed.weight":
        return [("model.embed_tokens.weight", None)]
    if name == "norm.weight":
        return [("model.norm.weight", None)]
    if name == "lm_head.weight":
        return [("lm_head.weight", None)]
    if name == "value_head.weight":
        return [(f"{cfg.value_head_prefix}.weight", None)]
    _, li, rest = name.split(".", 2)
    pre = f"model.layers.{li}."
    q, kv = cfg.q_size, cfg.kv_size
    if rest in ("qkv.weight", "qkv.bias"):
        kind = rest.split(".")[1]
        return [(pre + f"self_attn.q_proj.{kind}", ("rows", 0, q)),
                (pre + f"self_attn.k_proj.{kind}", ("rows", q, q + kv)),
                (pre + f"self_attn.v_proj.{kind}", ("rows", q + kv, q + 2 * kv))]
    simple = {"norm1.weight": "input_layernorm.weight", "norm2.weight": "post_attention_layernorm.weight",
              "o.weight": "self_attn.o_proj.weight", "q_norm.weight": "self_attn.q_norm.weight",
              "k_norm.weight": "self_attn.k_norm.weight", "down.weight": "mlp.down_proj.weight",
              "router.weight": "mlp.gate.weight"}
    if rest in simple:
        return [(pre + simple[rest], None)]
    if rest == "gate_up.weight":
        F = cfg.intermediate_size
        return [(pre + "mlp.gate_proj.weight", ("rows", 0, F)), (pre + "mlp.up_proj.weight", ("rows", F, 2 * F))]
    if rest == "experts.gate_up":
        I = cfg.moe_intermediate_size
        out = []
        for e in range(cfg.num_experts):
            out.append((pre + f"mlp.experts.{e}.gate_proj.weight", ("expert", e, 0, I)))
            out.append((pre + f"mlp.experts.{e}.up_proj.weight", ("expert", e, I, 2 * I)))
        return out
    if rest == "experts.down":
        return [(pre + f"mlp.experts.{e}.down_proj.weight", ("expert", e, 0, cfg.hidden_size))
                for e in range(cfg.num_experts)]
    raise KeyError(name)


def _alternate_names(hf_name: str) -> list[str]:
    """Other spellings of a tensor name found in the wild: checkpoints saved from a bare base model (no "model."
    prefix) and vision-language checkpoints written before the language model moved under "model.language_model."."""
    alts = []
    if hf_name.startswith("model.language_model."):
        alts.append("model." + hf_name[len("model.language_model."):])
    if hf_name.startswith("model.visual."):
        alts.append(hf_name[len("model."):])
    if hf_name.startswith("model."):
        alts.append(hf_name[len("model."):])
    return alts


def _select(t: torch.Tensor, sel):
    if sel is None:
        return t
    if sel[0] == "rows":
        return t[sel[1]:sel[2]]
    if sel[0] == "view":
        return t.reshape(sel[1])
    return t[sel[1], sel[2]:sel[3]]


def iter_hf_tensors(model: TransformerLM) -> Iterator[tuple[str, torch.Tensor]]:
    z3 = getattr(model, "z3", None)
    tpt = getattr(model, "tp_train", None)
    if tpt is not None:
        # tensor-parallel shard: rebuild the full fused layout from all shards and name it with the full configuration
        from .transformer import build_param_specs

        full = tpt.gather_full(model)
        for spec in build_param_specs(tpt.full_cfg, model.with_lm_head, model.with_value_head):
            t = full[spec.offset:spec.offset + spec.numel].view(spec.shape)
            for hf_name, sel in hf_names_for(tpt.full_cfg, spec.name):
                yield hf_name, _select(t, sel)
        return
    full = z3.gather_full() if z3 is not None else None     # ZeRO-3: parameters are sharded, gather the logical buffer
    for spec, p in model.named_specs():
        t = p.detach() if full is None else full[spec.offset:spec.offset + spec.numel].view(spec.shape)
        for hf_name, sel in hf_names_for(model.cfg, spec.name):
            yield hf_name, _select(t, sel)


def hf_state_dict(model: TransformerLM) -> dict[str, torch.Tensor]:
    return {k: v for k, v in iter_hf_tensors(model)}


@torch.no_grad()
def save_pretrained(model: TransformerLM, path: str, tokenizer=None, extra_config: dict | None = None,
                    rank: int = 0, world: int = 1, max_shard_bytes: int = MAX_SHARD_BYTES) -> None:
    """Write HF safetensors shards. With world > 1 every rank writes the shards whose index is congruent to its rank
    (all ranks hold the full bf16 parameters), rank 0 writes the index, config and tokenizer."""
    from ..utils.st_io import available as _native_st, save_file as _native_save

    if _native_st():
        save_file = _native_save          # parallel native writer, same file format
    else:
        from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards: list[list[tuple[str, torch.Tensor]]] = [[]]
    size = 0
    for name, t in iter_hf_tensors(model):
        nbytes = t.numel() * t.element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append([])
            size = 0
        shards[-1].append((name, t))
        size += nbytes
    n = len(shards)
    index = {"metadata": {"total_size": 0}, "weight_map": {}}
    for i, shard in enumerate(shards):
        fname = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
        for name, t in shard:
            index["weight_map"][name] = fname
            index["metadata"]["total_size"] += t.numel() * t.element_size()
        if i % world == rank:
            save_file({name: t.contiguous().cpu() for name, t in shard}, os.path.join(path, fname),
                      metadata={"format": "pt"})
    if rank == 0:
        if n > 1:
            with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
                json.dump(index, f, indent=2)
        extra = dict(extra_config or {})
        if model.with_value_head:
            extra.setdefault("value_head_prefix", model.cfg.value_head_prefix)
            extra.setdefault("normalize_reward", model.cfg.normalize_reward)
            extra.setdefault("mean", model.cfg.mean)
            extra.setdefault("std", model.cfg.std)
        tpt = getattr(model, "tp_train", None)
        (tpt.full_cfg if tpt is not None else model.cfg).save_pretrained(path, extra)
        if tokenizer is not None:
            tokenizer.save_pretrained(path)


def _open_shards(path: str):
    from safetensors import safe_open

    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        files = sorted(set(wm.values()))
    else:
        files = [f for f in sorted(os.listdir(path)) if f.endswith(".safetensors")]
        wm = None
    handles = {fn: safe_open(os.path.join(path, fn), framework="pt", device="cpu") for fn in files}
    if wm is None:
        wm = {k: fn for fn, h in handles.items() for k in h.keys()}
    return wm, handles


@torch.no_grad()
def load_weights(model: TransformerLM, path: str, strict: bool = True) -> list[str]:
    """Fill the model's flat buffer from an HF checkpoint directory. Returns the list of missing HF tensors
    (a missing value head is tolerated when strict is False so a critic can start from a policy checkpoint)."""
    wm, handles = _open_shards(path)
    missing = []
    for spec, p in model.named_specs():
        for hf_name, sel in hf_names_for(model.cfg, spec.name):
            src_name = hf_name
            for alt in _alternate_names(hf_name):
                if src_name in wm:
                    break
                if alt in wm:
                    src_name = alt
            if src_name not in wm:
                tied = [n for n in ("model.embed_tokens.weight", "model.language_model.embed_tokens.weight") if n in wm]
                if hf_name == "lm_head.weight" and tied:
                    src_name = tied[0]
                else:
                    missing.append(hf_name)
                    continue
            t = handles[wm[src_name]].get_tensor(src_name)
            _select(p, sel).copy_(t.to(p.dtype))
    hard = [m for m in missing if not m.startswith(model.cfg.value_head_prefix + ".")]
    if hard and strict:
        raise KeyError(f"checkpoint {path} lacks tensors: {hard[:8]}{'...' if len(hard) > 8 else ''}")
    return missing


def load_pretrained(path_or_preset: str, device="cuda", with_lm_head: bool = True, with_value_head: bool = False,
                    shard_world: int = 1, seed: int = 0, init_value_head: bool = False,
                    value_head_prefix: str | None = None) -> TransformerLM:
    """Build a model from an HF checkpoint directory, or random-init it from an architecture preset name
    (``qwen2.5-1.5b``, ``llama3-8b``, ...; presets exist because the benchmark machines have no network)."""
    if path_or_preset in PRESETS:
        cfg = ModelConfig.from_pretrained(path_or_preset)
        if value_head_prefix:
            cfg.value_head_prefix = value_head_prefix
        return TransformerLM(cfg, device=device, with_lm_head=with_lm_head, with_value_head=with_value_head,
                             seed=seed, shard_world=shard_world)
    cfg = ModelConfig.from_pretrained(path_or_preset)
    if value_head_prefix:
        cfg.value_head_prefix = value_head_prefix
    model = TransformerLM(cfg, device=device, with_lm_head=with_lm_head, with_value_head=with_value_head, seed=None,
                          shard_world=shard_world)
    if with_value_head:
        g = torch.Generator(device="cpu").manual_seed(seed)
        vh = model.p("value_head.weight")
        vh.data.copy_((torch.randn(vh.shape, generator=g) / (cfg.hidden_size + 1) ** 0.5).to(vh.dtype))
    missing = load_weights(model, path_or_preset, strict=False)
    hard = [m for m in missing if not m.startswith(cfg.value_head_prefix + ".")]
    if hard:
        raise KeyError(f"checkpoint {path_or_preset} lacks tensors: {hard[:8]}")
    if with_value_head and missing and not init_value_head:
        import logging

        logging.getLogger(__name__).warning("value head not found in %s: initialised N(0, 1/(hidden+1))", path_or_preset)
    return model
