"""Model configuration: the union of the HF Llama / Qwen2 / Qwen3-MoE config fields this framework's own model
definition needs, with converters from and to ``config.json`` and presets for the benchmark architectures."""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field


@dataclass
class ModelConfig:
    model_type: str = "llama"                 # llama | qwen2 | qwen3 | qwen3_moe | qwen2_vl
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 0                         # 0 -> hidden_size // num_attention_heads
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = False              # bias on q/k/v projections (Qwen2 family)
    qk_norm: bool = False                     # per-head RMSNorm on q and k before RoPE (Qwen3 family)
    # mixture of experts (Qwen3-MoE)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: tuple = ()
    router_aux_loss_coef: float = 0.001
    # sequence-regression heads (reward / critic models)
    value_head_prefix: str = "score"
    normalize_reward: bool = False
    mean: float = 0.0
    std: float = 1.0
    pad_token_id: int = 0
    eos_token_id: int = 2
    bos_token_id: int = 1
    # vision-language models (Qwen2-VL): the tower's config.json section, placeholder token ids, M-RoPE sections
    vision: dict | None = None
    image_token_id: int = -1
    video_token_id: int = -1
    vision_start_token_id: int = -1
    vision_end_token_id: int = -1
    mrope_section: tuple = ()
    extra: dict = field(default_factory=dict)  # unknown config.json keys, preserved on save
    # rows of lm_head.weight held by this model object: 0 = all of the vocabulary; a tensor-parallel training shard
    # with a vocabulary-parallel head holds vocab_size / tp of them (never written to config.json)
    lm_head_vocab: int = 0

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden_size // self.num_attention_heads
        self.mlp_only_layers = tuple(self.mlp_only_layers or ())
        self.mrope_section = tuple(self.mrope_section or ())

    @property
    def is_vlm(self) -> bool:
        return self.vision is not None

    def vision_config(self):
        from .vision import VisionConfig

        return VisionConfig.from_dict(self.vision) if self.vision is not None else None

    # ------------------------------------------------------------------ derived sizes
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    def is_moe_layer(self, idx: int) -> bool:
        return (self.num_experts > 0 and idx not in self.mlp_only_layers
                and (idx + 1) % max(self.decoder_sparse_step, 1) == 0)

    def num_params(self) -> int:
        H, L = self.hidden_size, self.num_hidden_layers
        n = self.vocab_size * H * (1 if self.tie_word_embeddings else 2) + H
        for i in range(L):
            n += self.qkv_size * H + (self.qkv_size if self.attention_bias else 0) + self.q_size * H + 2 * H
            if self.qk_norm:
                n += 2 * self.head_dim
            if self.is_moe_layer(i):
                n += self.num_experts * H + self.num_experts * 3 * self.moe_intermediate_size * H
            else:
                n += 3 * self.intermediate_size * H
        return n

    # ------------------------------------------------------------------ HF interop
    _HF_KEYS = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "rms_norm_eps", "rope_theta", "max_position_embeddings",
                "tie_word_embeddings", "num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                "decoder_sparse_step", "mlp_only_layers", "router_aux_loss_coef", "pad_token_id", "eos_token_id",
                "bos_token_id")

    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        mt = d.get("model_type", "llama")
        vlm = {}
        if mt == "qwen2_vl":
            # the text fields sit in "text_config" (newer files) or at the top level (older files)
            top = d
            d = {**{k: v for k, v in top.items() if k not in ("text_config", "vision_config")},
                 **(top.get("text_config") or {})}
            d["model_type"] = mt
            rs = d.get("rope_scaling") or d.get("rope_parameters") or {}
            vlm = {"vision": dict(top.get("vision_config") or {}), "mrope_section": tuple(rs.get("mrope_section") or ()),
                   **{k: int(top[k]) for k in ("image_token_id", "video_token_id", "vision_start_token_id",
                                                "vision_end_token_id") if top.get(k) is not None}}
            if "tie_word_embeddings" in top and "tie_word_embeddings" not in (top.get("text_config") or {}):
                d["tie_word_embeddings"] = top["tie_word_embeddings"]
        kw = {k: d[k] for k in cls._HF_KEYS if k in d and d[k] is not None}
        kw.update(vlm)
        if isinstance(kw.get("eos_token_id"), (list, tuple)):
            kw["eos_token_id"] = int(kw["eos_token_id"][0])
        rope = d.get("rope_parameters") or {}
        if "rope_theta" not in kw and "rope_theta" in rope:
            kw["rope_theta"] = rope["rope_theta"]
        kw["model_type"] = mt
        kw["head_dim"] = d.get("head_dim") or 0
        kw["attention_bias"] = bool(d.get("attention_bias", mt in ("qwen2", "qwen2_vl")))
        kw["qk_norm"] = mt in ("qwen3", "qwen3_moe")
        for k in ("value_head_prefix", "normalize_reward", "mean", "std"):
            if k in d:
                kw[k] = d[k]
        known = set(kw) | {"model_type", "architectures", "head_dim", "attention_bias", "rope_parameters",
                           "text_config", "vision_config", "rope_scaling"}
        kw["extra"] = {k: v for k, v in d.items() if k not in known}
        return cls(**kw)

    def to_hf_dict(self) -> dict:
        arch = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                "qwen3_moe": "Qwen3MoeForCausalLM"}.get(self.model_type, "LlamaForCausalLM")
        d = dict(self.extra)
        d.update({k: getattr(self, k) for k in self._HF_KEYS})
        d["mlp_only_layers"] = list(self.mlp_only_layers)
        if self.num_experts == 0:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                      "decoder_sparse_step", "mlp_only_layers", "router_aux_loss_coef"):
                d.pop(k, None)
        d.update({"model_type": self.model_type, "architectures": [arch], "head_dim": self.head_dim,
                  "attention_bias": self.attention_bias, "torch_dtype": "bfloat16", "hidden_act": "silu"})
        if self.is_vlm:
            rope = {"type": "mrope", "rope_type": "default", "mrope_section": list(self.mrope_section)}
            text = {k: v for k, v in d.items() if k not in ("architectures", "attention_bias", "head_dim")}
            text.update({"model_type": "qwen2_vl_text", "rope_scaling": rope})
            d = dict(self.extra)
            d.update({"model_type": "qwen2_vl", "architectures": ["Qwen2VLForConditionalGeneration"],
                      "text_config": text, "vision_config": {**self.vision, "model_type": "qwen2_vl"},
                      "image_token_id": self.image_token_id, "video_token_id": self.video_token_id,
                      "vision_start_token_id": self.vision_start_token_id,
                      "vision_end_token_id": self.vision_end_token_id,
                      "tie_word_embeddings": self.tie_word_embeddings, "torch_dtype": "bfloat16",
                      "vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "rope_scaling": rope})
        return d

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        if path in PRESETS:
            return dataclasses.replace(PRESETS[path])
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def save_pretrained(self, path: str, extra: dict | None = None) -> None:
        os.makedirs(path, exist_ok=True)
        d = self.to_hf_dict()
        if extra:
            d.update(extra)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(d, f, indent=2)


PRESETS: dict[str, ModelConfig] = {
    # 2 layers, hidden 64: the CPU oracle architecture
    "tiny-llama": ModelConfig("llama", 1024, 64, 176, 2, 4, 2, rms_norm_eps=1e-6, rope_theta=10000.0),
    # small model with head_dim 128 so that every sm_100a kernel applies
    "tiny-qwen2": ModelConfig("qwen2", 2048, 256, 512, 2, 2, 1, head_dim=128, rope_theta=1e6, attention_bias=True,
                              tie_word_embeddings=True),
    # 4 query / 2 kv heads: divisible by a tensor-parallel size of 2
    "tiny-qwen2-gqa": ModelConfig("qwen2", 2048, 256, 512, 2, 4, 2, head_dim=128, rope_theta=1e6, attention_bias=True),
    "qwen2.5-1.5b": ModelConfig("qwen2", 151936, 1536, 8960, 28, 12, 2, rms_norm_eps=1e-6, rope_theta=1e6,
                                tie_word_embeddings=True, attention_bias=True),
    "qwen2.5-7b": ModelConfig("qwen2", 152064, 3584, 18944, 28, 28, 4, rms_norm_eps=1e-6, rope_theta=1e6,
                              attention_bias=True),
    "qwen2.5-32b": ModelConfig("qwen2", 152064, 5120, 27648, 64, 40, 8, rms_norm_eps=1e-6, rope_theta=1e6,
                               attention_bias=True),
    # vision-language: Qwen2-VL language model + 32-block ViT (patch 14, 2x2 merge), M-RoPE sections (16, 24, 24)
    "qwen2-vl-2b": ModelConfig("qwen2_vl", 151936, 1536, 8960, 28, 12, 2, rms_norm_eps=1e-6, rope_theta=1e6,
                               tie_word_embeddings=True, attention_bias=True, mrope_section=(16, 24, 24),
                               image_token_id=151655, video_token_id=151656, vision_start_token_id=151652,
                               vision_end_token_id=151653, eos_token_id=151645, pad_token_id=151643,
                               vision=dict(depth=32, embed_dim=1280, hidden_size=1536, num_heads=16, mlp_ratio=4,
                                           in_channels=3, patch_size=14, spatial_merge_size=2, temporal_patch_size=2,
                                           hidden_act="quick_gelu")),
    "tiny-qwen2-vl": ModelConfig("qwen2_vl", 2048, 256, 512, 2, 2, 1, head_dim=128, rope_theta=1e6,
                                 attention_bias=True, mrope_section=(16, 24, 24), image_token_id=2040,
                                 video_token_id=2041, vision_start_token_id=2042, vision_end_token_id=2043,
                                 vision=dict(depth=2, embed_dim=128, hidden_size=256, num_heads=4, mlp_ratio=2,
                                             in_channels=3, patch_size=14, spatial_merge_size=2,
                                             temporal_patch_size=2, hidden_act="quick_gelu")),
    "llama3-8b": ModelConfig("llama", 128256, 4096, 14336, 32, 32, 8, rms_norm_eps=1e-5, rope_theta=500000.0),
    "qwen3-30b-a3b": ModelConfig("qwen3_moe", 151936, 2048, 6144, 48, 32, 4, head_dim=128, rms_norm_eps=1e-6,
                                 rope_theta=1e6, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                                 norm_topk_prob=True, qk_norm=True),
    "tiny-qwen3-moe": ModelConfig("qwen3_moe", 1024, 128, 256, 2, 2, 1, head_dim=128, rope_theta=1e6, num_experts=8,
                                  num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True, qk_norm=True),
}
