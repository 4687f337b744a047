"""Tokenizer / dtype / padding helpers with the reference's names (openrlhf/utils/utils.py:8-122)."""
from __future__ import annotations

from typing import List

import torch

from ..rl.experience import pad_stack
from .strategy import get_strategy  # noqa: F401  (re-exported: ``from openrlhf.utils import get_strategy``)


def convert_to_torch_dtype(param_dtype: str) -> torch.dtype:
    table = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
             "fp32": torch.float32, "float32": torch.float32}
    if param_dtype not in table:
        raise ValueError(f"unsupported param dtype {param_dtype}")
    return table[param_dtype]


def is_vlm_model(pretrain: str) -> bool:
    """True when the checkpoint's HF config has a vision tower."""
    try:
        from transformers import AutoConfig

        return hasattr(AutoConfig.from_pretrained(pretrain, trust_remote_code=True), "vision_config")
    except Exception:  # noqa: BLE001
        return False


class SyntheticTokenizer:
    """Whitespace-free integer tokenizer for architecture presets (no tokenizer files exist for random-init
    benchmark models): text is a space-separated list of token ids."""

    def __init__(self, vocab_size: int, eos_token_id: int = 2, pad_token_id: int = 0):
        self.vocab_size, self.eos_token_id, self.pad_token_id = vocab_size, eos_token_id, pad_token_id
        self.eos_token, self.pad_token = str(eos_token_id), str(pad_token_id)
        self.padding_side = "left"
        self.chat_template = None

    def _enc(self, text: str) -> list[int]:
        out = []
        for w in text.split():
            try:
                out.append(int(w) % self.vocab_size)
            except ValueError:
                out.append(sum(w.encode()) % self.vocab_size)
        return out

    def __call__(self, text=None, add_special_tokens=False, return_tensors=None, max_length=None, truncation=False,
                 padding=False, **_kw):
        single = isinstance(text, str)
        texts = [text] if single else list(text)
        ids = [self._enc(t) for t in texts]
        if truncation and max_length:
            ids = [x[:max_length] for x in ids]
        if return_tensors == "pt":
            width = max((len(x) for x in ids), default=0)
            mat = torch.full((len(ids), width), self.pad_token_id, dtype=torch.long)
            att = torch.zeros((len(ids), width), dtype=torch.long)
            for i, x in enumerate(ids):
                if self.padding_side == "left":
                    mat[i, width - len(x):] = torch.tensor(x, dtype=torch.long)
                    att[i, width - len(x):] = 1
                else:
                    mat[i, :len(x)] = torch.tensor(x, dtype=torch.long)
                    att[i, :len(x)] = 1
            return {"input_ids": mat, "attention_mask": att}
        return {"input_ids": ids[0] if single else ids,
                "attention_mask": [1] * len(ids[0]) if single else [[1] * len(x) for x in ids]}

    def encode(self, text, add_special_tokens=False):
        return self._enc(text)

    def decode(self, ids, skip_special_tokens=False):
        ids = ids.tolist() if hasattr(ids, "tolist") else ids
        return " ".join(str(int(i)) for i in ids)

    def batch_decode(self, seqs, skip_special_tokens=False):
        return [self.decode(s, skip_special_tokens) for s in seqs]

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=False, **_kw):
        text = " ".join(m["content"] if isinstance(m, dict) else str(m) for m in messages)
        return self._enc(text) if tokenize else text

    def save_pretrained(self, path):
        import json
        import os

        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "synthetic_tokenizer.json"), "w") as f:
            json.dump({"vocab_size": self.vocab_size, "eos_token_id": self.eos_token_id,
                       "pad_token_id": self.pad_token_id}, f)


class SyntheticImageProcessor:
    """Image -> flattened patches in the Qwen2-VL order (merge x merge neighbours adjacent, temporal patch made of
    the frame repeated), without files: sides are rounded to a multiple of patch * merge, pixels scaled to [-1, 1]."""

    def __init__(self, patch_size=14, merge_size=2, temporal_patch_size=2, max_side=448):
        self.patch_size, self.merge_size, self.temporal_patch_size, self.max_side = (
            patch_size, merge_size, temporal_patch_size, max_side)

    def _one(self, img):
        import numpy as np

        P, m, Tp = self.patch_size, self.merge_size, self.temporal_patch_size
        unit = P * m
        w, h = img.size
        gh = max(1, min(round(h / unit), self.max_side // unit)) * m
        gw = max(1, min(round(w / unit), self.max_side // unit)) * m
        arr = np.asarray(img.convert("RGB").resize((gw * P, gh * P)), dtype=np.float32) / 127.5 - 1.0
        x = torch.from_numpy(arr).permute(2, 0, 1)                                   # [C, H, W]
        x = x[None].repeat(Tp, 1, 1, 1)                                              # [Tp, C, H, W]
        x = x.view(Tp, 3, gh // m, m, P, gw // m, m, P).permute(2, 5, 3, 6, 1, 0, 4, 7)
        return x.reshape(gh * gw, 3 * Tp * P * P), (1, gh, gw)

    def __call__(self, images, return_tensors="pt", **_kw):
        outs = [self._one(im) for im in images]
        return {"pixel_values": torch.cat([o[0] for o in outs]),
                "image_grid_thw": torch.tensor([o[1] for o in outs], dtype=torch.long)}


class SyntheticProcessor:
    """Processor for vision-language presets: SyntheticTokenizer for the text, SyntheticImageProcessor for the images;
    every ``<image>`` tag in the text becomes vision_start + one placeholder per merged patch + vision_end."""

    def __init__(self, tokenizer: SyntheticTokenizer, cfg):
        v = cfg.vision_config()
        self.tokenizer = tokenizer
        self.image_processor = SyntheticImageProcessor(v.patch_size, v.spatial_merge_size, v.temporal_patch_size)
        self.image_token_id, self.video_token_id = cfg.image_token_id, cfg.video_token_id
        self.vision_start_token_id, self.vision_end_token_id = cfg.vision_start_token_id, cfg.vision_end_token_id
        self.merge = v.spatial_merge_size
        for attr in ("pad_token", "pad_token_id", "eos_token", "eos_token_id", "vocab_size", "chat_template"):
            setattr(self, attr, getattr(tokenizer, attr))

    @property
    def padding_side(self):
        return self.tokenizer.padding_side

    @padding_side.setter
    def padding_side(self, v):
        self.tokenizer.padding_side = v

    def __call__(self, text=None, images=None, return_tensors=None, **kw):
        if not images:
            return self.tokenizer(text=text, return_tensors=return_tensors, **kw)
        texts = [text] if isinstance(text, str) else list(text)
        enc = self.image_processor(images)
        grids = enc["image_grid_thw"].tolist()
        rows, gi = [], 0
        for t in texts:
            ids = []
            for k, piece in enumerate(t.split("<image>")):
                if k:
                    tt, gh, gw = grids[gi]
                    gi += 1
                    ids += ([self.vision_start_token_id] + [self.image_token_id] * (tt * gh * gw // self.merge ** 2)
                            + [self.vision_end_token_id])
                ids += self.tokenizer._enc(piece)
            rows.append(ids)
        assert gi == len(grids), f"{len(grids)} images for {gi} <image> tags"
        assert len(rows) == 1 or return_tensors != "pt", "batched image prompts are tokenised one at a time"
        out = {"input_ids": torch.tensor(rows, dtype=torch.long) if return_tensors == "pt" else rows,
               "attention_mask": torch.ones(1, len(rows[0]), dtype=torch.long) if return_tensors == "pt"
               else [[1] * len(r) for r in rows]}
        out.update(enc)
        return out

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=False, **kw):
        parts = []
        for m in messages:
            c = m["content"] if isinstance(m, dict) else m
            if isinstance(c, list):
                c = " ".join("<image>" if p.get("type") == "image" else p.get("text", "") for p in c)
            parts.append(str(c))
        text = " ".join(parts)
        return self.tokenizer._enc(text) if tokenize else text

    def decode(self, ids, skip_special_tokens=False):
        return self.tokenizer.decode(ids, skip_special_tokens)

    def batch_decode(self, seqs, skip_special_tokens=False):
        return self.tokenizer.batch_decode(seqs, skip_special_tokens)

    def encode(self, text, add_special_tokens=False):
        return self.tokenizer.encode(text)

    def save_pretrained(self, path):
        self.tokenizer.save_pretrained(path)


def get_tokenizer(pretrain, model=None, padding_side="left", strategy=None, use_fast=True):
    """HF tokenizer (or processor for VLMs) with pad = eos when no pad token exists; architecture presets and
    checkpoints without tokenizer files get the synthetic integer tokenizer."""
    import os

    from ..models.config import PRESETS

    if pretrain in PRESETS or (os.path.isdir(pretrain) and os.path.exists(os.path.join(pretrain, "synthetic_tokenizer.json"))
                               and not os.path.exists(os.path.join(pretrain, "tokenizer_config.json"))):
        cfg = PRESETS.get(pretrain)
        if cfg is None:
            from ..models.config import ModelConfig

            cfg = ModelConfig.from_pretrained(pretrain)
        tok = SyntheticTokenizer(cfg.vocab_size, cfg.eos_token_id, cfg.pad_token_id)
        tok.padding_side = padding_side
        return SyntheticProcessor(tok, cfg) if cfg.is_vlm else tok
    is_vlm = getattr(model, "is_vlm", False) if model is not None else is_vlm_model(pretrain)
    if is_vlm:
        from transformers import AutoProcessor

        tok = AutoProcessor.from_pretrained(pretrain, trust_remote_code=True)
        inner = tok.tokenizer
        inner.padding_side = padding_side
        if inner.pad_token is None:
            inner.pad_token, inner.pad_token_id = inner.eos_token, inner.eos_token_id
        for attr in ("pad_token", "pad_token_id", "eos_token", "eos_token_id"):
            setattr(tok, attr, getattr(inner, attr))
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(pretrain, trust_remote_code=True, use_fast=use_fast)
        tok.padding_side = padding_side
        if tok.pad_token is None:
            tok.pad_token, tok.pad_token_id = tok.eos_token, tok.eos_token_id
    cfg = getattr(model, "config", None) or getattr(model, "cfg", None)
    if cfg is not None and tok.pad_token_id is not None:
        cfg.pad_token_id = tok.pad_token_id
    return tok


def convert_token_to_id(token, tokenizer):
    if not isinstance(token, str):
        raise ValueError("token should be int or str")
    ids = tokenizer.encode(token, add_special_tokens=False)
    assert len(ids) == 1
    return ids[0]


def zero_pad_sequences(sequences: List[torch.Tensor], side: str = "left", value: int = 0, stack: bool = False):
    return pad_stack(list(sequences), side, value, stack)


def remove_pad_token(input_ids: torch.Tensor, attention_mask: torch.Tensor):
    """Per-row token tensors with the padding (left or right) removed."""
    return [ids[mask.bool()] for ids, mask in zip(input_ids, attention_mask)]


def get_strategy(args):
    """The strategy object of a parsed flag namespace (the reference exposes it from this module:
    openrlhf/utils/utils.py); built in utils/strategy.py."""
    from .strategy import get_strategy as build

    return build(args)
