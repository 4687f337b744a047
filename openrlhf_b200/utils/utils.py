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
        return tok
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
