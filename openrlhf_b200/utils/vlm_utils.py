"""Vision-language helpers: image loading (path / URL / base64 / bytes / PIL), processor tokenisation of prompts with
images, de-duplication of expanded media pad tokens, and merging of per-sample multimodal training inputs
(openrlhf/utils/vlm_utils.py:18-170). The language side of this framework is text-only; these helpers keep the data
path and the agent API working for processors that accept images."""
from __future__ import annotations

import base64
import io
import logging
import re
from typing import Any, Dict, List, Optional, Union

import torch

logger = logging.getLogger(__name__)


def _is_base64_image(s: str) -> bool:
    if s.startswith("data:image"):
        return True
    return len(s) > 256 and re.fullmatch(r"[A-Za-z0-9+/=\s]+", s[:512]) is not None


def load_images(image_refs: Union[str, List[Any], Any]) -> list:
    """Accepts one reference or a list; broken items are skipped with a warning."""
    from PIL import Image

    if image_refs is None:
        return []
    if not isinstance(image_refs, (list, tuple)):
        image_refs = [image_refs]
    out = []
    for ref in image_refs:
        try:
            if isinstance(ref, Image.Image):
                img = ref
            elif isinstance(ref, (bytes, bytearray)):
                img = Image.open(io.BytesIO(ref))
            elif isinstance(ref, dict) and "bytes" in ref:
                img = Image.open(io.BytesIO(ref["bytes"]))
            elif isinstance(ref, str) and ref.startswith(("http://", "https://")):
                import requests

                img = Image.open(io.BytesIO(requests.get(ref, timeout=30).content))
            elif isinstance(ref, str) and _is_base64_image(ref):
                img = Image.open(io.BytesIO(base64.b64decode(ref.split(",", 1)[-1])))
            else:
                img = Image.open(ref)
            out.append(img.convert("RGB"))
        except Exception as e:  # noqa: BLE001
            logger.warning("skipping an image that failed to load: %s", e)
    return out


def process_prompt_with_images(processor, prompt: str, images):
    """Returns (token ids, multimodal training inputs dict or None, PIL images)."""
    pil = load_images(images)
    if not pil:
        ids = processor.tokenizer(prompt, add_special_tokens=False)["input_ids"]
        return list(ids), None, []
    enc = processor(text=[prompt], images=pil, return_tensors="pt", add_special_tokens=False)
    ids = enc["input_ids"][0].tolist()
    mm = {k: v for k, v in enc.items() if k not in ("input_ids", "attention_mask")}
    return ids, mm, pil


def dedup_media_tokens(token_ids: List[int], pad_token_ids: set) -> List[int]:
    """Collapse runs of the same media pad token to a single token (the generation engine re-expands them)."""
    out: List[int] = []
    for t in token_ids:
        if out and t in pad_token_ids and out[-1] == t:
            continue
        out.append(t)
    return out


def accumulate_mm_inputs(existing: Optional[Dict], new: Optional[Dict]) -> Optional[Dict]:
    if new is None:
        return existing
    if existing is None:
        return dict(new)
    out = dict(existing)
    for k, v in new.items():
        out[k] = torch.cat([out[k], v], dim=0) if k in out and isinstance(v, torch.Tensor) else v
    return out


def merge_mm_train_inputs(mm_train_inputs_list: list, device) -> Dict[str, torch.Tensor]:
    merged: Dict[str, list] = {}
    for mm in mm_train_inputs_list:
        if not mm:
            continue
        for k, v in mm.items():
            merged.setdefault(k, []).append(v)
    return {k: torch.cat(v, dim=0).to(device) for k, v in merged.items() if isinstance(v[0], torch.Tensor)}
