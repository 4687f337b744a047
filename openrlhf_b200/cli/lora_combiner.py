"""``python -m openrlhf.cli.lora_combiner``: merge a saved LoRA adapter into its base model and write a plain HF
checkpoint (openrlhf/cli/lora_combiner.py:10-52)."""
from __future__ import annotations

import argparse

from ..models.hf_io import load_pretrained, save_pretrained
from ..models.lora import load_adapter
from ..utils.utils import get_tokenizer
from . import flags as F


def apply_lora(model_name_or_path: str, lora_path: str, output_path: str, is_rm: bool = False,
               value_head_prefix: str = "score", device: str = "cpu"):
    print(f"Loading the base model from {model_name_or_path}")
    model = load_pretrained(model_name_or_path, device=device, with_lm_head=not is_rm, with_value_head=is_rm,
                            value_head_prefix=value_head_prefix)
    print(f"Loading the LoRA adapter from {lora_path}")
    adapters = load_adapter(model, lora_path)
    print("Applying and unloading the LoRA weights")
    adapters.merge_into(model)
    model.lora = None
    tok = get_tokenizer(model_name_or_path, None, "right", None)
    print(f"Saving the target model to {output_path}")
    save_pretrained(model, output_path, tokenizer=tok)


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    F.add_flags(p, [("--model_path", str, None), ("--lora_path", str, None), ("--output_path", str, None),
                    ("--is_rm", F.BOOL, False), ("--ds.param_dtype", str, "bf16"), ("--ds.value_head_prefix", str, "score")])
    a = F.finalize(p)
    apply_lora(a.model_path, a.lora_path, a.output_path, a.is_rm, a.ds.value_head_prefix)
