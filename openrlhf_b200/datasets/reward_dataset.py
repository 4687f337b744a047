"""Preference-pair dataset for reward-model and DPO training (openrlhf/datasets/reward_dataset.py:48-200): chosen /
rejected (+ margin), forced EOS, left padding for the reward model (value read at the last token), right padding
for DPO (``extra`` = prompt length)."""
from __future__ import annotations

from typing import Callable

from torch.utils.data import Dataset

from ..rl.experience import pad_stack
from .utils import exist_and_not_none


def preprocess_data(data, input_template=None, prompt_key=None, chosen_key="chosen", rejected_key="rejected",
                    apply_chat_template=None, is_dpo=False):
    if apply_chat_template:
        if prompt_key:
            prompt = apply_chat_template(data[prompt_key], tokenize=False, add_generation_prompt=True)
            chosen = apply_chat_template(data[prompt_key] + data[chosen_key], tokenize=False)[len(prompt):]
            rejected = apply_chat_template(data[prompt_key] + data[rejected_key], tokenize=False)[len(prompt):]
        else:
            prompt = ""
            chosen = apply_chat_template(data[chosen_key], tokenize=False)
            rejected = apply_chat_template(data[rejected_key], tokenize=False)
            if is_dpo:
                prompt = apply_chat_template(data[chosen_key][:-1], tokenize=False, add_generation_prompt=True)
                chosen, rejected = chosen[len(prompt):], rejected[len(prompt):]
    else:
        prompt = data[prompt_key] if prompt_key else ""
        if prompt_key and input_template:
            prompt = input_template.format(prompt)
        chosen, rejected = data[chosen_key], data[rejected_key]
    return prompt, chosen, rejected, (data["margin"] if exist_and_not_none(data, "margin") else 0)


class RewardDataset(Dataset):
    def __init__(self, dataset, tokenizer: Callable, max_length: int, strategy, input_template=None, is_dpo=False,
                 num_processors: int = 8) -> None:
        super().__init__()
        self.is_dpo, self.tokenizer, self.strategy, self.max_length = is_dpo, tokenizer, strategy, max_length
        self.input_template = input_template
        d = strategy.args.data
        self.prompt_key = getattr(d, "prompt_key", None)
        self.chosen_key, self.rejected_key = getattr(d, "chosen_key", None), getattr(d, "rejected_key", None)
        self.apply_chat_template = None
        if getattr(d, "apply_chat_template", False):
            self.apply_chat_template = tokenizer.apply_chat_template
            if getattr(d, "tokenizer_chat_template", None):
                tokenizer.chat_template = d.tokenizer_chat_template
        rows = dataset.map(self.process_data, remove_columns=dataset.column_names, num_proc=num_processors)
        rows = rows.filter(lambda x: x["prompt"] is not None)
        self.prompts, self.chosens, self.rejects, self.extras = rows["prompt"], rows["chosen"], rows["reject"], rows["extra"]

    def _tok(self, text):
        return self.tokenizer(text, max_length=self.max_length, padding=False, truncation=True, return_tensors="pt",
                              add_special_tokens=False)

    def process_data(self, data):
        prompt, chosen, reject, margin = preprocess_data(data, self.input_template, self.prompt_key, self.chosen_key,
                                                         self.rejected_key, self.apply_chat_template, self.is_dpo)
        extra = margin
        if self.is_dpo:
            extra = int(self._tok(prompt)["attention_mask"].int().sum().item())
            if extra >= self.max_length - 2:
                prompt = None
        return {"prompt": prompt, "chosen": chosen, "reject": reject, "extra": extra}

    def __len__(self):
        return len(self.chosens)

    def _encode_with_eos(self, text):
        text = text.rstrip("\n")
        if not text.endswith(self.tokenizer.eos_token):
            text += " " + self.tokenizer.eos_token
        t = self._tok(text)
        t["input_ids"][0][-1] = self.tokenizer.eos_token_id
        t["attention_mask"][0][-1] = True
        return t

    def __getitem__(self, idx):
        c = self._encode_with_eos(self.prompts[idx] + self.chosens[idx])
        r = self._encode_with_eos(self.prompts[idx] + self.rejects[idx])
        return c["input_ids"], c["attention_mask"], r["input_ids"], r["attention_mask"], self.extras[idx]

    def collate_fn(self, item_list):
        c_ids, c_m, r_ids, r_m, extras = zip(*item_list)
        side = "right" if self.is_dpo else "left"
        pad = self.tokenizer.pad_token_id
        return (pad_stack(list(c_ids), side, pad), pad_stack(list(c_m), side), pad_stack(list(r_ids), side, pad),
                pad_stack(list(r_m), side), list(extras))
