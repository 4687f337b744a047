"""SFT dataset (openrlhf/datasets/sft_dataset.py:35-228): prompt/response split (chat-template prefix trick), multi-turn
response ranges, loss mask on ``[prompt_len-1 : -1]``, forced EOS as last token, right-pad collate, pretrain mode."""
from __future__ import annotations

from typing import Callable

import torch
from torch.utils.data import Dataset

from ..rl.experience import pad_stack


def preprocess_data(data, input_template=None, input_key="input", output_key=None, apply_chat_template=None):
    if apply_chat_template:
        if output_key:
            p, r = data[input_key], data[output_key]
            if isinstance(p, str) and isinstance(r, str):
                p, r = [{"role": "user", "content": p}], [{"role": "assistant", "content": r}]
            prompt = apply_chat_template(p, tokenize=False, add_generation_prompt=True)
            response = apply_chat_template(p + r, tokenize=False)[len(prompt):]
        else:
            prompt = apply_chat_template(data[input_key][:-1], tokenize=False, add_generation_prompt=True)
            response = apply_chat_template(data[input_key], tokenize=False)[len(prompt):]
    else:
        prompt = data[input_key]
        if input_template:
            prompt = input_template.format(prompt)
        response = data[output_key] if output_key else ""
    return prompt, response


class SFTDataset(Dataset):
    def __init__(self, dataset, tokenizer: Callable, max_length: int, strategy, input_template=None,
                 pretrain_mode: bool = False, num_processors: int = 8, multiturn: bool = False) -> None:
        super().__init__()
        self.tokenizer, self.strategy, self.max_length = tokenizer, strategy, max_length
        self.pretrain_mode, self.multiturn, self.input_template = pretrain_mode, multiturn, input_template
        d = strategy.args.data
        self.input_key, self.output_key = getattr(d, "input_key", None), getattr(d, "output_key", None)
        self.apply_chat_template = None
        if getattr(d, "apply_chat_template", False):
            self.apply_chat_template = tokenizer.apply_chat_template
            if getattr(d, "tokenizer_chat_template", None):
                tokenizer.chat_template = d.tokenizer_chat_template
        rows = dataset.map(self.process_data, remove_columns=dataset.column_names, num_proc=num_processors)
        rows = rows.filter(lambda x: x["prompt"] is not None)
        self.prompts, self.responses = rows["prompt"], rows["response"]
        self.prompt_ids_lens = rows["prompt_ids_len"]
        self.response_ranges = rows["response_ranges"] if multiturn else None

    def _ntok(self, text: str) -> int:
        t = self.tokenizer(text, max_length=self.max_length, padding=False, truncation=True, return_tensors="pt",
                           add_special_tokens=False)
        return int(t["attention_mask"].int().sum().item())

    def process_data(self, data):
        ranges = None
        if self.multiturn and self.output_key:
            data[self.input_key].append(data[self.output_key])
            data[self.output_key] = None
        if self.multiturn:
            if self.output_key and data[self.output_key]:
                raise AssertionError("put the whole trajectory into data[input_key]; do not set output_key")
            ranges = []
            msgs = data[self.input_key]
            for i, m in enumerate(msgs):
                if m["role"] != "assistant":
                    continue
                before = self.apply_chat_template(msgs[:i], tokenize=False, add_generation_prompt=True)
                reply = self.apply_chat_template(msgs[:i + 1], tokenize=False)[len(before):]
                start = self._ntok(before)
                ranges.append((start, start + self._ntok(reply) - 1))      # closed interval
        prompt, response = preprocess_data(data, None if self.pretrain_mode else self.input_template, self.input_key,
                                           self.output_key, None if self.pretrain_mode else self.apply_chat_template)
        n_prompt = 0
        if not self.pretrain_mode:
            n_prompt = self._ntok(prompt)
            if not prompt or not response or n_prompt >= self.max_length - 2:
                prompt = None
        return {"prompt": prompt, "response": response, "prompt_ids_len": n_prompt, "response_ranges": ranges}

    def __len__(self):
        return len(self.prompts)

    def __getitem__(self, idx):
        text = self.prompts[idx]
        if not self.pretrain_mode:
            text = (text + self.responses[idx]).rstrip("\n")
            if not text.endswith(self.tokenizer.eos_token):
                text += " " + self.tokenizer.eos_token
        tok = self.tokenizer(text, max_length=self.max_length, padding=False, truncation=True, return_tensors="pt",
                             add_special_tokens=False)
        ids, att = tok["input_ids"], tok["attention_mask"]
        mask = self.get_loss_mask(ids, idx)
        if not self.pretrain_mode:                       # survive truncation with a real EOS at the end
            ids[0][-1] = self.tokenizer.eos_token_id
            att[0][-1] = True
        return ids, att, mask

    def get_loss_mask(self, input_ids, idx):
        if self.pretrain_mode:
            return torch.ones_like(input_ids, dtype=torch.float32)
        m = torch.zeros_like(input_ids, dtype=torch.float32)
        if not self.multiturn:
            m[0, self.prompt_ids_lens[idx] - 1:-1] = 1
        else:
            for a, b in self.response_ranges[idx]:
                m[0, a - 1:b] = 1
        return m

    def collate_fn(self, item_list):
        ids, att, mask = zip(*item_list)
        return (pad_stack(list(ids), "right", self.tokenizer.pad_token_id), pad_stack(list(att), "right"),
                pad_stack(list(mask), "right"))
