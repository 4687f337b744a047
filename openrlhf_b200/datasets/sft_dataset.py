"""Supervised fine-tuning dataset.

Every row is encoded once, when the dataset is built: the row is rendered to its full training text together with the
character spans the model is trained to produce (the response of a prompt / response pair, every assistant turn of a
conversation, or everything in pre-training mode), the text is tokenised, the spans become token spans, and the item
that ``__getitem__`` returns is assembled from those stored ids and spans without touching the tokenizer again.

Behaviour follows the reference's SFT dataset (openrlhf/datasets/sft_dataset.py:35-228): the chat-template prefix
trick separates prompt from response (the response is what the template adds after the generation prompt), rows with
an empty side or a prompt that nearly fills ``max_length`` are dropped, the text ends with the EOS token, a truncated
sample still ends with a real EOS id, and the loss mask is shifted by one position (position t is trained to predict
token t + 1), so a span of target tokens [a, b) sets mask[a - 1 : b - 1].
"""
from __future__ import annotations

from typing import Callable

import torch
from torch.utils.data import Dataset

from ..rl.experience import pad_stack


def render_row(row: dict, *, input_key: str, output_key: str | None, template: str | None, chat: Callable | None,
               multiturn: bool, pretrain: bool) -> tuple[str, str, list[tuple[int, int]]]:
    """(prompt text, full text, character spans of the target parts inside the full text) of one row.

    Pre-training rows are their raw input and one span over all of it. Prompt / response rows have one span: the
    response. Conversations (``multiturn``) have one span per assistant message, found with the template-prefix trick:
    the text of the conversation up to and including the message, minus the text up to the message with the
    generation prompt appended."""
    if pretrain:
        text = row[input_key]
        return "", text, [(0, len(text))]
    if multiturn:
        msgs = list(row[input_key])
        if output_key and row.get(output_key):
            msgs.append(row[output_key])           # a trajectory whose last assistant turn sits in its own column
        full = chat(msgs, tokenize=False)
        spans = []
        for i, m in enumerate(msgs):
            if m["role"] == "assistant":
                head = chat(msgs[:i], tokenize=False, add_generation_prompt=True)
                upto = chat(msgs[:i + 1], tokenize=False)
                spans.append((len(head), len(upto)))
        prompt = chat(msgs[:-1], tokenize=False, add_generation_prompt=True)
        return prompt, full, spans
    if chat is not None:
        turns = row[input_key]
        if output_key:
            reply = row[output_key]
            if isinstance(turns, str) and isinstance(reply, str):
                turns, reply = [{"role": "user", "content": turns}], [{"role": "assistant", "content": reply}]
            prompt = chat(turns, tokenize=False, add_generation_prompt=True)
            full = chat(turns + reply, tokenize=False)
        else:
            prompt = chat(turns[:-1], tokenize=False, add_generation_prompt=True)
            full = chat(turns, tokenize=False)
        full = prompt + full[len(prompt):]
    else:
        prompt = row[input_key]
        if template:
            prompt = template.format(prompt)
        full = prompt + (row[output_key] if output_key else "")
    return prompt, full, [(len(prompt), len(full))]


class SFTDataset(Dataset):
    def __init__(self, dataset, tokenizer: Callable, max_length: int, strategy, input_template=None,
                 pretrain_mode: bool = False, num_processors: int = 8, multiturn: bool = False) -> None:
        super().__init__()
        self.tokenizer, self.strategy, self.max_length = tokenizer, strategy, max_length
        self.pretrain_mode, self.multiturn = pretrain_mode, multiturn
        d = strategy.args.data
        chat = None
        if getattr(d, "apply_chat_template", False) and not pretrain_mode:
            chat = tokenizer.apply_chat_template
            if getattr(d, "tokenizer_chat_template", None):
                tokenizer.chat_template = d.tokenizer_chat_template
        if multiturn:
            assert chat is not None, "multi-turn rows are rendered with the tokenizer's chat template"
        self._render = dict(input_key=getattr(d, "input_key", None), output_key=getattr(d, "output_key", None),
                            template=None if pretrain_mode else input_template, chat=chat, multiturn=multiturn,
                            pretrain=pretrain_mode)
        rows = dataset.map(self._encode, remove_columns=dataset.column_names, num_proc=num_processors)
        rows = rows.filter(lambda r: r["keep"])
        self.input_ids, self.target_spans = rows["input_ids"], rows["target_spans"]

    # ------------------------------------------------------------------ construction-time encoding
    def _ids(self, text: str) -> list[int]:
        out = self.tokenizer(text, max_length=self.max_length, padding=False, truncation=True, add_special_tokens=False)
        ids = out["input_ids"]
        return list(ids[0]) if ids and isinstance(ids[0], (list, tuple)) else list(ids)

    def _encode(self, row):
        prompt, text, spans = render_row(row, **self._render)
        empty = {"input_ids": [], "target_spans": [], "keep": False}
        if not self.pretrain_mode:
            if not prompt or all(b <= a for a, b in spans):
                return empty                                   # nothing to condition on, or nothing to learn
            # the text ends with the EOS token (outside the template's own spans in a conversation, inside the
            # response span of a prompt / response pair)
            stripped = text.rstrip("\n")
            spans = [(min(a, len(stripped)), min(b, len(stripped))) for a, b in spans]
            text = stripped
            if not text.endswith(self.tokenizer.eos_token):
                text += " " + self.tokenizer.eos_token
            if not self.multiturn:
                spans = [(spans[0][0], len(text))]
            if len(self._ids(prompt)) >= self.max_length - 2:
                return empty                                   # the prompt alone (nearly) fills the window
        ids = self._ids(text)
        # character spans -> token spans: tokens of the text before the span, then tokens of the span itself (the
        # boundaries produced by chat templates fall between tokens)
        tok_spans = []
        for a, b in spans:
            start = len(self._ids(text[:a])) if a > 0 else 0
            stop = len(ids) if b >= len(text) and not self.multiturn else start + len(self._ids(text[a:b]))
            tok_spans.append((min(start, len(ids)), min(stop, len(ids))))
        if not self.pretrain_mode and ids:
            ids[-1] = self.tokenizer.eos_token_id               # a truncated sample still ends with a real EOS
        return {"input_ids": ids, "target_spans": tok_spans, "keep": len(ids) > 0}

    # ------------------------------------------------------------------ items
    def __len__(self):
        return len(self.input_ids)

    def __getitem__(self, idx):
        ids = torch.tensor(self.input_ids[idx], dtype=torch.long).unsqueeze(0)
        att = torch.ones_like(ids)
        if self.pretrain_mode:
            return ids, att, torch.ones_like(ids, dtype=torch.float32)
        mask = torch.zeros_like(ids, dtype=torch.float32)
        for a, b in self.target_spans[idx]:
            if b > max(a, 1):
                mask[0, max(a, 1) - 1:b - 1] = 1                # position t predicts token t + 1
        return ids, att, mask

    def collate_fn(self, item_list):
        ids, att, mask = zip(*item_list)
        return (pad_stack(list(ids), "right", self.tokenizer.pad_token_id), pad_stack(list(att), "right"),
                pad_stack(list(mask), "right"))
