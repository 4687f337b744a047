"""Prompt dataset for RL (openrlhf/datasets/prompts_dataset.py:26-109): items are (datasource, prompt, label, images);
prompts go through the chat template (with a generation prompt) or ``input_template.format``; ``<image>`` tags become
VLM content lists."""
from __future__ import annotations

import copy

from torch.utils.data import Dataset


def _with_image_parts(text: str):
    """"<image>Find x." -> [{"type": "image"}, {"type": "text", "text": "Find x."}]; plain strings pass through."""
    if "<image>" not in text:
        return text
    content = []
    for i, piece in enumerate(text.split("<image>")):
        if i:
            content.append({"type": "image"})
        if piece.strip():
            content.append({"type": "text", "text": piece.strip()})
    return content


def preprocess_data(data, input_template=None, input_key="input", label_key=None, apply_chat_template=None):
    if apply_chat_template:
        chat = data[input_key]
        if isinstance(chat, str):
            chat = [{"role": "user", "content": _with_image_parts(chat)}]
        else:
            chat = copy.deepcopy(chat)
            for msg in chat:
                if isinstance(msg.get("content"), str):
                    msg["content"] = _with_image_parts(msg["content"])
        prompt = apply_chat_template(chat, tokenize=False, add_generation_prompt=True)
    else:
        prompt = data[input_key]
        if input_template:
            prompt = input_template.format(prompt)
    return prompt, ("" if label_key is None else data[label_key])


class PromptDataset(Dataset):
    def __init__(self, dataset, tokenizer, strategy, input_template=None) -> None:
        super().__init__()
        self.strategy, self.tokenizer, self.input_template = strategy, tokenizer, input_template
        d = strategy.args.data
        input_key, label_key = getattr(d, "input_key", None), getattr(d, "label_key", None)
        tmpl = tokenizer.apply_chat_template if getattr(d, "apply_chat_template", False) else None
        self.image_key = getattr(d, "image_key", "images")
        self.prompts, self.labels, self.images, self.datasources = [], [], [], []
        for row in dataset:
            p, l = preprocess_data(row, input_template, input_key, label_key, tmpl)
            self.prompts.append(p)
            self.labels.append(l)
            self.images.append(row.get(self.image_key, None))
            self.datasources.append(row.get("datasource", "default"))

    def __len__(self):
        return len(self.prompts)

    def __getitem__(self, idx):
        return self.datasources[idx], self.prompts[idx], self.labels[idx], self.images[idx]

    def collate_fn(self, item_list):
        cols = list(zip(*item_list)) if item_list else [(), (), (), ()]
        return tuple(list(c) for c in cols)
