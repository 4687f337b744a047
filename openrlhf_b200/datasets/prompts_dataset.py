"""Prompt dataset for RL (openrlhf/datasets/prompts_dataset.py:26-109): items are (datasource, prompt, label, images);
prompts go through the chat template (with a generation prompt) or ``input_template.format``; ``<image>`` tags become
VLM content lists."""
from __future__ import annotations

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


def render_prompt(row: dict, input_key: str, chat, template: str | None) -> str:
    """The text a rollout engine is prompted with: the chat template with a generation prompt (string inputs become a
    single user message; ``<image>`` tags become content parts), or the plain input through ``template.format``."""
    value = row[input_key]
    if chat is None:
        return template.format(value) if template else value
    if isinstance(value, str):
        messages = [{"role": "user", "content": _with_image_parts(value)}]
    else:
        messages = [dict(m, content=_with_image_parts(m["content"])) if isinstance(m.get("content"), str) else dict(m)
                    for m in value]
    return chat(messages, tokenize=False, add_generation_prompt=True)


class PromptDataset(Dataset):
    """Items are (datasource, prompt text, label, images), rendered once at construction."""

    def __init__(self, dataset, tokenizer, strategy, input_template=None) -> None:
        super().__init__()
        self.strategy, self.tokenizer, self.input_template = strategy, tokenizer, input_template
        d = strategy.args.data
        input_key, label_key = getattr(d, "input_key", None), getattr(d, "label_key", None)
        chat = tokenizer.apply_chat_template if getattr(d, "apply_chat_template", False) else None
        self.image_key = getattr(d, "image_key", "images")
        self.items = [(row.get("datasource", "default"), render_prompt(row, input_key, chat, input_template),
                       "" if label_key is None else row[label_key], row.get(self.image_key, None))
                      for row in dataset]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, idx):
        return self.items[idx]

    def collate_fn(self, item_list):
        if not item_list:
            return [], [], [], []
        sources, prompts, labels, images = (list(col) for col in zip(*item_list))
        return sources, prompts, labels, images
