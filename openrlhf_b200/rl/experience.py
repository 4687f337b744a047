"""The ``Experience`` container and its batching utilities.

API-compatible with the reference's packed-sample experience API (openrlhf/trainer/ppo_utils/experience.py:28-283):
same field names and shapes, same split / batch / strip-padding / balance functions. Layout conventions:
step tensors are ``(B, T)`` or ``(B, A)`` with right padding, episode tensors are ``(B,)``; ``action_mask`` has
``T-1`` columns (column i = "predicting token i+1").
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Iterable

import torch

STEP_FIELDS = ("sequences", "attention_mask", "action_mask", "action_log_probs", "base_action_log_probs",
               "rollout_log_probs", "values", "returns", "advantages", "kl")
EPISODE_FIELDS = ("rewards", "scores", "response_length", "truncated", "total_length")
LIST_FIELDS = ("prompts", "labels", "images", "mm_train_inputs")


def pad_stack(tensors: list[torch.Tensor], side: str = "right", value: float = 0, stack: bool = False) -> torch.Tensor:
    """Pad 1-D (or (1, L)) tensors along the last dim to a common length and stack / concatenate them."""
    assert side in ("left", "right")
    width = max(t.shape[-1] for t in tensors)
    out = []
    for t in tensors:
        gap = width - t.shape[-1]
        if gap:
            pad = (gap, 0) if side == "left" else (0, gap)
            t = torch.nn.functional.pad(t, pad, value=value)
        out.append(t)
    return torch.stack(out, 0) if stack else torch.cat(out, 0)


def _map_tensors(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, list):
        return [_map_tensors(o, fn) for o in obj]
    if isinstance(obj, dict):
        return {k: _map_tensors(v, fn) for k, v in obj.items()}
    return obj


def to(obj, device):
    """Tensors inside `obj` (a tensor, or lists / dicts of them) moved to `device`; everything else is returned as is."""
    return _map_tensors(obj, lambda t: t.to(device))


def pin_memory(obj):
    """Tensors inside `obj` copied into page-locked host memory (for asynchronous host-to-device copies)."""
    return _map_tensors(obj, lambda t: t.pin_memory())


@dataclass
class Experience:
    # trajectory
    sequences: torch.Tensor = None            # (B, T) prompt + response token ids
    attention_mask: torch.Tensor = None       # (B, T)
    action_mask: torch.Tensor = None          # (B, A)
    # log-probs under the policies involved
    action_log_probs: torch.Tensor = None     # (B, A) current / old policy
    base_action_log_probs: torch.Tensor = None  # (B, A) reference policy
    rollout_log_probs: torch.Tensor = None    # (B, A) rollout engine
    # value estimation
    values: torch.Tensor = None               # (B, A)
    returns: torch.Tensor = None              # (B, A)
    advantages: torch.Tensor = None           # (B, A)
    kl: torch.Tensor = None                   # (B, A)
    # per-episode scalars
    rewards: torch.Tensor = None              # (B,)
    scores: torch.Tensor = None               # (B,)
    response_length: torch.Tensor = None      # (B,)
    truncated: torch.Tensor = None            # (B,)
    total_length: torch.Tensor = None         # (B,)
    # metadata
    index: list = None
    prompts: list = field(default_factory=list)
    labels: list = field(default_factory=list)
    images: list = field(default_factory=list)
    mm_train_inputs: list = field(default_factory=list)
    info: dict = field(default_factory=dict)

    @staticmethod
    def is_step_tensor_field(name: str) -> bool:
        return name in STEP_FIELDS

    @staticmethod
    def is_episode_tensor_field(name: str) -> bool:
        return name in EPISODE_FIELDS

    def _apply(self, fn) -> "Experience":
        for f in dataclasses.fields(self):
            setattr(self, f.name, _map_tensors(getattr(self, f.name), fn))
        return self

    @torch.no_grad()
    def to_device(self, device) -> "Experience":
        return self._apply(lambda t: t.to(device, non_blocking=True))

    def pin_memory(self) -> "Experience":
        return self._apply(lambda t: t.pin_memory() if not t.is_cuda else t)

    def __len__(self) -> int:
        return 0 if self.sequences is None else len(self.sequences)

    @staticmethod
    def concat_experiences(experiences_list: list["Experience"], pad_token_id: int) -> "Experience":
        """Row-concatenate batched experiences, right-padding step tensors (sequences with pad_token_id, others 0)."""
        if not experiences_list:
            return Experience()

        def merge(values: list, pad: int):
            head = values[0]
            if head is None:
                return None
            if isinstance(head, torch.Tensor):
                return pad_stack(values, "right", pad) if head.dim() >= 2 else torch.cat(values, 0)
            if isinstance(head, list):
                return [x for v in values for x in v]
            if isinstance(head, dict):
                keys: list = []
                for d in values:
                    keys += [k for k in d if k not in keys]
                return {k: merge([d[k] for d in values if k in d], pad) for k in keys}
            raise ValueError(f"cannot merge values of type {type(head)}")

        out = {}
        for f in dataclasses.fields(Experience):
            out[f.name] = merge([getattr(e, f.name) for e in experiences_list],
                                pad_token_id if f.name == "sequences" else 0)
        return Experience(**out)


# ------------------------------------------------------------------------------------------------- batch utilities
def split_experience_batch(experience: Experience) -> list[Experience]:
    """(B, ...) experience -> B single-sample experiences (tensors lose their batch dim)."""
    B = len(experience.sequences)
    experience.index = None
    singles = []
    for i in range(B):
        kw: dict[str, Any] = {}
        for f in dataclasses.fields(Experience):
            v = getattr(experience, f.name)
            if isinstance(v, torch.Tensor):
                if len(v) != B:
                    raise ValueError(f"{f.name} has {len(v)} rows, expected {B}")
                kw[f.name] = v[i]
            elif isinstance(v, dict):
                row = {}
                for k, x in v.items():
                    if not isinstance(x, (torch.Tensor, list)):
                        raise TypeError(f"{f.name}[{k}] must be a tensor or a list, got {type(x)}")
                    if len(x) != B:
                        raise ValueError(f"{f.name}[{k}] has {len(x)} rows, expected {B}")
                    row[k] = x[i]
                kw[f.name] = row
            elif isinstance(v, list):
                kw[f.name] = [v[i]] if len(v) == B else v
            else:
                kw[f.name] = v
        singles.append(Experience(**kw))
    return singles


def make_experience_batch(items: list[Experience], packing_samples: bool = False) -> Experience:
    """Single-sample experiences -> one batch; step tensors are right-padded with zeros and stacked."""
    if not items:
        raise ValueError("cannot batch an empty list of experiences")
    kw: dict[str, Any] = {}
    for f in dataclasses.fields(Experience):
        col = [getattr(it, f.name) for it in items]
        head = col[0]
        if head is None:
            kw[f.name] = None
        elif isinstance(head, torch.Tensor):
            if f.name in STEP_FIELDS:
                kw[f.name] = pad_stack(col, "right", 0, stack=True)
            elif f.name in EPISODE_FIELDS or head.dim() == 0:
                kw[f.name] = torch.stack(col)
            else:
                raise ValueError(f"no batching rule for tensor field {f.name}")
        elif isinstance(head, dict):
            merged = {}
            for k in head:
                vals = [c[k] for c in col]
                if any(type(v) is not type(vals[0]) for v in vals):
                    raise TypeError(f"mixed value types in {f.name}[{k}]")
                merged[k] = torch.tensor(vals) if all(isinstance(v, (int, float)) for v in vals) else vals
            kw[f.name] = merged
        elif isinstance(head, list):
            kw[f.name] = [x for c in col for x in c]
        else:
            kw[f.name] = head
    return Experience(**kw)


def remove_padding_in_sequences(items: Iterable[Experience]) -> list[Experience]:
    """Strip right padding (as given by attention_mask) from every step tensor of single-sample experiences."""
    items = list(items)
    for it in items:
        n_valid = int(it.attention_mask.shape[0] - it.attention_mask.flip(0).argmax()) if it.attention_mask.any() else 0
        n_pad = it.attention_mask.shape[0] - n_valid
        if n_pad == 0:
            continue
        for name in STEP_FIELDS:
            v = getattr(it, name)
            if isinstance(v, torch.Tensor):
                setattr(it, name, v[: v.shape[0] - n_pad])
    return items


def balance_experiences(experiences: list[Experience], args) -> list[Experience]:
    """Distribute samples over data-parallel ranks so that every rank gets a similar token count: sort by total
    length, cut into rounds of `dp` samples, and deal long rounds forwards and short rounds backwards.

    Returns one batch per DP rank (fewer if there are fewer samples than ranks)."""
    singles: list[Experience] = []
    for e in experiences:
        singles += split_experience_batch(e)
    singles.sort(key=lambda s: int(s.total_length), reverse=True)
    dp = args.actor.num_nodes * args.actor.num_gpus_per_node // args.ds.ring_attn_size // args.ds.tensor_parallel_size
    rounds = [singles[i:i + dp] for i in range(0, len(singles), dp)]
    n_long = len(rounds) // 2
    long_rounds, short_rounds = rounds[:n_long], [r[::-1] for r in rounds[n_long:]]
    order = []
    for i in range(n_long):
        order += [long_rounds[i], short_rounds[-(i + 1)]]
    if len(short_rounds) > n_long:
        order.append(short_rounds[0])
    per_rank: list[list[Experience]] = [[] for _ in range(dp)]
    for rnd in order:
        for r, item in enumerate(rnd):
            per_rank[r].append(item)
    return [make_experience_batch(b) for b in per_rank if b]
