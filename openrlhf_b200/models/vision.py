"""Vision side of the Qwen2-VL architecture: patch embedding, ViT blocks with 2-D rotary positions, the 2x2 patch
merger, multimodal (3-component) rotary positions for the language model, and the scatter of image embeddings into the
token stream.

The reference reaches vision-language models through ``AutoModelForImageTextToText`` (openrlhf/models/actor.py:126-157,
246-265: the processor's ``pixel_values`` / ``image_grid_thw`` are forwarded to the HF model, which computes its own
M-RoPE positions). Here the tower is part of this framework's own model definition: its parameters are further views
(``visual.*``) of the same flat buffer as the language model, so the optimizer engine, checkpoints and the
trainer -> rollout weight copy cover them without special cases. The linear layers run on the same GEMM kernels as the
language model; attention inside an image frame is bidirectional with head_dim 80 and uses the library SDPA.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as TF

from ..ops import functional as F


@dataclass
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584            # output width = the language model's hidden size
    num_heads: int = 16
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    hidden_act: str = "quick_gelu"

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def mlp_dim(self) -> int:
        return int(self.embed_dim * self.mlp_ratio)

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @classmethod
    def from_dict(cls, d: dict) -> "VisionConfig":
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: d[k] for k in keys if k in d and d[k] is not None})

    def to_dict(self) -> dict:
        return {k: getattr(self, k) for k in self.__dataclass_fields__.keys()}


def vision_param_shapes(v: VisionConfig):
    """(name, shape, decay, init) of every tower parameter, in checkpoint order."""
    E, M = v.embed_dim, v.mlp_dim
    out = [("visual.patch_embed.weight", (E, v.patch_dim), True, "normal")]
    for i in range(v.depth):
        b = f"visual.blocks.{i}."
        out += [(b + "norm1.weight", (E,), False, "ones"), (b + "norm1.bias", (E,), False, "zeros"),
                (b + "attn.qkv.weight", (3 * E, E), True, "normal"), (b + "attn.qkv.bias", (3 * E,), False, "zeros"),
                (b + "attn.proj.weight", (E, E), True, "normal"), (b + "attn.proj.bias", (E,), False, "zeros"),
                (b + "norm2.weight", (E,), False, "ones"), (b + "norm2.bias", (E,), False, "zeros"),
                (b + "mlp.fc1.weight", (M, E), True, "normal"), (b + "mlp.fc1.bias", (M,), False, "zeros"),
                (b + "mlp.fc2.weight", (E, M), True, "normal"), (b + "mlp.fc2.bias", (E,), False, "zeros")]
    G = E * v.spatial_merge_size ** 2
    out += [("visual.merger.ln_q.weight", (E,), False, "ones"), ("visual.merger.ln_q.bias", (E,), False, "zeros"),
            ("visual.merger.mlp.0.weight", (G, G), True, "normal"), ("visual.merger.mlp.0.bias", (G,), False, "zeros"),
            ("visual.merger.mlp.2.weight", (v.hidden_size, G), True, "normal"),
            ("visual.merger.mlp.2.bias", (v.hidden_size,), False, "zeros")]
    return out


# ---------------------------------------------------------------------------------------------- tower forward
def _patch_positions(grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """(row, column) of every patch in the processor's order: patches are grouped in merge x merge blocks so that the
    merger can concatenate neighbours with a reshape. Returns int64 [N, 2]."""
    out = []
    for t, h, w in grid_thw.tolist():
        hh = torch.arange(h)[:, None].expand(h, w)
        ww = torch.arange(w)[None, :].expand(h, w)

        def blocked(x):
            return x.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)

        out.append(torch.stack([blocked(hh), blocked(ww)], dim=-1).repeat(t, 1))
    return torch.cat(out, 0)


def _vision_rotary(grid_thw: torch.Tensor, v: VisionConfig, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [N, head_dim] fp32: the first quarter of the rotary pairs turns with the row, the second with the
    column (then the usual duplicated-halves layout)."""
    dim = v.head_dim // 2
    inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    pos = _patch_positions(grid_thw, v.spatial_merge_size)                    # [N, 2]
    ang = (pos[:, :, None].float() * inv[None, None, :]).flatten(1)           # [N, dim]
    ang = torch.cat([ang, ang], dim=-1).to(device)
    return ang.cos(), ang.sin()


def _rotate_half(x):
    a, b = x.chunk(2, dim=-1)
    return torch.cat([-b, a], dim=-1)


def _act(x, name: str):
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name in ("gelu", "gelu_pytorch_tanh"):
        return TF.gelu(x, approximate="tanh" if name.endswith("tanh") else "none")
    if name == "silu":
        return TF.silu(x)
    raise ValueError(f"unsupported vision activation {name}")


def vision_forward(p, v: VisionConfig, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
    """pixel_values [N, patch_dim] (the HF image processor's flattened patches), grid_thw int [n_images, 3] ->
    image embeddings [N / merge^2, hidden_size] in token order. ``p(name)`` returns a tower parameter."""
    w0 = p("visual.patch_embed.weight")
    x = F.linear(pixel_values.to(w0.dtype), w0)
    N, E, nh, hd = x.shape[0], v.embed_dim, v.num_heads, v.head_dim
    cos, sin = _vision_rotary(grid_thw, v, x.device)
    g = grid_thw.tolist()
    frames = [h * w for t, h, w in g for _ in range(t)]
    assert sum(frames) == N, f"pixel_values has {N} patches, image_grid_thw describes {sum(frames)}"
    scale = 1.0 / math.sqrt(hd)
    for i in range(v.depth):
        b = f"visual.blocks.{i}."
        y = TF.layer_norm(x, (E,), p(b + "norm1.weight"), p(b + "norm1.bias"), 1e-6)
        qkv = F.linear(y, p(b + "attn.qkv.weight"), p(b + "attn.qkv.bias")).view(N, 3, nh, hd)
        q, k, val = qkv[:, 0].float(), qkv[:, 1].float(), qkv[:, 2]
        q = (q * cos[:, None] + _rotate_half(q) * sin[:, None]).to(val.dtype)
        k = (k * cos[:, None] + _rotate_half(k) * sin[:, None]).to(val.dtype)
        outs, a0 = [], 0
        for n in frames:                                    # bidirectional attention inside one frame
            qs, ks, vs = (z[a0:a0 + n].transpose(0, 1)[None] for z in (q, k, val))
            outs.append(TF.scaled_dot_product_attention(qs, ks, vs, scale=scale)[0].transpose(0, 1))
            a0 += n
        a = torch.cat(outs, 0).reshape(N, E)
        x = x + F.linear(a, p(b + "attn.proj.weight"), p(b + "attn.proj.bias"))
        y = TF.layer_norm(x, (E,), p(b + "norm2.weight"), p(b + "norm2.bias"), 1e-6)
        y = _act(F.linear(y, p(b + "mlp.fc1.weight"), p(b + "mlp.fc1.bias")), v.hidden_act)
        x = x + F.linear(y, p(b + "mlp.fc2.weight"), p(b + "mlp.fc2.bias"))
    m2 = v.spatial_merge_size ** 2
    y = TF.layer_norm(x, (E,), p("visual.merger.ln_q.weight"), p("visual.merger.ln_q.bias"), 1e-6).view(N // m2, E * m2)
    y = TF.gelu(F.linear(y, p("visual.merger.mlp.0.weight"), p("visual.merger.mlp.0.bias")))
    return F.linear(y, p("visual.merger.mlp.2.weight"), p("visual.merger.mlp.2.bias"))


# ---------------------------------------------------------------------------------------------- language-model side
def image_runs(ids: list[int], grids: list[tuple[int, int, int]], image_token_id: int, merge: int,
               video_token_id: int | None = None) -> list[tuple[int, int, tuple[int, int, int]]]:
    """Match the placeholder runs of one sequence to the next grids, in order: [(start, length, grid)]. A run counts
    only when it is complete (t * h/merge * w/merge placeholders in a row); a stray placeholder token, e.g. one the
    policy sampled itself, stays an ordinary text token."""
    media = {image_token_id} | ({video_token_id} if video_token_id is not None and video_token_id >= 0 else set())
    out, i, gi, n = [], 0, 0, len(ids)
    while i < n and gi < len(grids):
        if ids[i] in media:
            t, h, w = grids[gi]
            cnt = t * (h // merge) * (w // merge)
            if i + cnt <= n and all(x in media for x in ids[i:i + cnt]):
                out.append((i, cnt, (t, h, w)))
                gi += 1
                i += cnt
                continue
        i += 1
    return out


def mrope_positions(ids: list[int], grids: list[tuple[int, int, int]], image_token_id: int, merge: int,
                    video_token_id: int | None = None) -> tuple[torch.Tensor, int]:
    """3-component positions of one sequence. Text tokens count up with all components equal; the tokens of an image
    (a run of `image_token_id`, t * h/merge * w/merge long) keep the temporal component at the run's start and walk
    the grid with the other two; the text that follows continues after the largest position used so far.

    Returns (int32 [3, len(ids)], delta) where the position of the k-th token generated after the sequence is
    ``len(ids) + k + delta`` in every component."""
    n = len(ids)
    pos = torch.zeros(3, n, dtype=torch.int32)
    nxt, i = 0, 0
    for start, cnt, (t, h, w) in image_runs(ids, grids, image_token_id, merge, video_token_id):
        if start > i:
            pos[:, i:start] = torch.arange(nxt, nxt + start - i, dtype=torch.int32)
            nxt += start - i
        lh, lw = h // merge, w // merge
        tt = torch.arange(t).view(t, 1, 1).expand(t, lh, lw).reshape(-1)
        hh = torch.arange(lh).view(1, lh, 1).expand(t, lh, lw).reshape(-1)
        ww = torch.arange(lw).view(1, 1, lw).expand(t, lh, lw).reshape(-1)
        pos[:, start:start + cnt] = (torch.stack([tt, hh, ww]) + nxt).to(torch.int32)
        nxt += max(t, lh, lw)
        i = start + cnt
    if n > i:
        pos[:, i:] = torch.arange(nxt, nxt + n - i, dtype=torch.int32)
        nxt += n - i
    return pos, nxt - n


def mrope_rows(table: torch.Tensor, pos3: torch.Tensor, sections) -> torch.Tensor:
    """Per-token rotary rows [T, head_dim/2, 2] from the ordinary table [max_pos, head_dim/2, 2]: frequency j takes the
    temporal, height or width position according to which section of `sections` (summing to head_dim/2) it lies in."""
    half = table.shape[1]
    assert sum(sections) == half, f"mrope sections {sections} must sum to {half}"
    comp = torch.repeat_interleave(torch.arange(len(sections)), torch.tensor(list(sections))).to(table.device)
    idx = pos3.to(table.device).long()[comp % 3]                 # [half, T]: position used by each frequency
    j = torch.arange(half, device=table.device)[:, None].expand_as(idx)
    return table[idx, j].transpose(0, 1).contiguous()            # [T, half, 2]


def scatter_image_embeds(embeds: torch.Tensor, where: torch.Tensor, image_embeds: torch.Tensor) -> torch.Tensor:
    """Replace the embeddings at the placeholder positions `where` (int64, in order) by the tower's output rows."""
    assert where.numel() == image_embeds.shape[0], \
        f"{where.numel()} image placeholder tokens matched but {image_embeds.shape[0]} image embeddings"
    return embeds.index_put((where.to(embeds.device),), image_embeds.to(embeds.dtype))
