"""Conversion between padded (B, T) batches and the packed token stream the model consumes.

Replaces flash-attn's bert_padding round trip used by the reference (openrlhf/models/ring_attn_utils.py:103-182):
labels are the sequence rolled by -1 inside the padded matrix, positions restart per sample, and the packed stream
can be cut into contiguous context-parallel slices.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PackedBatch:
    input_ids: torch.Tensor      # int64 [T]
    labels: torch.Tensor         # int64 [T] next token of each position (garbage at each sample's last position)
    position_ids: torch.Tensor   # int32 [T]
    cu_seqlens: torch.Tensor     # int32 [B+1]
    max_seqlen: int
    indices: torch.Tensor        # int64 [T] flat index of each packed token in the (B*T) padded matrix
    batch: int
    seqlen: int


def pack_padded(sequences: torch.Tensor, attention_mask: torch.Tensor) -> PackedBatch:
    B, T = sequences.shape
    mask = attention_mask.bool()
    rolled = torch.roll(sequences, shifts=-1, dims=1)
    indices = torch.nonzero(mask.reshape(-1), as_tuple=False).squeeze(-1)
    lens = mask.sum(-1).to(torch.int32)
    cu = torch.zeros(B + 1, dtype=torch.int32, device=sequences.device)
    cu[1:] = torch.cumsum(lens, 0)
    pos = (torch.cumsum(mask.long(), -1) - 1).clamp_min(0).reshape(-1)[indices].to(torch.int32)
    return PackedBatch(sequences.reshape(-1)[indices].long(), rolled.reshape(-1)[indices].long(), pos, cu,
                       int(lens.max().item()) if B > 0 else 0, indices, B, T)


def unpack_to_padded(values: torch.Tensor, pb: PackedBatch, fill: float = 0.0) -> torch.Tensor:
    """Scatter per-token values [T] back into a (B, T) matrix."""
    out = torch.full((pb.batch * pb.seqlen,), fill, dtype=values.dtype, device=values.device)
    out = out.index_put((pb.indices,), values)
    return out.view(pb.batch, pb.seqlen)


def pack_lists(seqs: list[torch.Tensor], device=None) -> PackedBatch:
    """Pack a list of 1-D token tensors directly (no padded intermediate)."""
    device = device or seqs[0].device
    lens = torch.tensor([len(s) for s in seqs], dtype=torch.int32)
    ids = torch.cat([s.to(device) for s in seqs]).long()
    cu = torch.zeros(len(seqs) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lens]).to(device)
    labels = torch.cat([torch.cat([s[1:], s[:1]]) for s in seqs]).to(device).long()
    T = int(lens.max())
    idx = torch.cat([torch.arange(int(n)) + i * T for i, n in enumerate(lens)]).to(device)
    return PackedBatch(ids, labels, pos, cu.to(device), T, idx, len(seqs), T)
