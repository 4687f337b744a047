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
    cu_list: list | None = None   # cu_seqlens as Python ints when the packer had them on the host (no device read)


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


def _to_device(t: torch.Tensor, device):
    """Host -> device without stalling the host: a pageable source makes the copy wait for the stream to drain (one
    pipeline bubble per call), a pinned source with non_blocking does not."""
    device = torch.device(device)
    if device.type != "cuda" or t.is_cuda:
        return t.to(device)
    return t.pin_memory().to(device, non_blocking=True)


def pack_lists(seqs: list[torch.Tensor], device=None) -> PackedBatch:
    """Pack a list of 1-D token tensors directly (no padded intermediate). Sequences that live on the host are
    concatenated there and moved with one asynchronous copy per field."""
    device = device or seqs[0].device
    lens = torch.tensor([len(s) for s in seqs], dtype=torch.int32)
    cu = torch.zeros(len(seqs) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    T = int(lens.max())
    pos_c = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lens])
    idx_c = torch.cat([torch.arange(int(n)) + i * T for i, n in enumerate(lens)])
    if all(not s.is_cuda for s in seqs):
        ids = _to_device(torch.cat(list(seqs)).long(), device)
        labels = _to_device(torch.cat([torch.cat([s[1:], s[:1]]) for s in seqs]).long(), device)
    else:
        ids = torch.cat([s.to(device) for s in seqs]).long()
        labels = torch.cat([torch.cat([s[1:], s[:1]]) for s in seqs]).to(device).long()
    return PackedBatch(ids, labels, _to_device(pos_c, device), _to_device(cu, device), T, _to_device(idx_c, device),
                       len(seqs), T, cu.tolist())


def pack_lists_cp(seqs: list[torch.Tensor], world: int, pad_id: int = 0, device=None):
    """Pack documents for context parallelism: every document is padded at its end to a multiple of 128 tokens (the
    pad tokens attend to the document but nothing attends to them), and a trailing pad document rounds the stream up
    to a multiple of 128*world rows, so that each rank's chunk is a whole number of 128-row tiles and no tile
    straddles two ranks. Returns (PackedBatch over the global stream, valid [T] bool: real tokens).

    The reference pads the packed stream to a multiple of the ring size and slices it per rank
    (openrlhf/models/ring_attn_utils.py:101-141)."""
    device = device or seqs[0].device
    docs, valid = [], []
    for s in seqs:
        n = len(s)
        padn = (-n) % 128
        docs.append(torch.cat([s.to(device).long(), torch.full((padn,), pad_id, dtype=torch.long, device=device)]))
        valid.append(torch.cat([torch.ones(n, dtype=torch.bool), torch.zeros(padn, dtype=torch.bool)]))
    total = sum(len(d) for d in docs)
    tail = (-total) % (128 * world)
    if tail:
        docs.append(torch.full((tail,), pad_id, dtype=torch.long, device=device))
        valid.append(torch.zeros(tail, dtype=torch.bool))
    pb = pack_lists(docs, device=device)
    v = torch.cat(valid).to(device)
    # the last real token of a document has no next token inside it
    ends = torch.tensor([0] + [len(d) for d in docs]).cumsum(0)
    for i, s in enumerate(seqs):
        v[int(ends[i]) + len(s) - 1] = False
    return pb, v


def cp_slice(pb: PackedBatch, rank: int, world: int):
    """This rank's rows of a batch packed by pack_lists_cp: (input_ids, labels, position_ids) of T/world rows each;
    cu_seqlens stays global."""
    T = pb.input_ids.numel()
    assert T % (128 * world) == 0
    lo, hi = rank * (T // world), (rank + 1) * (T // world)
    return pb.input_ids[lo:hi], pb.labels[lo:hi], pb.position_ids[lo:hi].contiguous()
