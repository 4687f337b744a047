"""Trainer -> rollout weight synchronisation as a precomputed copy plan (one kernel launch per sync).

The trainer keeps every parameter in one flat bf16 buffer (models/transformer.py), possibly sharded over ranks in
equal contiguous slices (ZeRO-3). A rollout engine with tensor parallelism wants, per TP rank, its slice of every
matrix, again in one flat buffer. ``build_plan`` turns (parameter layout, source sharding, TP slicing) into a list of
strided row-block copies {source rank, source offset, destination offset, rows, row length, strides};
``ReshardPlan.run`` uploads it once and each sync is a single launch of the copy kernel that reads the sources over
peer memory (plain loads; local when source rank == this rank).

The reference does this with one NCCL broadcast (or a CUDA-IPC handle exchange) per parameter followed by vLLM's
``load_weights`` slicing on every worker (openrlhf/trainer/ray/ppo_actor.py:420-465,
openrlhf/trainer/ray/vllm_worker_wrap.py:32-50).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ..models.config import ModelConfig
from ..models.transformer import ALIGN, ParamSpec, build_param_specs


@dataclass
class CopyEntry:
    src_off: int
    dst_off: int
    rows: int
    row_elems: int
    src_ld: int
    dst_ld: int
    src_rank: int


def _tp_row_ranges(name: str, shape, cfg: ModelConfig, tp_rank: int, tp: int, vocab_parallel: bool = False):
    """(row ranges, column range) of the parameter that TP rank `tp_rank` holds. Column-parallel matrices are cut by
    rows of the fused layouts (q | k | v heads, gate | up), row-parallel ones by columns; the rest is replicated."""
    D = cfg.head_dim
    leaf = name.split(".")[-2] + "." + name.split(".")[-1] if "." in name else name
    rows_all = [(0, shape[0])]
    cols_all = (0, shape[-1]) if len(shape) > 1 else (0, 1)
    if tp == 1:
        return rows_all, cols_all
    if vocab_parallel and name == "lm_head.weight":
        assert shape[0] % tp == 0
        s = shape[0] // tp
        return [(tp_rank * s, (tp_rank + 1) * s)], cols_all
    Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    if leaf in ("qkv.weight", "qkv.bias"):
        assert Hq % tp == 0 and Hkv % tp == 0, "heads must divide the tensor-parallel size"
        q0, k0, v0 = 0, Hq * D, (Hq + Hkv) * D
        hq, hk = Hq // tp * D, Hkv // tp * D
        return [(q0 + tp_rank * hq, q0 + (tp_rank + 1) * hq), (k0 + tp_rank * hk, k0 + (tp_rank + 1) * hk),
                (v0 + tp_rank * hk, v0 + (tp_rank + 1) * hk)], cols_all
    if leaf == "gate_up.weight":
        I = shape[0] // 2
        assert I % tp == 0
        s = I // tp
        return [(tp_rank * s, (tp_rank + 1) * s), (I + tp_rank * s, I + (tp_rank + 1) * s)], cols_all
    if leaf in ("o.weight", "down.weight"):
        assert shape[1] % tp == 0
        s = shape[1] // tp
        return rows_all, (tp_rank * s, (tp_rank + 1) * s)
    return rows_all, cols_all


def tp_param_specs(cfg: ModelConfig, tp_rank: int, tp: int, with_lm_head: bool = True,
                   with_value_head: bool = False, vocab_parallel: bool = False) -> list[ParamSpec]:
    """Layout of one TP rank's flat buffer (same order and alignment rule as the trainer's)."""
    out, off = [], 0
    for s in build_param_specs(cfg, with_lm_head, with_value_head):
        if len(s.shape) == 3:          # experts [E, rows, cols]: kept whole (expert parallelism shards by expert)
            shape = s.shape
        else:
            rows, cols = _tp_row_ranges(s.name, s.shape, cfg, tp_rank, tp, vocab_parallel)
            nrows = sum(b - a for a, b in rows)
            shape = (nrows, cols[1] - cols[0]) if len(s.shape) == 2 else (nrows,)
        n = 1
        for d in shape:
            n *= d
        out.append(ParamSpec(s.name, tuple(shape), off, n, s.decay, s.init))
        off += (n + ALIGN - 1) // ALIGN * ALIGN
    return out


def build_plan(cfg: ModelConfig, tp_rank: int = 0, tp: int = 1, src_world: int = 1, src_shard_elems: int | None = None,
               with_lm_head: bool = True, with_value_head: bool = False,
               vocab_parallel: bool = False) -> tuple[list[CopyEntry], int]:
    """Copy plan for one destination TP rank. Sources: `src_world` == 1 (every rank holds the whole flat buffer: read
    locally, source rank 0 in the table the caller passes) or a flat buffer cut into `src_world` slices of
    `src_shard_elems` elements (ZeRO-3: entries are split where a row block crosses a slice boundary).
    Returns (entries, destination buffer size in elements)."""
    src_specs = build_param_specs(cfg, with_lm_head, with_value_head)
    dst_specs = tp_param_specs(cfg, tp_rank, tp, with_lm_head, with_value_head, vocab_parallel)
    entries: list[CopyEntry] = []

    def emit(src_off, dst_off, rows, row_elems, src_ld, dst_ld):
        """One strided block; split by source slice when the source is sharded."""
        if rows <= 0 or row_elems <= 0:
            return
        if src_world == 1:
            entries.append(CopyEntry(src_off, dst_off, rows, row_elems, src_ld, dst_ld, 0))
            return
        S = src_shard_elems
        contiguous = (row_elems == src_ld) or rows == 1
        if contiguous:
            # a dense run of rows*row_elems elements: cut at slice boundaries, keep dst dense only if it is dense too
            total, done = rows * row_elems, 0
            while done < total:
                a = src_off + done
                r = a // S
                n = min(total - done, (r + 1) * S - a)
                if dst_ld == row_elems or rows == 1:
                    entries.append(CopyEntry(a - r * S, dst_off + done, 1, n, n, n, r))
                else:   # dense source, strided destination: go row by row inside this piece
                    p = 0
                    while p < n:
                        row, col = divmod(done + p, row_elems)
                        m = min(n - p, row_elems - col)
                        entries.append(CopyEntry(a + p - r * S, dst_off + row * dst_ld + col, 1, m, m, m, r))
                        p += m
                done += n
            return
        # strided source rows: runs of rows that lie entirely inside one slice stay one strided block; a row that
        # straddles a slice boundary is cut there
        i = 0
        while i < rows:
            a = src_off + i * src_ld
            r = a // S
            if (a + row_elems - 1) // S != r:
                emit(a, dst_off + i * dst_ld, 1, row_elems, row_elems, row_elems)
                i += 1
                continue
            # last row j >= i whose end is still inside slice r
            j = min(rows - 1, i + ((r + 1) * S - a - row_elems) // src_ld)
            entries.append(CopyEntry(a - r * S, dst_off + i * dst_ld, j - i + 1, row_elems, src_ld, dst_ld, r))
            i = j + 1

    for s, d in zip(src_specs, dst_specs):
        if len(s.shape) == 3 or len(s.shape) == 1 and tp == 1:
            emit(s.offset, d.offset, 1, s.numel, s.numel, s.numel)
            continue
        rows, cols = _tp_row_ranges(s.name, s.shape, cfg, tp_rank, tp, vocab_parallel)
        r_out = 0
        if len(s.shape) == 1:
            for a, b in rows:
                emit(s.offset + a, d.offset + r_out, 1, b - a, b - a, b - a)
                r_out += b - a
            continue
        ld = s.shape[1]
        width = cols[1] - cols[0]
        for a, b in rows:
            emit(s.offset + a * ld + cols[0], d.offset + r_out * width, b - a, width, ld, width)
            r_out += b - a
    size = dst_specs[-1].offset + (dst_specs[-1].numel + ALIGN - 1) // ALIGN * ALIGN
    for e in entries:
        assert e.row_elems % 8 == 0 and e.src_off % 8 == 0 and e.dst_off % 8 == 0 and e.src_ld % 8 == 0 \
            and e.dst_ld % 8 == 0, f"16-byte granularity violated: {e}"
    return entries, size


def run_plan_reference(entries: list[CopyEntry], srcs: list[torch.Tensor], dst: torch.Tensor) -> None:
    """Pure PyTorch executor (CPU tests; oracle for the kernel)."""
    for e in entries:
        src = srcs[e.src_rank]
        for r in range(e.rows):
            dst[e.dst_off + r * e.dst_ld: e.dst_off + r * e.dst_ld + e.row_elems] = \
                src[e.src_off + r * e.src_ld: e.src_off + r * e.src_ld + e.row_elems]


class ReshardPlan:
    """A plan uploaded to the device once; ``run`` is one kernel launch."""

    MAX_ROW_ELEMS = 1 << 30      # the record packs rows / row_elems / leading dimensions as int32

    @classmethod
    def split_large(cls, entries: list[CopyEntry]) -> list[CopyEntry]:
        """Cut single-row entries longer than MAX_ROW_ELEMS into chunks (a whole ZeRO shard of a 7B+ model is one
        contiguous run of several billion elements); multi-row entries must already fit."""
        out = []
        for e in entries:
            if e.rows == 1 and e.row_elems > cls.MAX_ROW_ELEMS:
                done = 0
                while done < e.row_elems:
                    n = min(cls.MAX_ROW_ELEMS, e.row_elems - done)
                    out.append(CopyEntry(e.src_off + done, e.dst_off + done, 1, n, n, n, e.src_rank))
                    done += n
            else:
                out.append(e)
        return out

    def __init__(self, entries: list[CopyEntry], device):
        import numpy as np

        entries = self.split_large(entries)
        lim = 2 ** 31 - 1
        for e in entries:
            if max(e.rows, e.row_elems, e.src_ld, e.dst_ld) > lim:
                raise ValueError(f"copy entry exceeds the int32 fields of the device record: {e}")

        rec = np.zeros(len(entries), dtype=[("src_off", "<i8"), ("dst_off", "<i8"), ("rows", "<i4"), ("row_elems", "<i4"),
                                            ("src_ld", "<i4"), ("dst_ld", "<i4"), ("src_rank", "<i4"), ("pad", "<i4")])
        for i, e in enumerate(entries):
            rec[i] = (e.src_off, e.dst_off, e.rows, e.row_elems, e.src_ld, e.dst_ld, e.src_rank, 0)
        self.n = len(entries)
        self.dev = torch.from_numpy(rec.view(np.uint8).copy()).to(device)

    def run(self, src_ptrs: list[int], dst: torch.Tensor, max_ctas: int = 0) -> None:
        """max_ctas > 0: launch about that many blocks only (a copy that overlaps compute kernels on another stream
        must leave room on every SM for them)."""
        from ..ops import _lib

        arr = (ctypes.c_void_p * len(src_ptrs))(*[ctypes.c_void_p(int(p)) for p in src_ptrs])
        rc = _lib.lib().b200_reshard_copy_budget(_lib.ptr(self.dev), ctypes.c_int(self.n), arr,
                                                 ctypes.c_int(len(src_ptrs)), _lib.ptr(dst), ctypes.c_int(max_ctas),
                                                 _lib.stream_ptr())
        _lib.check_rc(rc, "reshard_copy")
