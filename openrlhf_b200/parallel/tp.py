"""Tensor-parallel linear layers whose collective is fused into the GEMM kernel (rollout engine, TP > 1).

* ``row_parallel``: o_proj / down_proj. Each rank multiplies its K-slice; the GEMM epilogue adds every output tile
  into the fp32 accumulation buffer of *all* TP ranks with 16-byte ``red.add`` over NVLink, so when the flag barrier
  that follows has passed, every rank holds the all-reduced result. ``row_parallel_scatter`` is the reduce-scatter
  form: a tile goes only to the rank that owns its rows (vLLM runs a GEMM and then a custom all-reduce:
  the reference reaches it through ``--vllm.tensor_parallel_size``, openrlhf/trainer/ray/vllm_engine.py:270).
* ``column_parallel_gathered``: qkv / gate_up with sequence-parallel input. The activation rows live sharded over
  the ranks in a symmetric buffer; the A-tile TMA loads of the GEMM fetch each row block from its owner.

Accumulation buffers are double-buffered: buffer b is cleared locally while buffer 1-b is in use, and two flag
barriers per call order "all clears done -> pushes -> all pushes landed".
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from .symm import _ptr_array


class TPContext:
    def __init__(self, group, max_rows: int, max_cols: int, hidden: int, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.tp = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.max_rows, self.max_cols = max_rows, max_cols
        self.acc = [symm_mem.empty(max_rows * max_cols, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.acc_ptrs = []
        for a in self.acc:
            a.zero_()
            self.acc_ptrs.append(_ptr_array(symm_mem.rendezvous(a, self.group).buffer_ptrs))
        self.act = symm_mem.empty(max_rows * hidden, dtype=torch.bfloat16, device=self.device)
        self.act.zero_()
        self.act_ptrs = _ptr_array(symm_mem.rendezvous(self.act, self.group).buffer_ptrs)
        self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self.pad_ptrs = _ptr_array(symm_mem.rendezvous(self.pad, self.group).buffer_ptrs)
        self.epoch = 0
        self.cur = 0
        self.wait_limit_s = 20.0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self, channel: int = 2):
        self.epoch += 1
        rc = _lib.lib().b200_symm_barrier(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.tp),
                                          ctypes.c_int(channel), ctypes.c_uint(self.epoch),
                                          ctypes.c_double(self.wait_limit_s), _lib.ptr(_lib.status_word(self.device)),
                                          _lib.stream_ptr())
        _lib.check_rc(rc, "symm_barrier")

    def row_parallel(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """x [M, K_local], w [N, K_local] -> fp32 [M, N] = sum over TP ranks of x @ w.T (valid on every rank)."""
        M, K = x.shape
        N = w.shape[0]
        assert M * N <= self.max_rows * self.max_cols
        b = self.cur
        self.cur ^= 1
        self.acc[self.cur][: M * N].zero_()      # prepare the other buffer for the next call
        self.barrier(2)                          # every rank's buffer b is clean (cleared during the previous call)
        rc = _lib.lib().b200_gemm_bf16_tp(
            _lib.ptr(x), None, _lib.ptr(w), None, self.acc_ptrs[b], None, ctypes.c_int(M), ctypes.c_int(N),
            ctypes.c_int(K), ctypes.c_int(x.stride(0)), ctypes.c_int(w.stride(0)), ctypes.c_int(N),
            ctypes.c_int(self.tp), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0),
            _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_tp_push")
        self.barrier(3)                          # all pushes have landed everywhere
        return self.acc[b][: M * N].view(M, N)

    def row_parallel_scatter(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Reduce-scatter form of row_parallel: x [M, K_local], w [N, K_local] -> fp32 [M / tp, N], this rank's rows of
        sum over TP ranks of x @ w.T. Each output tile crosses NVLink once, to the owner of its rows only; feed the
        result (after the norm) to column_parallel_gathered, which reads the row shards from their owners."""
        M, K = x.shape
        N = w.shape[0]
        assert M % self.tp == 0 and (M // self.tp) * N <= self.max_rows * self.max_cols
        rows = M // self.tp
        b = self.cur
        self.cur ^= 1
        self.acc[self.cur][: min(M * N, self.max_rows * self.max_cols)].zero_()   # whatever form the next call has
        self.barrier(2)
        rc = _lib.lib().b200_gemm_bf16_tp(
            _lib.ptr(x), None, _lib.ptr(w), None, self.acc_ptrs[b], None, ctypes.c_int(M), ctypes.c_int(N),
            ctypes.c_int(K), ctypes.c_int(x.stride(0)), ctypes.c_int(w.stride(0)), ctypes.c_int(N),
            ctypes.c_int(self.tp), ctypes.c_int(rows), ctypes.c_int(2), ctypes.c_int(0),
            _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_tp_reduce_scatter")
        self.barrier(3)
        return self.acc[b][: rows * N].view(rows, N)

    def column_parallel_gathered(self, x_shard: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None):
        """x_shard [M/tp, K] (this rank's rows), w [N_local, K] -> bf16 [M, N_local] over the gathered rows."""
        rows, K = x_shard.shape
        assert rows % 128 == 0, "row shards must be multiples of the 128-row tile"
        self.act[: rows * K].view(rows, K).copy_(x_shard)
        self.barrier(4)                          # every rank's shard is in its symmetric buffer
        M, N = rows * self.tp, w.shape[0]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        rc = _lib.lib().b200_gemm_bf16_tp(
            None, self.act_ptrs, _lib.ptr(w), _lib.ptr(out), None, _lib.ptr(bias), ctypes.c_int(M), ctypes.c_int(N),
            ctypes.c_int(K), ctypes.c_int(K), ctypes.c_int(w.stride(0)), ctypes.c_int(N), ctypes.c_int(self.tp),
            ctypes.c_int(rows), ctypes.c_int(1), ctypes.c_int(0), _lib.ptr(_lib.status_word(self.device)),
            _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_tp_gather")
        self.barrier(5)                          # peers are done reading my shard before it is overwritten
        return out
