"""Tensor-parallel rollout: every rank of a TP group runs the same RolloutEngine (same requests, same scheduling,
same sampled tokens) on its shard of the weights.

* qkv / gate_up are column-parallel (each rank owns Hq/tp query heads, Hkv/tp kv heads and I/tp FFN columns, so its KV
  cache and decode attention cover only its heads);
* o_proj / down_proj are row-parallel: their split-K GEMMs leave fp32 slabs in a symmetric workspace and the fused
  "reduce + residual + RMSNorm" kernel that follows reads the slabs of ALL ranks through peer pointers, in a fixed
  order - the all-reduce costs no extra launch and every rank gets bit-identical activations, hence identical samples
  without any token broadcast;
* the device-side barrier between GEMM and reduction advances its own epoch counter, so the whole decode step stays
  inside one CUDA graph;
* weights arrive through the weight-sync copy plan (parallel/reshard.py) that slices the trainer's fused layouts.

The reference gets tensor-parallel rollout from vLLM (--vllm.tensor_parallel_size, openrlhf/trainer/ray/vllm_engine.py:270:
column / row parallel linears followed by a custom all-reduce kernel).
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.transformer import TransformerLM
from ..ops import _lib
from ..parallel.reshard import ReshardPlan, build_plan, tp_param_specs
from ..parallel.symm import _ptr_array
from .engine import RolloutEngine


def local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0 and cfg.intermediate_size % tp == 0
    return dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // tp,
                               num_key_value_heads=cfg.num_key_value_heads // tp,
                               intermediate_size=cfg.intermediate_size // tp, head_dim=cfg.head_dim)


class TPDecode:
    """Symmetric workspaces, barrier state and the weight-shard plan of one TP rank."""

    def __init__(self, cfg: ModelConfig, group, max_rows: int, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.cfg = cfg
        n = 32 * max_rows * cfg.hidden_size          # up to 32 split-K slabs of [rows, hidden]
        self.ws = [symm_mem.empty(n, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.ws_ptrs = [_ptr_array(symm_mem.rendezvous(w, self.group).buffer_ptrs) for w in self.ws]
        self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self.pad_ptrs = _ptr_array(symm_mem.rendezvous(self.pad, self.group).buffer_ptrs)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)   # advanced by the barrier kernel itself
        entries, self.shard_numel = build_plan(cfg, self.rank, self.size)
        self.plan = ReshardPlan(entries, self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self):
        rc = _lib.lib().b200_symm_barrier_dev(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.size),
                                              ctypes.c_int(3), _lib.ptr(self.epoch), ctypes.c_double(20.0),
                                              _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "symm_barrier_dev")

    def load_shard(self, full_flat: torch.Tensor, shard_flat: torch.Tensor):
        """full_flat: the trainer's flat bf16 parameter buffer on this GPU; shard_flat: the engine's buffer."""
        self.plan.run([full_flat.data_ptr()], shard_flat)


def make_tp_engine(cfg: ModelConfig, full_flat: torch.Tensor, group=None, **engine_kwargs) -> RolloutEngine:
    """Build this rank's tensor-parallel rollout engine from the full flat parameter buffer on its GPU."""
    device = full_flat.device
    group = group if group is not None else dist.group.WORLD
    tp = dist.get_world_size(group)
    lcfg = local_config(cfg, tp)
    model = TransformerLM(lcfg, device=device, seed=None)
    want = tp_param_specs(cfg, dist.get_rank(group), tp)
    assert [(s.name, s.shape, s.offset) for s in model.specs] == [(s.name, s.shape, s.offset) for s in want], \
        "shard layout of the local model and of the copy plan differ"
    model.tp_group = group
    model.requires_grad_(False)
    ctx = TPDecode(cfg, group, engine_kwargs.get("max_num_seqs", 256), device)
    ctx.load_shard(full_flat, model.flat)
    return RolloutEngine(model, tp=ctx, **engine_kwargs)
