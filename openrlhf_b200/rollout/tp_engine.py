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
from ..parallel.reshard import ReshardPlan, build_plan, run_plan_reference, tp_param_specs
from .engine import RolloutEngine


def local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0 and cfg.intermediate_size % tp == 0
    return dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // tp,
                               num_key_value_heads=cfg.num_key_value_heads // tp,
                               intermediate_size=cfg.intermediate_size // tp, head_dim=cfg.head_dim)


class TPDecode:
    """Symmetric workspaces, barrier state and the weight-shard plan of one TP rank.

    `source` says where the weights come from at every sync (see runtime/roles.py::build_trainable):
    ("alias", model)  the trainer's full flat buffer on this GPU: the plan slices it locally;
    ("zero3", engine) ZeRO-3 parameter slices spread over the zero group: the plan reads every piece from its owner's
                      slice over peer memory, so the full layout is never assembled anywhere;
    ("full", tensor)  a plain full flat buffer.
    CPU ranks (tests of the control flow) run the same plans with the PyTorch executor and all-reduce the row-parallel
    projections over the group."""

    def __init__(self, cfg: ModelConfig, group, max_rows: int, device, source=None):
        self.group = group if group is not None else dist.group.WORLD
        self.size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.cfg = cfg
        self.source = source
        kind = source[0] if source is not None else "full"
        self.z3 = source[1] if kind == "zero3" else None
        if self.z3 is not None and self.on_gpu and self.z3.world > 1:
            entries, self.shard_numel = build_plan(cfg, self.rank, self.size, src_world=self.z3.world,
                                                   src_shard_elems=self.z3.per)
        else:
            entries, self.shard_numel = build_plan(cfg, self.rank, self.size)
        self.entries = entries
        if not self.on_gpu:
            return
        import torch.distributed._symmetric_memory as symm_mem

        from ..parallel.symm import _ptr_array

        n = 32 * max_rows * cfg.hidden_size          # up to 32 split-K slabs of [rows, hidden]
        self.ws = [symm_mem.empty(n, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.ws_ptrs = [_ptr_array(symm_mem.rendezvous(w, self.group).buffer_ptrs) for w in self.ws]
        self.pad = symm_mem.empty(1024, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self.pad_ptrs = _ptr_array(symm_mem.rendezvous(self.pad, self.group).buffer_ptrs)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)   # advanced by the barrier kernel itself
        self.plan = ReshardPlan(entries, self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self):
        rc = _lib.lib().b200_symm_barrier_dev(self.pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.size),
                                              ctypes.c_int(3), _lib.ptr(self.epoch), ctypes.c_double(20.0),
                                              _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "symm_barrier_dev")

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def load_shard(self, full_flat: torch.Tensor, shard_flat: torch.Tensor):
        """full_flat: a full flat bf16 parameter buffer on this device; shard_flat: the engine's buffer."""
        if self.z3 is not None and self.on_gpu and self.z3.world > 1:
            raise ValueError("this engine is fed from ZeRO-3 slices; call refresh()")
        if self.on_gpu:
            self.plan.run([full_flat.data_ptr()], shard_flat)
        else:
            run_plan_reference(self.entries, [full_flat], shard_flat)

    @torch.no_grad()
    def refresh(self, shard_flat: torch.Tensor):
        """Weight sync from the configured source into this rank's shard: one copy kernel."""
        kind, obj = self.source
        if kind == "zero3":
            if self.on_gpu and obj.world > 1:
                self.plan.run(obj.param_ptrs, shard_flat)      # every piece straight from its owner's slice
            else:
                self.load_shard(obj.gather_full(), shard_flat)
        elif kind == "tp_train":
            self.load_shard(obj.tp_train.gather_full(obj), shard_flat)
        else:
            self.load_shard(obj.flat if hasattr(obj, "flat") else obj, shard_flat)


def make_tp_engine(cfg: ModelConfig, source, group=None, **engine_kwargs) -> RolloutEngine:
    """Build this rank's tensor-parallel rollout engine. `source`: a full flat parameter tensor on this rank's device,
    or a (kind, object) pair as described at TPDecode."""
    if isinstance(source, torch.Tensor):
        source = ("full", source)
    kind, obj = source
    device = (obj.device if kind in ("full", "zero3") else obj.flat.device)
    group = group if group is not None else dist.group.WORLD
    tp = dist.get_world_size(group)
    lcfg = local_config(cfg, tp)
    dtype = (obj if kind == "full" else (obj.param_shard if kind == "zero3" else obj.flat)).dtype
    model = TransformerLM(lcfg, device=device, seed=None, dtype=dtype)
    want = tp_param_specs(cfg, dist.get_rank(group), tp)
    assert [(s.name, s.shape, s.offset) for s in model.specs] == [(s.name, s.shape, s.offset) for s in want], \
        "shard layout of the local model and of the copy plan differ"
    model.tp_group = group
    model.requires_grad_(False)
    ctx = TPDecode(cfg, group, engine_kwargs.get("max_num_seqs", 256), device, source)
    ctx.refresh(model.flat)
    return RolloutEngine(model, tp=ctx, **engine_kwargs)


class TPLockstepEngine:
    """Keeps the members of one tensor-parallel rollout engine in lockstep under a single controller.

    Only the leader (first rank of the TP group) receives requests. Before every ``step()`` it broadcasts the requests
    that arrived since the previous step over a host-side (gloo) control group; the followers sit in ``follow()``,
    add the same requests in the same order and run the same step. The engines are deterministic functions of their
    request stream (same scheduling, same sampler seed, bit-identical activations after the fused all-reduce), so
    every member admits, samples and retires the same rows without exchanging tokens. ``stop_followers()`` ends a
    generation phase. The reference leaves this to vLLM's multi-process executor
    (openrlhf/trainer/ray/vllm_engine.py:213-300, ``distributed_executor_backend``)."""

    def __init__(self, engine: RolloutEngine, ctrl_group, leader: int, is_leader: bool):
        self.engine = engine
        self.ctrl = ctrl_group
        self.leader = leader               # global rank of the leader (source of the broadcasts)
        self.is_leader = is_leader
        self._new: list = []
        self.following = False

    def __getattr__(self, name):
        return getattr(self.__dict__["engine"], name)

    def _bcast(self, msg):
        box = [msg]
        dist.broadcast_object_list(box, src=self.leader, group=self.ctrl)
        return box[0]

    # ---- leader side (same surface as RolloutEngine)
    def add_request(self, request_id, prompt_token_ids, sampling_params, multi_modal_data=None):
        assert self.is_leader, "requests go to the leader of a tensor-parallel rollout engine"
        self._new.append((request_id, list(prompt_token_ids), sampling_params, multi_modal_data))

    def has_unfinished(self) -> bool:
        return bool(self._new) or self.engine.has_unfinished()

    def step(self):
        assert self.is_leader
        new, self._new = self._new, []
        self._bcast(("step", new, self.engine.paused))
        for r in new:
            self.engine.add_request(*r)
        return self.engine.step()

    def stop_followers(self):
        if self.is_leader:
            self._bcast(("stop", None, False))

    def generate(self, prompt_token_ids, sampling_params, request_ids=None, multi_modal_data=None):
        """Blocking batch generation: on the leader, with the followers inside follow(); or, after spmd(), on every
        member with identical arguments (no control traffic needed)."""
        if self._spmd:
            return self.engine.generate(prompt_token_ids, sampling_params, request_ids, multi_modal_data)
        return self._leader_generate(prompt_token_ids, sampling_params, request_ids, multi_modal_data)

    _spmd = False

    def spmd(self, on: bool = True):
        """SPMD callers (every member issues identical generate() calls) bypass the control channel."""
        self._spmd = on
        return self

    def _leader_generate(self, prompts, sps, request_ids=None, mmd=None):
        from .engine import SamplingParams

        if isinstance(sps, SamplingParams):
            sps = [sps] * len(prompts)
        base = self.engine._batch_counter
        self.engine._batch_counter += len(prompts)
        keys = [("batch", base + i) for i in range(len(prompts))]
        for k, p, sp, mm in zip(keys, prompts, sps, mmd or [None] * len(keys)):
            self.add_request(k, p, sp, mm)
        got = {}
        while len(got) < len(keys):
            for ro in self.step():
                got[ro.request_id] = ro
        outs = []
        for i, k in enumerate(keys):
            ro = got[k]
            ro.request_id = request_ids[i] if request_ids else i
            outs.append(ro)
        return outs

    # ---- follower side
    def follow(self) -> int:
        """Mirror the leader until it calls stop_followers(); returns the number of mirrored steps."""
        assert not self.is_leader
        n = 0
        self.following = True
        try:
            while True:
                kind, new, paused = self._bcast(None)
                if kind == "stop":
                    return n
                self.engine.paused = paused
                for r in new:
                    self.engine.add_request(*r)
                self.engine.step()
                n += 1
        finally:
            self.following = False
