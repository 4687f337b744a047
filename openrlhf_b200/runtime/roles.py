"""Builders for the roles an RL worker hosts: trainable models with their ZeRO engine, frozen models, rollout engines.

One place decides how ``--ds.zero_stage``, ``--ds.ring_attn_size``, ``--ds.tensor_parallel_size``,
``--ds.adam_offload`` and ``--vllm.tensor_parallel_size`` turn into engines, so that the controller-driven worker
(``runtime/workers.py``), the SPMD hybrid worker (``trainer/hybrid_engine.py``) and the benchmark all run the same
objects. The reference makes the same decisions in ``DeepspeedStrategy.prepare`` (training engines:
openrlhf/utils/deepspeed/deepspeed.py:389-429, inference engines for frozen models: :460-487) and in
``create_vllm_engines`` (openrlhf/trainer/ray/vllm_engine.py:213-300).
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
import torch.distributed as dist

from ..models.hf_io import load_pretrained
from ..parallel.zero import LRScheduler, ZeroEngine


def _scheduler(node, max_steps: int) -> LRScheduler:
    return LRScheduler(node.adam.lr, max_steps, getattr(node, "lr_warmup_ratio", 0.03),
                       getattr(node, "min_lr_ratio", 0.1), getattr(node, "lr_scheduler", "cosine_with_min_lr"))


def use_zero3(strategy) -> bool:
    """Stage 3 shards parameters, gradients and optimizer state over the zero group; with one rank there is nothing
    to shard and the stage-2 engine (same arithmetic) is used."""
    return int(strategy.stage) == 3 and strategy.zero_world > 1 and dist.is_available() and dist.is_initialized()


def build_trainable(strategy, path: str, node: SimpleNamespace, *, device, max_steps: int, seed: int,
                    with_lm_head: bool = True, with_value_head: bool = False, value_head_prefix: str | None = None,
                    use_symm: bool | None = None):
    """Load (or random-init) a model and attach its training engine. Returns (model, engine, rollout_source) where
    rollout_source tells a colocated rollout engine where its weights come from:
    ("alias", model) - the engine may read the trainer's own buffer; ("zero3", engine) - parameters are sharded, the
    engine needs a copy of its own refreshed by the gather kernel; ("tp_train", model) - tensor-parallel shards."""
    a = strategy.args
    zw = strategy.zero_world
    lm = load_pretrained(path, device=device, with_lm_head=with_lm_head, with_value_head=with_value_head,
                         shard_world=zw, seed=seed, value_head_prefix=value_head_prefix)
    tp_train = strategy.ds_tensor_parallel_size > 1 and strategy.world_size > 1
    z3 = use_zero3(strategy)
    if z3 and tp_train:
        raise ValueError("--ds.zero_stage 3 is not combined with --ds.tensor_parallel_size > 1; use stage 2")
    source = ("alias", lm)
    if tp_train:
        from ..parallel.tp_train import shard_for_training

        lm = shard_for_training(lm, strategy.mesh.group("tp"), shard_world=zw)
        source = ("tp_train", lm)
    ep_range = strategy.attach_expert_parallel(lm, strategy.ep_max_tokens())
    opt = dict(lr=node.adam.lr, betas=tuple(node.adam.betas), eps=node.adam.eps, weight_decay=node.adam.weight_decay,
               max_norm=getattr(node, "max_norm", 1.0), group=strategy.zero_group(), scheduler=_scheduler(node, max_steps))
    if z3:
        from ..parallel.zero3 import Zero3Engine

        engine = Zero3Engine(lm, expert_range=ep_range, **opt)
        source = ("zero3", engine)
    else:
        engine = ZeroEngine(lm, zero_stage=int(strategy.stage), use_symm=False if tp_train else use_symm,
                            adam_offload=bool(getattr(a.ds, "adam_offload", False)), **opt)
    return lm, engine, source


def build_frozen(strategy, path: str, *, device, seed: int, with_lm_head: bool = True, with_value_head: bool = False,
                 value_head_prefix: str | None = None, offload: bool = False):
    """A model that only runs forward passes (reference policy, reward model). Under ZeRO stage 3 its parameters are
    sharded over the zero group and gathered layer by layer; with tensor-parallel training it is sharded over the TP
    group; otherwise every rank keeps a replica (on the host when `offload`)."""
    dev = "cpu" if offload else device
    lm = load_pretrained(path, device=dev, with_lm_head=with_lm_head, with_value_head=with_value_head, seed=seed,
                         shard_world=strategy.zero_world, value_head_prefix=value_head_prefix)
    lm.requires_grad_(False)
    if offload:
        return lm
    if strategy.ds_tensor_parallel_size > 1 and strategy.world_size > 1:
        from ..parallel.tp_train import shard_for_training

        lm = shard_for_training(lm, strategy.mesh.group("tp"))
        lm.requires_grad_(False)
    elif use_zero3(strategy):
        from ..parallel.zero3 import Zero3Engine

        ep_range = strategy.attach_expert_parallel(lm, strategy.ep_max_tokens())
        Zero3Engine(lm, group=strategy.zero_group(), train=False, expert_range=ep_range)   # attaches itself as lm.z3
    else:
        strategy.attach_expert_parallel(lm, strategy.ep_max_tokens())
    return lm


def rollout_tp_groups(world: int, tp: int, rank: int, first: int = 0, count: int | None = None):
    """Process groups of the tensor-parallel rollout engines: consecutive ranks [first + k*tp, first + (k+1)*tp).
    Every rank of the world must call this (group creation is collective). Returns
    (device group, gloo control group, ranks of my group) or (None, None, None) for a rank outside every group."""
    count = (world - first) // tp if count is None else count
    mine = (None, None, None)
    for k in range(count):
        ranks = list(range(first + k * tp, first + (k + 1) * tp))
        g = dist.new_group(ranks)
        ctl = dist.new_group(ranks, backend="gloo")
        if rank in ranks:
            mine = (g, ctl, ranks)
    return mine


def build_rollout(strategy, cfg, source, *, device, seed: int, tokenizer=None, tp_groups=(None, None, None),
                  max_num_seqs: int = 256, num_pages: int | None = None, use_cuda_graph: bool = True,
                  path: str | None = None):
    """The rollout engine of this rank. `source` comes from build_trainable (or ("load", path) for a rollout-only
    rank). Returns (engine, rollout_model, sync) where sync() refreshes the engine's weights from the trainer."""
    from ..models.transformer import TransformerLM
    from ..rollout.engine import RolloutEngine

    a = strategy.args
    kind, obj = source
    tp_group, tp_ctl, tp_ranks = tp_groups
    kw = dict(max_num_seqs=max_num_seqs, max_model_len=a.data.max_len, num_pages=num_pages,
              gpu_memory_utilization=a.vllm.gpu_memory_utilization, use_cuda_graph=use_cuda_graph,
              eos_token_id=getattr(tokenizer, "eos_token_id", None))
    quant = getattr(a.vllm, "quantization", None)
    prefix_cache = bool(getattr(a.vllm, "enable_prefix_caching", False))
    if tp_group is not None:
        from ..rollout.tp_engine import TPLockstepEngine, make_tp_engine

        if quant:
            raise ValueError("--vllm.quantization is not combined with --vllm.tensor_parallel_size > 1")
        tp = len(tp_ranks)
        # every member of the engine gets the same seed: identical samples on every rank without a token broadcast
        eng = make_tp_engine(cfg, source, tp_group, seed=seed + 1000 * (tp_ranks[0] // tp),
                             enable_prefix_caching=prefix_cache, **kw)
        lock = TPLockstepEngine(eng, tp_ctl, leader=tp_ranks[0], is_leader=strategy.rank == tp_ranks[0])
        return lock, eng.model, lambda: eng.tp.refresh(eng.model.flat)
    kw["enable_prefix_caching"] = prefix_cache
    if kind == "alias":
        eng = RolloutEngine(obj, seed=seed + strategy.rank, quantization=quant, **kw)
        return eng, obj, lambda: eng.update_weights(obj.flat)
    if kind == "load":
        model = load_pretrained(obj, device=device, seed=seed)
        model.requires_grad_(False)
        eng = RolloutEngine(model, seed=seed + strategy.rank, quantization=quant, **kw)
        return eng, model, None
    # the trainer holds shards (ZeRO-3 slices or tensor-parallel shards): the engine owns a full copy
    full = TransformerLM(cfg, device=device, seed=None, shard_world=strategy.zero_world)
    full.requires_grad_(False)
    if kind == "zero3":
        def sync():
            obj.gather_full(full.flat)           # K-SYNC: one copy kernel over the owners' parameter slices
            eng.update_weights(full.flat)
    else:
        def sync():
            eng.update_weights(obj.tp_train.gather_full(obj))
    eng = RolloutEngine(full, seed=seed + strategy.rank, quantization=quant, **kw)
    sync()
    return eng, full, sync
