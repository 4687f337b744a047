"""Worker-side classes of the RL runtime: one ``RLWorker`` process per GPU hosts the roles placed on that GPU.

Roles and their RPC surface mirror the reference's Ray actors (openrlhf/trainer/ray/ppo_actor.py:494-682 policy,
ppo_critic.py:186-324 critic, launcher.py:104-199 reference / reward, vllm_engine.py:63-208 rollout):

* rollout : ``generate_responses`` (n agent-executor coroutines per prompt over the async engine), ``sleep``,
            ``wake_up``, ``pause_generation``, ``resume_generation``, ``reset_prefix_cache``,
            ``get_num_unfinished_requests``
* actor   : ``forward`` (old log-probs), ``append``, ``fit``, ``broadcast_to_vllm``, ``save_model``,
            ``save_checkpoint``, ``get_checkpoint_states``, ``offload_states`` / ``reload_states``
* critic  : ``forward`` (values), ``append``, ``fit``, ``save_model``, ``save_checkpoint``
* ref / reward : ``forward``

All tensors crossing the process boundary are CPU tensors (shared memory). With ``--train.colocate_all`` every
worker holds every role and the rollout engine reads the buffer the actor's optimizer writes.
"""
from __future__ import annotations

import asyncio
import copy
import os
from types import SimpleNamespace

import torch
import torch.distributed as dist

from ..models.actor import Actor
from ..models.hf_io import load_pretrained
from ..models.loss import PolicyLoss, ValueLoss
from ..models.model import CriticModel, RewardModel
from ..models.utils import masked_mean
from ..ops import rl as K
from ..parallel.zero import LRScheduler, ZeroEngine
from ..rl.experience import Experience
from ..rl.replay_buffer import NaiveReplayBuffer
from ..rollout.async_engine import AsyncRolloutEngine
from ..rollout.engine import RolloutEngine, SamplingParams
from ..utils import checkpoint as ckpt
from ..utils.agent import AgentExecutorBase, SingleTurnAgentExecutor, load_python_object
from ..utils.loss_utils import get_loss_batch_info
from ..utils.strategy import Strategy, get_strategy
from ..utils.utils import get_tokenizer

ALL_ROLES = ("actor", "critic", "ref", "reward", "rollout")


def _bcast_opts(root: int):
    o = dist.BroadcastOptions()
    o.rootRank = root
    o.rootTensor = 0
    return o


def _cpu(x):
    return x.detach().to("cpu") if isinstance(x, torch.Tensor) else x


def _mm_kwargs(mm_train_inputs, device) -> dict:
    """Per-sample image inputs of a batch (list of dicts or None) -> keyword arguments of Actor.forward
    (openrlhf/trainer/ray/ppo_actor.py merges them the same way before the policy forward)."""
    if not mm_train_inputs or not any(mm_train_inputs):
        return {}
    from ..utils.vlm_utils import merge_mm_train_inputs

    return merge_mm_train_inputs(mm_train_inputs, device)


class RLWorker:
    """One process per GPU hosting the roles placed there. Every parallelism / memory flag takes effect here or raises:

    * ``--ds.zero_stage 3``: actor and critic train under ``Zero3Engine`` (parameters, gradients and optimizer state
      sharded, layer gathers and per-layer gradient reductions as peer-memory kernels); the frozen reference and reward
      models hold parameter slices only and gather layer by layer as well. Stages 1 / 2 run the ``ZeroEngine`` whose
      multi-rank optimizer step is the fused reduce + AdamW + parameter-store kernel pair over symmetric memory.
    * ``--ds.ring_attn_size``: every forward / training pass receives the context-parallel group.
    * ``--ds.tensor_parallel_size``: tensor-parallel training shards (parallel/tp_train.py).
    * ``--vllm.tensor_parallel_size``: consecutive ranks form one tensor-parallel rollout engine that the controller
      drives through its leader (rollout/tp_engine.py::TPLockstepEngine).
    * ``--ds.adam_offload``: optimizer state lives in pinned host memory between steps (stages 1 / 2).
    """

    def __init__(self, args: SimpleNamespace, roles=ALL_ROLES, max_steps: int = 1000, backend: str | None = None,
                 engine_opts: dict | None = None):
        self.args = args
        self.roles = set(roles)
        self.strategy: Strategy = get_strategy(args)
        self.strategy.setup_distributed(backend=backend)
        self.device = self.strategy.device()
        s = self.strategy
        self.actor = self.actor_engine = self.critic = self.critic_engine = None
        self.ref = self.reward = self.rollout = self.async_engine = self.ema_model = None
        self._sync_fn = None
        self._sync_pg = None
        self._rollout_source = None
        a = args
        temp = a.rollout.temperature
        seed = a.train.seed
        eo = dict(engine_opts or {})
        if getattr(a.ds, "adam_offload", False) and int(a.ds.zero_stage) == 3 and s.zero_world > 1:
            raise ValueError("--ds.adam_offload is available with ZeRO stages 1 / 2; stage 3 already shards the "
                             "optimizer state over the ranks")
        # tensor-parallel rollout engines: group creation is collective, so every rank of the world takes part even
        # when it hosts no rollout role
        self.rollout_tp = int(getattr(a.vllm, "tensor_parallel_size", 1) or 1)
        self._tp_groups = (None, None, None)
        if self.rollout_tp > 1:
            if s.world_size % self.rollout_tp:
                raise ValueError(f"--vllm.tensor_parallel_size {self.rollout_tp} does not divide the {s.world_size} "
                                 "workers that host rollout engines")
            if a.train.async_enable and "actor" in self.roles:
                raise ValueError("--train.async_enable with colocated tensor-parallel rollout engines is not "
                                 "supported: followers mirror their leader for whole generation phases")
            from .roles import rollout_tp_groups

            self._tp_groups = rollout_tp_groups(s.world_size, self.rollout_tp, s.rank)
        if "actor" in self.roles:
            from .roles import build_trainable

            lm, self.actor_engine, self._rollout_source = build_trainable(
                s, a.actor.model_name_or_path, a.actor, device=self.device, max_steps=max_steps, seed=seed,
                use_symm=eo.get("use_symm"))
            self.actor = Actor(lm, temperature=temp, packing_samples=a.ds.packing_samples,
                               freeze_visual_encoder=getattr(a.actor, "freeze_visual_encoder", False))
            if a.actor.gradient_checkpointing_enable:
                self.actor.gradient_checkpointing_enable()
            lo, hi = a.actor.eps_clip_low_high
            self.policy_loss = PolicyLoss(lo, hi, a.actor.dual_clip, policy_loss_type=a.actor.policy_loss_type,
                                          enable_vllm_is_correction=a.algo.advantage.is_correction_enable,
                                          vllm_is_truncated_threshold=a.algo.advantage.is_correction_threshold,
                                          vllm_is_correction_type=a.algo.advantage.is_correction_type)
            self.actor_buffer = NaiveReplayBuffer(a.train.micro_batch_size, 0, True, a.ds.packing_samples,
                                                  a.train.dynamic_batch_enable)
            if a.train.enable_ema:
                if self._rollout_source[0] != "alias":
                    raise ValueError("--train.enable_ema needs the full parameter buffer on every rank (ZeRO stage "
                                     "<= 2 without tensor-parallel training)")
                # the moving average lives on the device in fp32 and is updated by one fused elementwise pass
                n = lm.total_numel
                self.ema_flat = lm.flat[:n].float().clone()
                self.ema_model = True
            if a.ckpt.load_enable and os.path.exists(os.path.join(a.ckpt.path, "_actor")):
                _, self._resume_states = s.load_ckpt(SimpleNamespace(engine=self.actor_engine),
                                                     os.path.join(a.ckpt.path, "_actor"))
            else:
                self._resume_states = {}
        if "critic" in self.roles and a.critic.model_name_or_path:
            from .roles import build_trainable

            lm, self.critic_engine, _ = build_trainable(
                s, a.critic.model_name_or_path, a.critic, device=self.device, max_steps=max_steps, seed=seed + 1,
                with_lm_head=False, with_value_head=True, value_head_prefix=a.ds.value_head_prefix,
                use_symm=eo.get("use_symm"))
            self.critic = CriticModel(lm, normalize_reward=a.reward.normalize_enable,
                                      packing_samples=a.ds.packing_samples)
            if a.actor.gradient_checkpointing_enable:
                self.critic.gradient_checkpointing_enable()
            self.value_loss = ValueLoss(a.critic.value_clip)
            self.critic_buffer = NaiveReplayBuffer(a.train.micro_batch_size, 0, True, a.ds.packing_samples,
                                                   a.train.dynamic_batch_enable)
            if a.ckpt.load_enable and os.path.exists(os.path.join(a.ckpt.path, "_critic")):
                ckpt.load_sharded(self.critic_engine, os.path.join(a.ckpt.path, "_critic"))
        if "ref" in self.roles and a.algo.kl.init_coef > 0:
            from .roles import build_frozen

            lm = build_frozen(s, a.ref.model_name_or_path or a.actor.model_name_or_path, device=self.device, seed=seed,
                              offload=a.ref.offload)
            self.ref = Actor(lm, temperature=temp, packing_samples=a.ds.packing_samples).eval()
        if "reward" in self.roles and a.reward.model_name_or_path:
            from .roles import build_frozen

            lm = build_frozen(s, a.reward.model_name_or_path, device=self.device, seed=seed + 2, with_lm_head=False,
                              with_value_head=True, value_head_prefix=a.ds.value_head_prefix, offload=a.reward.offload)
            self.reward = RewardModel(lm, normalize_reward=a.reward.normalize_enable,
                                      packing_samples=a.ds.packing_samples).eval()
        if "rollout" in self.roles:
            from ..models.config import ModelConfig
            from .roles import build_rollout

            self.tokenizer = get_tokenizer(a.actor.model_name_or_path, None, "left", s,
                                           use_fast=not a.data.disable_fast_tokenizer)
            source = self._rollout_source or ("load", a.actor.model_name_or_path)
            cfg = self.actor.cfg if self.actor is not None else ModelConfig.from_pretrained(a.actor.model_name_or_path)
            if self._rollout_source is not None and self._rollout_source[0] == "tp_train":
                cfg = self._rollout_source[1].tp_train.full_cfg
            if self.rollout_tp > 1 and source[0] == "load":
                full = load_pretrained(a.actor.model_name_or_path, device=self.device, seed=seed)
                full.requires_grad_(False)
                self._staging = full
                source = ("alias", full)
            self.rollout, self.rollout_model, self._sync_fn = build_rollout(
                s, cfg, source, device=self.device, seed=seed, tokenizer=self.tokenizer, tp_groups=self._tp_groups,
                max_num_seqs=eo.get("max_num_seqs", getattr(a.vllm, "max_num_seqs", 256)),
                num_pages=eo.get("num_pages"), use_cuda_graph=eo.get("use_cuda_graph", not a.vllm.enforce_eager))
            # vision-language models: the processor's image part turns the PIL images an agent passes into patches
            self.rollout.image_processor = getattr(self.tokenizer, "image_processor", None)
            self.is_rollout_leader = self._tp_groups[2] is None or s.rank == self._tp_groups[2][0]
            self.async_engine = AsyncRolloutEngine(self.rollout, self.tokenizer)
            if a.train.agent_func_path:
                cls = load_python_object(a.train.agent_func_path, "AgentExecutor")
                if not issubclass(cls, AgentExecutorBase):
                    raise AssertionError("AgentExecutor must inherit from AgentExecutorBase")
                self.executor = cls()
            else:
                self.executor = SingleTurnAgentExecutor(a.reward.remote_url)
            if a.vllm.enable_sleep:
                self.rollout.sleep()

    # ------------------------------------------------------------------ generic
    def execute_batch(self, method_name: str, chunk: dict):
        """Run `method_name` once per item of the chunk (lists of equal length) and return the list of results."""
        n = len(next(iter(chunk.values())))
        fn = getattr(self, method_name)
        return [fn(**{k: v[i] for k, v in chunk.items()}) for i in range(n)]

    def empty_cache(self):
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
            torch.cuda.synchronize()

    def ping(self):
        return {"rank": self.strategy.rank, "roles": sorted(self.roles)}

    def shutdown(self):
        if dist.is_initialized():
            dist.destroy_process_group()

    # ------------------------------------------------------------------ rollout role
    async def generate_responses(self, prompt, label, sampling_params: SamplingParams, max_length: int,
                                 num_samples: int = 1, images=None, hf_tokenizer=None):
        jobs = [self.executor.execute(prompt=prompt, label=label, sampling_params=copy.deepcopy(sampling_params),
                                      max_length=max_length, hf_tokenizer=hf_tokenizer or self.tokenizer,
                                      llm_engine=self.async_engine, images=images) for _ in range(num_samples)]
        return await asyncio.gather(*jobs)

    def get_num_unfinished_requests(self) -> int:
        return self.async_engine.get_num_unfinished_requests()

    def follow_generation(self) -> int:
        """Follower of a tensor-parallel rollout engine: mirror the leader's steps until it ends the phase."""
        return self.rollout.follow()

    def end_generation(self) -> bool:
        """Leader of a tensor-parallel rollout engine: release the followers at the end of a generation phase."""
        if hasattr(self.rollout, "stop_followers"):
            self.rollout.stop_followers()
        return True

    def sleep(self, level: int = 1):
        self.rollout.sleep(level)

    def wake_up(self, tags=None):
        self.rollout.wake_up(tags)

    def pause_generation(self):
        self.rollout.pause_generation()

    def resume_generation(self):
        self.rollout.resume_generation()

    def reset_prefix_cache(self):
        return self.rollout.reset_prefix_cache()

    # ------------------------------------------------------------------ inference forwards (one micro-batch per call)
    @torch.no_grad()
    def forward(self, sequences, action_mask, attention_mask, role: str = "actor", mm_train_inputs=None, **_unused):
        seq, am, att = sequences.to(self.device), action_mask.to(self.device), attention_mask.to(self.device)
        cp = self.strategy.ring_attn_group
        if role == "critic":
            self.critic.eval()
            out = self.critic(seq, am, att, ring_attn_group=cp)
            self.critic.train()
        else:
            model = self.actor if role == "actor" else self.ref
            dev = next(model.parameters()).device
            was = model.training
            model.eval()
            out = model(seq.to(dev), am.to(dev), att.to(dev), ring_attn_group=cp if dev.type == "cuda" else None,
                        **_mm_kwargs(mm_train_inputs, dev))
            model.train(was)
        return _cpu(out)

    @torch.no_grad()
    def forward_reward(self, sequences, attention_mask, pad_sequence=True, **_unused):
        dev = next(self.reward.parameters()).device
        cp = self.strategy.ring_attn_group if dev.type == "cuda" else None
        return _cpu(self.reward(sequences.to(dev), attention_mask.to(dev), ring_attn_group=cp))

    # ------------------------------------------------------------------ training
    def append(self, experience: Experience, role: str = "actor"):
        (self.actor_buffer if role == "actor" else self.critic_buffer).append(experience)

    def _loader(self, buffer):
        s = self.strategy
        if self.args.train.dynamic_batch_enable:
            buffer.setup_dynamic_batch(s)
        # duplicates of one replica (context / tensor parallel ranks) must see identical batches: no shuffling
        shuffle = s.ring_attn_size == 1 and s.ds_tensor_parallel_size == 1 and not self.args.train.dynamic_batch_enable
        from torch.utils.data import DataLoader

        return DataLoader(buffer, batch_size=buffer.sample_batch_size, shuffle=shuffle, drop_last=False,
                          collate_fn=buffer.collate_fn)

    def _windows(self, buffer, loader):
        """Yield (experience, normalisers, is_last_micro_batch_of_step)."""
        a = self.args
        if a.train.dynamic_batch_enable:
            for step, exp in enumerate(loader):
                info = get_loss_batch_info(self.strategy, exp.action_mask, replay_buffer=buffer, step=step,
                                           dynamic_batch=True)
                yield exp, info, bool(buffer.dynamic_optimizer_step[step])
            return
        gas = self.strategy.accumulated_gradient
        pending = []
        items = list(loader)
        for i, exp in enumerate(items):
            pending.append(exp)
            if len(pending) == gas or i == len(items) - 1:
                tot = torch.zeros(2, dtype=torch.float64)
                for e in pending:
                    m = e.action_mask.float()
                    tot[0] += m.sum()
                    tot[1] += (m.sum(-1) > 0).sum()
                # totals of the optimizer-step window over the data-parallel group only (context- / tensor-parallel
                # duplicates hold the same samples and must not be counted again), divided by gas because every
                # micro-loss is divided by gas once more before backward (openrlhf/utils/loss_utils.py:62-80)
                tot = self._dp_sum(tot)
                info = {"dp_size": self.strategy.mesh.dp, "batch_num_tokens": float(tot[0]) / gas,
                        "global_batch_size": float(tot[1]) / gas}
                for j, e in enumerate(pending):
                    yield e, info, j == len(pending) - 1
                pending = []

    def _dp_sum(self, t: torch.Tensor) -> torch.Tensor:
        """Sum a small CPU tensor over the data-parallel group of this worker."""
        s = self.strategy
        if s.world_size == 1 or not dist.is_initialized() or s.mesh.dp == 1:
            return t
        g = s.dp_group()
        work = t.to(self.device) if dist.get_backend(g) == "nccl" else t.clone()
        dist.all_reduce(work, group=g)
        return work.to(t.device)

    def fit(self, kl_ctl: float = 0.0, role: str = "actor") -> dict:
        """PPO epochs over this rank's replay buffer; returns token-/sample-weighted mean metrics."""
        return self._fit_actor(kl_ctl) if role == "actor" else self._fit_critic()

    def _fit_actor(self, kl_ctl: float) -> dict:
        a = self.args
        buf = self.actor_buffer
        eng = self.actor_engine
        sums: dict[str, float] = {}
        wsum_tok = wsum_smp = 0.0
        self.actor.train()
        for _ in range(a.train.max_epochs):
            loader = self._loader(buf)
            for exp, info, last in self._windows(buf, loader):
                exp.to_device(self.device)
                mask = exp.action_mask.float()
                logp, out = self.actor(exp.sequences, exp.action_mask, exp.attention_mask, return_output=True,
                                       return_entropy=a.actor.entropy_coef is not None,
                                       ring_attn_group=self.strategy.ring_attn_group,
                                       **_mm_kwargs(getattr(exp, "mm_train_inputs", None), self.device))
                norm = {k: info[k] for k in ("dp_size", "batch_num_tokens", "global_batch_size")}
                loss, clip_ratio, ppo_kl, vllm_kl = self.policy_loss(logp, exp.action_log_probs, exp.advantages, mask,
                                                                     exp.rollout_log_probs, **norm)
                st = {"policy_loss": loss.detach(), "ppo_clip_ratio": clip_ratio, "ppo_kl": ppo_kl}
                if vllm_kl is not None:
                    st["vllm_kl"] = vllm_kl
                if a.algo.kl.use_loss and exp.base_action_log_probs is not None:
                    kl = K.approx_kl_reference(logp, exp.base_action_log_probs, a.algo.kl.estimator)
                    from ..models.loss import aggregate_loss

                    kl_loss = aggregate_loss(kl, mask, self.policy_loss.token_level_loss, **norm)
                    loss = loss + kl_ctl * kl_loss
                    st["kl"] = masked_mean(kl.detach(), mask)
                if a.actor.aux_loss_coef and out.aux_loss is not None:
                    loss = loss + a.actor.aux_loss_coef * out.aux_loss
                if out.entropy is not None:
                    from ..models.loss import aggregate_loss

                    ent = aggregate_loss(out.entropy, mask, self.policy_loss.token_level_loss, **norm)
                    st["entropy_loss"] = masked_mean(out.entropy.detach(), mask)
                    if a.actor.entropy_coef:
                        loss = loss - a.actor.entropy_coef * ent
                gas = 1 if a.train.dynamic_batch_enable else self.strategy.accumulated_gradient
                eng.backward(loss / gas)
                if last:
                    eng.step()
                    if self.ema_model is not None:
                        with torch.no_grad():     # on the device: no host copy of the parameters per step
                            n = self.ema_flat.numel()
                            self.ema_flat.lerp_(self.actor.model.flat[:n].float(), 1 - a.train.ema_beta)
                ntok, nsmp = float(mask.sum()), float(mask.shape[0])
                for k, v in st.items():
                    sums[k] = sums.get(k, 0.0) + float(v) * ntok
                wsum_tok += ntok
                for k, v in exp.info.items():
                    if isinstance(v, torch.Tensor) and v.numel() == mask.shape[0]:
                        sums["info/" + k] = sums.get("info/" + k, 0.0) + float(v.float().sum())
                for k in ("response_length", "total_length", "truncated"):
                    v = getattr(exp, k)
                    if v is not None:
                        sums["info/" + k] = sums.get("info/" + k, 0.0) + float(v.float().sum())
                wsum_smp += nsmp
        buf.clear()
        packed = torch.tensor([wsum_tok, wsum_smp] + [sums[k] for k in sorted(sums)], dtype=torch.float64)
        if self.strategy.world_size > 1:
            packed = self.strategy.all_reduce(packed, "sum")
        status = {}
        for i, k in enumerate(sorted(sums)):
            if k.startswith("info/"):
                status[k[5:]] = float(packed[2 + i] / max(float(packed[1]), 1.0))
            else:
                status[k] = float(packed[2 + i] / max(float(packed[0]), 1.0))
        status["actor_lr"] = eng.current_lr()
        status["actor_grad_norm"] = eng.grad_norm()
        return status

    def _fit_critic(self) -> dict:
        a = self.args
        buf, eng = self.critic_buffer, self.critic_engine
        tot = vals = ntok_all = 0.0
        self.critic.train()
        for _ in range(a.train.max_epochs):
            loader = self._loader(buf)
            for exp, info, last in self._windows(buf, loader):
                exp.to_device(self.device)
                mask = exp.action_mask.float()
                values = self.critic(exp.sequences, exp.action_mask, exp.attention_mask,
                                     ring_attn_group=self.strategy.ring_attn_group)
                norm = {k: info[k] for k in ("dp_size", "batch_num_tokens", "global_batch_size")}
                loss = self.value_loss(values, exp.values, exp.returns, mask, **norm)
                gas = 1 if a.train.dynamic_batch_enable else self.strategy.accumulated_gradient
                eng.backward(loss / gas)
                if last:
                    eng.step()
                n = float(mask.sum())
                tot += float(loss) * n
                vals += float((values.detach() * mask).sum())
                ntok_all += n
        buf.clear()
        t = torch.tensor([tot, vals, ntok_all], dtype=torch.float64)
        if self.strategy.world_size > 1:
            t = self.strategy.all_reduce(t, "sum")
        d = max(float(t[2]), 1.0)
        return {"critic_loss": float(t[0]) / d, "values": float(t[1]) / d, "critic_lr": eng.current_lr(),
                "critic_grad_norm": eng.grad_norm()}

    # ------------------------------------------------------------------ weight sync / state management
    def setup_sync_group(self, host: str, port: int, rank: int, world: int, backend: str | None = None) -> bool:
        """Join the weight-update group of a placement with separate rollout GPUs: trainer rank 0 plus every rollout
        rank (openrlhf/trainer/ray/ppo_actor.py:163-217 builds the same group next to the training world)."""
        from ..utils.distributed_util import stateless_process_group

        backend = backend or ("nccl" if self.device.type == "cuda" else "gloo")
        self._sync_pg = stateless_process_group(host, port, rank, world, backend, self.device)
        self._sync_rank, self._sync_world = rank, world
        return True

    @torch.no_grad()
    def broadcast_to_vllm(self):
        """Actor -> rollout weights.

        Colocated (hybrid engine): stages 1 / 2 at rollout TP 1 share one buffer, nothing moves; every other case is
        one launch of the copy kernel (ZeRO-3 slices -> full copy, full buffer or ZeRO-3 slices -> tensor-parallel
        shard, tensor-parallel training shards -> full copy). Separate rollout GPUs: trainer rank 0 broadcasts the
        flat bf16 buffer over the weight-update group and every rollout rank cuts its own shard out of it."""
        if self.actor is not None and self.rollout is not None:
            if self._sync_fn is not None:
                self._sync_fn()
            return True
        pg = self._sync_pg
        if pg is None:
            if self.actor is not None and self.rollout is None:
                # separate rollout GPUs, and this is not the broadcasting trainer rank: take part in assembling the
                # full buffer where that is a collective (gloo ranks under ZeRO-3, tensor-parallel training shards)
                kind, obj = self._rollout_source
                if kind == "zero3" and self.device.type != "cuda":
                    obj.gather_full()
                elif kind == "tp_train":
                    obj.tp_train.gather_full(obj)
            return True
        if self.actor is not None:
            if self._sync_rank != 0:
                return True
            # the logical parameter range only: shard padding differs between the trainer's and the engines' buffers
            src = self._full_actor_flat()[: self._logical_numel()]
            pg.broadcast([src], _bcast_opts(0)).wait()
        else:
            buf = getattr(self, "_staging", None)
            dst = (buf.flat if buf is not None else self.rollout_model.flat)[: self._logical_numel()]
            pg.broadcast([dst], _bcast_opts(0)).wait()
            if buf is not None:
                self.rollout.update_weights(buf.flat)
            elif self.rollout.quantization == "fp8":
                self.rollout._refresh_fp8()
        return True

    def _logical_numel(self) -> int:
        """Elements of the full flat parameter layout of the policy (without shard padding)."""
        from ..models.transformer import ALIGN, build_param_specs

        if self.actor is not None:
            kind, obj = self._rollout_source
            cfg = obj.tp_train.full_cfg if kind == "tp_train" else self.actor.cfg
        else:
            cfg = getattr(self, "_staging", self.rollout_model).cfg
        last = build_param_specs(cfg)[-1]
        return last.offset + (last.numel + ALIGN - 1) // ALIGN * ALIGN

    def _full_actor_flat(self) -> torch.Tensor:
        kind, obj = self._rollout_source
        if kind == "zero3":
            return obj.gather_full()
        if kind == "tp_train":
            return obj.tp_train.gather_full(obj)
        return obj.flat

    def offload_states(self, role: str = "actor"):
        (self.actor_engine if role == "actor" else self.critic_engine).offload_states()

    def reload_states(self, role: str = "actor"):
        (self.actor_engine if role == "actor" else self.critic_engine).reload_states()

    def get_checkpoint_states(self):
        return getattr(self, "_resume_states", {})

    def save_model(self, role: str = "actor"):
        a = self.args
        if role == "actor":
            lm = self.actor.model
            if self.ema_model is not None:
                # export the moving average through the actor's own layout, then put the live weights back
                n = self.ema_flat.numel()
                live = lm.flat[:n].clone()
                lm.flat[:n].copy_(self.ema_flat.to(lm.flat.dtype))
                try:
                    self.strategy.save_model(lm, getattr(self, "tokenizer", None), a.ckpt.output_dir)
                finally:
                    lm.flat[:n].copy_(live)
                return
            self.strategy.save_model(lm, getattr(self, "tokenizer", None), a.ckpt.output_dir)
        elif a.critic.save_value_network:
            self.strategy.save_model(self.critic, getattr(self, "tokenizer", None), a.ckpt.output_dir + "_critic")

    def save_checkpoint(self, tag: str, client_states=None, role: str = "actor", metric_value=None, metric_key=None):
        a = self.args
        eng = self.actor_engine if role == "actor" else self.critic_engine
        d = os.path.join(a.ckpt.path, "_actor" if role == "actor" else "_critic")
        if not a.ckpt.disable_ds:
            holder = SimpleNamespace(engine=eng)
            self.strategy.save_ckpt(holder, d, tag, a.ckpt.max_num, a.ckpt.max_mem, client_states or {},
                                    metric_value=metric_value, metric_key=metric_key)
        if a.ckpt.save_hf and role == "actor":
            self.strategy.save_model(self.actor.model, getattr(self, "tokenizer", None),
                                     os.path.join(a.ckpt.path, f"{tag}_hf"))
