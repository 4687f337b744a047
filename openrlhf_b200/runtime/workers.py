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
    def __init__(self, args: SimpleNamespace, roles=ALL_ROLES, max_steps: int = 1000, backend: str | None = None):
        self.args = args
        self.roles = set(roles)
        self.strategy: Strategy = get_strategy(args)
        self.strategy.setup_distributed(backend=backend)
        self.device = self.strategy.device()
        s = self.strategy
        dp = s.mesh.dp
        self.actor = self.actor_engine = self.critic = self.critic_engine = None
        self.ref = self.reward = self.rollout = self.async_engine = self.ema_model = None
        a = args
        temp = a.rollout.temperature
        if "actor" in self.roles:
            lm = load_pretrained(a.actor.model_name_or_path, device=self.device, shard_world=dp, seed=a.train.seed)
            self._rollout_full = None
            if s.ds_tensor_parallel_size > 1 and s.world_size > 1:
                # --ds.tensor_parallel_size: train this rank's shard (parallel/tp_train.py); the rollout engine keeps
                # the full model, refreshed from the gathered shards at every weight sync
                from ..parallel.tp_train import shard_for_training

                if "rollout" in self.roles:
                    self._rollout_full = lm
                    lm.requires_grad_(False)
                lm = shard_for_training(lm, s.mesh.group("tp"), shard_world=dp)
            self.actor = Actor(lm, temperature=temp, packing_samples=a.ds.packing_samples,
                               freeze_visual_encoder=getattr(a.actor, "freeze_visual_encoder", False))
            if a.actor.gradient_checkpointing_enable:
                self.actor.gradient_checkpointing_enable()
            sched = LRScheduler(a.actor.adam.lr, max_steps, a.actor.lr_warmup_ratio, a.actor.min_lr_ratio,
                                a.actor.lr_scheduler)
            self.actor_engine = ZeroEngine(lm, lr=a.actor.adam.lr, betas=tuple(a.actor.adam.betas),
                                           eps=a.actor.adam.eps, weight_decay=a.actor.adam.weight_decay,
                                           max_norm=a.actor.max_norm, zero_stage=a.ds.zero_stage, group=s.dp_group(),
                                           scheduler=sched)
            lo, hi = a.actor.eps_clip_low_high
            self.policy_loss = PolicyLoss(lo, hi, a.actor.dual_clip, policy_loss_type=a.actor.policy_loss_type,
                                          enable_vllm_is_correction=a.algo.advantage.is_correction_enable,
                                          vllm_is_truncated_threshold=a.algo.advantage.is_correction_threshold,
                                          vllm_is_correction_type=a.algo.advantage.is_correction_type)
            self.actor_buffer = NaiveReplayBuffer(a.train.micro_batch_size, 0, True, a.ds.packing_samples,
                                                  a.train.dynamic_batch_enable)
            if a.train.enable_ema:
                from ..models.transformer import TransformerLM

                self.ema_model = TransformerLM(lm.cfg, device="cpu", dtype=torch.float32, seed=None)
                self.ema_model.flat.copy_(lm.flat[: self.ema_model.flat.numel()].float().cpu())
            if a.ckpt.load_enable and os.path.exists(os.path.join(a.ckpt.path, "_actor")):
                _, self._resume_states = s.load_ckpt(SimpleNamespace(engine=self.actor_engine),
                                                     os.path.join(a.ckpt.path, "_actor"))
            else:
                self._resume_states = {}
        if "critic" in self.roles and a.critic.model_name_or_path:
            lm = load_pretrained(a.critic.model_name_or_path, device=self.device, with_lm_head=False,
                                 with_value_head=True, shard_world=dp, seed=a.train.seed + 1,
                                 value_head_prefix=a.ds.value_head_prefix)
            self.critic = CriticModel(lm, normalize_reward=a.reward.normalize_enable,
                                      packing_samples=a.ds.packing_samples)
            if a.actor.gradient_checkpointing_enable:
                self.critic.gradient_checkpointing_enable()
            sched = LRScheduler(a.critic.adam.lr, max_steps, a.critic.lr_warmup_ratio, a.critic.min_lr_ratio,
                                a.critic.lr_scheduler)
            self.critic_engine = ZeroEngine(lm, lr=a.critic.adam.lr, betas=tuple(a.critic.adam.betas),
                                            eps=a.critic.adam.eps, weight_decay=a.critic.adam.weight_decay,
                                            max_norm=a.critic.max_norm, zero_stage=a.ds.zero_stage,
                                            group=s.dp_group(), scheduler=sched)
            self.value_loss = ValueLoss(a.critic.value_clip)
            self.critic_buffer = NaiveReplayBuffer(a.train.micro_batch_size, 0, True, a.ds.packing_samples,
                                                   a.train.dynamic_batch_enable)
            if a.ckpt.load_enable and os.path.exists(os.path.join(a.ckpt.path, "_critic")):
                ckpt.load_sharded(self.critic_engine, os.path.join(a.ckpt.path, "_critic"))
        if "ref" in self.roles and a.algo.kl.init_coef > 0:
            dev = "cpu" if a.ref.offload else self.device
            lm = load_pretrained(a.ref.model_name_or_path or a.actor.model_name_or_path, device=dev, seed=a.train.seed)
            lm.requires_grad_(False)
            if s.ds_tensor_parallel_size > 1 and s.world_size > 1 and dev != "cpu":
                from ..parallel.tp_train import shard_for_training

                lm = shard_for_training(lm, s.mesh.group("tp"))
                lm.requires_grad_(False)
            self.ref = Actor(lm, temperature=temp, packing_samples=a.ds.packing_samples).eval()
        if "reward" in self.roles and a.reward.model_name_or_path:
            dev = "cpu" if a.reward.offload else self.device
            lm = load_pretrained(a.reward.model_name_or_path, device=dev, with_lm_head=False, with_value_head=True,
                                 seed=a.train.seed + 2, value_head_prefix=a.ds.value_head_prefix)
            lm.requires_grad_(False)
            self.reward = RewardModel(lm, normalize_reward=a.reward.normalize_enable,
                                      packing_samples=a.ds.packing_samples).eval()
        if "rollout" in self.roles:
            if self.actor is not None and getattr(self, "_rollout_full", None) is not None:
                rl_model = self._rollout_full        # tensor-parallel training: the engine owns a full copy
            elif self.actor is not None:
                rl_model = self.actor.model          # hybrid engine: one weight buffer for trainer and rollout
            else:
                rl_model = load_pretrained(a.actor.model_name_or_path, device=self.device, seed=a.train.seed)
                rl_model.requires_grad_(False)
            self.tokenizer = get_tokenizer(a.actor.model_name_or_path, None, "left", s,
                                           use_fast=not a.data.disable_fast_tokenizer)
            self.rollout = RolloutEngine(rl_model, max_num_seqs=getattr(a.vllm, "max_num_seqs", 256),
                                         max_model_len=a.data.max_len,
                                         gpu_memory_utilization=a.vllm.gpu_memory_utilization,
                                         seed=a.train.seed + s.rank, eos_token_id=self.tokenizer.eos_token_id,
                                         use_cuda_graph=not a.vllm.enforce_eager,
                                         quantization=getattr(a.vllm, "quantization", None))
            # vision-language models: the processor's image part turns the PIL images an agent passes into patches
            self.rollout.image_processor = getattr(self.tokenizer, "image_processor", None)
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
        if role == "critic":
            self.critic.eval()
            out = self.critic(seq, am, att)
            self.critic.train()
        else:
            model = self.actor if role == "actor" else self.ref
            dev = next(model.parameters()).device
            was = model.training
            model.eval()
            out = model(seq.to(dev), am.to(dev), att.to(dev), **_mm_kwargs(mm_train_inputs, dev))
            model.train(was)
        return _cpu(out)

    @torch.no_grad()
    def forward_reward(self, sequences, attention_mask, pad_sequence=True, **_unused):
        dev = next(self.reward.parameters()).device
        return _cpu(self.reward(sequences.to(dev), attention_mask.to(dev)))

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
                        with torch.no_grad():
                            n = self.ema_model.flat.numel()
                            self.ema_model.flat.mul_(a.train.ema_beta).add_(
                                self.actor.model.flat[:n].float().cpu(), alpha=1 - a.train.ema_beta)
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
                values = self.critic(exp.sequences, exp.action_mask, exp.attention_mask)
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
    def broadcast_to_vllm(self):
        """Actor -> rollout weights. Colocated: the engine already reads the updated buffer. Separate rollout ranks:
        broadcast the flat bf16 buffer from actor rank 0 over the global group (NCCL path, the baseline)."""
        if self.actor is not None and self.rollout is not None:
            tpt = getattr(self.actor.model, "tp_train", None)
            if tpt is not None:
                full = tpt.gather_full(self.actor.model)        # all shards -> full fused layout on every rank
                self.rollout.update_weights(full)
                return True
            self.rollout.update_weights(self.actor.model.flat)
            return True
        if dist.is_initialized() and dist.get_world_size() > 1:
            flat = (self.actor.model.flat if self.actor is not None else self.rollout.model.flat)
            dist.broadcast(flat, src=0)
        return True

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
                lm = self.ema_model
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
