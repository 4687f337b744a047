"""Hybrid-engine RL worker: one process per GPU hosts every role that lives on that GPU.

The reference's hybrid engine (``--train.colocate_all``: openrlhf/cli/train_ppo_ray.py:40-50,84-142) packs a vLLM
engine, a DeepSpeed actor, and optionally reference / critic / reward models onto the same GPUs as fractional Ray
actors and moves weights between them with CUDA IPC. Here the roles are plain objects of one process: the rollout
engine reads the very buffer the ZeRO engine updates (weight sync at TP=1 is a no-op), and phase changes are method
calls. ``rl_step`` is one synchronous RL step: generate -> rewards -> old/ref log-probs (+values) -> advantages ->
PPO epochs over micro-batches -> weight sync, the unit the reference times in ``PPOTrainer.train_step``
(openrlhf/trainer/ppo_trainer.py:213-264).
"""
from __future__ import annotations

import time
from types import SimpleNamespace
from typing import Callable

import torch
import torch.distributed as dist

from ..models.actor import Actor
from ..models.config import ModelConfig
from ..models.packing import pack_lists
from ..models.transformer import TransformerLM
from ..ops import rl as K
from ..parallel.zero import LRScheduler, ZeroEngine
from ..rl.advantages import compute_advantages_and_returns
from ..rl.experience import Experience
from ..rl.kl_controller import FixedKLController
from ..rollout.engine import RolloutEngine, SamplingParams


def default_rl_args(**over) -> SimpleNamespace:
    """The subset of the train_ppo_ray flag tree this worker reads, with the reference's defaults."""
    a = SimpleNamespace(
        algo=SimpleNamespace(
            advantage=SimpleNamespace(estimator="reinforce_baseline", gamma=1.0, lambd=0.95, no_std_norm=False,
                                      is_correction_enable=False, is_correction_type="tis",
                                      is_correction_threshold=(0.5, 5.0)),
            kl=SimpleNamespace(init_coef=0.0, estimator="k1", use_loss=False, target=None, horizon=10000)),
        rollout=SimpleNamespace(n_samples_per_prompt=8, max_new_tokens=2048, temperature=1.0, top_p=1.0,
                                micro_batch_size=8),
        train=SimpleNamespace(micro_batch_size=4, batch_size=128, max_epochs=1),
        actor=SimpleNamespace(eps_clip_low_high=(0.2, 0.2), dual_clip=None, entropy_coef=None, policy_loss_type="ppo",
                              adam=SimpleNamespace(lr=1e-6, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0),
                              max_norm=1.0, lr_scheduler="cosine_with_min_lr", lr_warmup_ratio=0.03, min_lr_ratio=0.1,
                              gradient_checkpointing_enable=False, aux_loss_coef=0.0),
        critic=SimpleNamespace(value_clip=0.5, adam=SimpleNamespace(lr=9e-6, betas=(0.9, 0.95), eps=1e-8,
                                                                     weight_decay=0.0), max_norm=1.0),
        reward=SimpleNamespace(clip_range=(-10.0, 10.0), overlong_buffer_len=None, stop_properly_penalty_coef=None),
        data=SimpleNamespace(max_len=4096),
        ds=SimpleNamespace(zero_stage=2),
    )
    for k, v in over.items():
        node = a
        parts = k.split(".")
        for p in parts[:-1]:
            node = getattr(node, p)
        setattr(node, parts[-1], v)
    return a


class HybridRLWorker:
    def __init__(self, model_cfg: ModelConfig | str, args: SimpleNamespace | None = None, device=None,
                 reward_fn: Callable | None = None, max_steps: int = 1000, seed: int = 0, group=None,
                 max_num_seqs: int = 256, num_pages: int | None = None, use_cuda_graph: bool = True,
                 with_critic: bool | None = None, use_symm: bool = False, reward_model=None):
        self.args = args or default_rl_args()
        a = self.args
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        cfg = ModelConfig.from_pretrained(model_cfg) if isinstance(model_cfg, str) else model_cfg
        self.cfg = cfg
        self.symm = None
        flat = None
        if use_symm and self.world > 1:
            from ..parallel.symm import SymmBuffers
            from ..models.transformer import build_param_specs, ALIGN

            specs = build_param_specs(cfg)
            total = specs[-1].offset + (specs[-1].numel + ALIGN - 1) // ALIGN * ALIGN
            self.symm = SymmBuffers(group, ZeroEngine.padded_numel(total, self.world), self.device)
            flat = self.symm.param
        self.model = TransformerLM(cfg, device=self.device, seed=seed, shard_world=self.world, flat=flat)
        self.actor = Actor(self.model, temperature=a.rollout.temperature)
        if a.actor.gradient_checkpointing_enable:
            self.actor.gradient_checkpointing_enable()
        sched = LRScheduler(a.actor.adam.lr, max_steps, a.actor.lr_warmup_ratio, a.actor.min_lr_ratio,
                            a.actor.lr_scheduler)
        self.zero3 = a.ds.zero_stage == 3 and self.world > 1 and not use_symm
        self.rollout_model = self.model
        ref_init = None
        if self.zero3:
            # stage 3: the trainer keeps only its slice of the parameters (plus two layer slots); the rollout engine
            # gets a full copy of its own that the weight sync refreshes from the owners' slices (one copy kernel)
            from ..parallel.zero3 import Zero3Engine

            self.rollout_model = TransformerLM(cfg, device=self.device, seed=None, shard_world=self.world)
            self.rollout_model.requires_grad_(False)
            self.rollout_model.flat.copy_(self.model.flat[: self.rollout_model.flat.numel()])
            ref_init = self.rollout_model.flat
            self.engine = Zero3Engine(self.model, lr=a.actor.adam.lr, betas=tuple(a.actor.adam.betas),
                                      eps=a.actor.adam.eps, weight_decay=a.actor.adam.weight_decay,
                                      max_norm=a.actor.max_norm, group=group, scheduler=sched)
        else:
            self.engine = ZeroEngine(self.model, lr=a.actor.adam.lr, betas=tuple(a.actor.adam.betas),
                                     eps=a.actor.adam.eps, weight_decay=a.actor.adam.weight_decay,
                                     max_norm=a.actor.max_norm, zero_stage=a.ds.zero_stage, group=group,
                                     scheduler=sched, symm=self.symm)
        self.ref = None
        if a.algo.kl.init_coef > 0:
            ref_model = TransformerLM(cfg, device=self.device, seed=None)
            ref_model.flat.copy_((ref_init if ref_init is not None else self.model.flat)[: ref_model.flat.numel()])
            ref_model.requires_grad_(False)
            self.ref = Actor(ref_model, temperature=a.rollout.temperature)
        self.critic = self.critic_engine = None
        use_critic = with_critic if with_critic is not None else a.algo.advantage.estimator == "gae"
        if use_critic:
            cm = TransformerLM(cfg, device=self.device, seed=seed + 1, with_lm_head=False, with_value_head=True,
                               shard_world=self.world)
            self.critic = cm
            self.critic_engine = ZeroEngine(cm, lr=a.critic.adam.lr, betas=tuple(a.critic.adam.betas),
                                            eps=a.critic.adam.eps, weight_decay=a.critic.adam.weight_decay,
                                            max_norm=a.critic.max_norm, zero_stage=a.ds.zero_stage, group=group,
                                            scheduler=LRScheduler(a.critic.adam.lr, max_steps, 0.03, 0.1))
        self.reward_model = reward_model      # models.model.RewardModel: scores full sequences when no reward_fn is set
        self.reward_fn = reward_fn
        self.kl_ctl = FixedKLController(a.algo.kl.init_coef)
        self.rollout_tp = int(getattr(getattr(a, "vllm", None), "tensor_parallel_size", 1) or 1)
        self.tp_group = None
        if self.rollout_tp > 1 and self.world > 1:
            # consecutive ranks form one tensor-parallel rollout engine: same requests on every member, weights sliced
            # from this rank's full trainer buffer by the weight-sync copy plan at every sync
            from ..rollout.tp_engine import make_tp_engine

            assert self.world % self.rollout_tp == 0
            for k in range(self.world // self.rollout_tp):
                ranks = list(range(k * self.rollout_tp, (k + 1) * self.rollout_tp))
                g_ = dist.new_group(ranks)
                if self.rank in ranks:
                    self.tp_group = g_
            self.rollout = make_tp_engine(self.cfg, self.rollout_model.flat, self.tp_group,
                                          max_num_seqs=max_num_seqs * self.rollout_tp, max_model_len=a.data.max_len,
                                          num_pages=(num_pages * self.rollout_tp) if num_pages else None,
                                          seed=seed + 1000 * (self.rank // self.rollout_tp),
                                          use_cuda_graph=use_cuda_graph)
        else:
            self.rollout = RolloutEngine(self.rollout_model, max_num_seqs=max_num_seqs, max_model_len=a.data.max_len,
                                         num_pages=num_pages, seed=seed + 1000 * self.rank,
                                         use_cuda_graph=use_cuda_graph)
        self.timing: dict[str, float] = {}
        self.global_step = 0

    # ------------------------------------------------------------------ phases
    @torch.no_grad()
    def generate(self, prompts: list[list[int]]) -> list[Experience]:
        """Sample n responses per prompt; returns one single-sample Experience per response (device tensors)."""
        a = self.args
        n = a.rollout.n_samples_per_prompt
        sp = SamplingParams(temperature=a.rollout.temperature, top_p=a.rollout.top_p, top_k=-1,
                            max_tokens=a.rollout.max_new_tokens, min_tokens=1, n=n, logprobs=1,
                            ignore_eos=getattr(a.rollout, "ignore_eos", False))
        if self.tp_group is not None:
            # every member of the TP engine generates for the union of the members' prompts and keeps its own share
            gathered = [None] * self.rollout_tp
            dist.all_gather_object(gathered, [list(map(int, p)) for p in prompts], group=self.tp_group)
            me = dist.get_rank(self.tp_group)
            start = sum(len(g_) for g_ in gathered[:me])
            outs = self.rollout.generate([p for g_ in gathered for p in g_], sp)[start:start + len(prompts)]
        else:
            outs = self.rollout.generate(prompts, sp)
        exps = []
        dev = self.device
        for pi, ro in enumerate(outs):
            p = torch.tensor(ro.prompt_token_ids, dtype=torch.long)
            for c in ro.outputs:
                r = torch.tensor(c.token_ids, dtype=torch.long)
                seq = torch.cat([p, r])
                T = seq.numel()
                am = torch.zeros(T - 1, dtype=torch.bool)
                am[len(p) - 1:] = True
                rl = torch.zeros(T - 1, dtype=torch.float32)
                rl[len(p) - 1:] = torch.tensor(c.logprob_values, dtype=torch.float32)
                exps.append(Experience(
                    sequences=seq, attention_mask=torch.ones(T, dtype=torch.long), action_mask=am,
                    rollout_log_probs=rl, response_length=torch.tensor(float(len(r))),
                    total_length=torch.tensor(float(T)), truncated=torch.tensor(c.finish_reason == "length"),
                    index=[pi * n + c.index], info={}))
        return exps

    @torch.no_grad()
    def _forward_logprobs(self, actor: Actor, seqs: list[torch.Tensor], micro: int) -> list[torch.Tensor]:
        """Per-sample next-token log-probs (length T-1 each) for a list of 1-D token tensors, packed `micro` at a time."""
        out = []
        was = actor.training
        actor.eval()
        for s in range(0, len(seqs), micro):
            chunk = seqs[s:s + micro]
            pb = pack_lists(chunk, self.device)
            logp, _, _ = actor.forward_packed(pb)
            cu = pb.cu_list if pb.cu_list is not None else pb.cu_seqlens.tolist()   # host copy: no device sync
            for i in range(len(chunk)):
                out.append(logp[cu[i]:cu[i + 1] - 1])
        actor.train(was)
        return out

    @torch.no_grad()
    def _forward_values(self, seqs: list[torch.Tensor], micro: int) -> list[torch.Tensor]:
        out = []
        for s in range(0, len(seqs), micro):
            chunk = seqs[s:s + micro]
            pb = pack_lists(chunk, self.device)
            h, _ = self.critic(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
            v = self.critic.values(h)
            cu = pb.cu_list if pb.cu_list is not None else pb.cu_seqlens.tolist()   # host copy: no device sync
            for i in range(len(chunk)):
                out.append(v[cu[i]:cu[i + 1] - 1])
        return out

    @torch.no_grad()
    def make_experience(self, exps: list[Experience]) -> list[Experience]:
        a = self.args
        seqs = [e.sequences for e in exps]
        micro = a.rollout.micro_batch_size
        if exps[0].rewards is None:
            if self.reward_fn is None and self.reward_model is None:
                raise ValueError("no rewards on the samples and no reward function / model configured")
            if self.reward_fn is not None:
                r = self.reward_fn(exps)
            else:
                from ..utils.utils import zero_pad_sequences

                r = []
                self.reward_model.eval()
                for s0 in range(0, len(seqs), micro):
                    chunk = [t.to(self.device) for t in seqs[s0:s0 + micro]]
                    ids = zero_pad_sequences(chunk, side="right", value=0, stack=True)
                    att = zero_pad_sequences([torch.ones_like(t) for t in chunk], side="right", value=0, stack=True)
                    r += list(self.reward_model(ids, attention_mask=att).float().unbind(0))
            for e, ri in zip(exps, r):
                e.rewards = torch.as_tensor(ri, dtype=torch.float32).reshape(())
                e.scores = e.rewards.clone()
        old = self._forward_logprobs(self.actor, seqs, micro)
        ref = self._forward_logprobs(self.ref, seqs, micro) if self.ref is not None else None
        vals = self._forward_values(seqs, micro) if self.critic is not None else None
        for i, e in enumerate(exps):
            m = e.action_mask.to(self.device)
            e.action_mask = m
            e.sequences = e.sequences.to(self.device)
            e.rollout_log_probs = e.rollout_log_probs.to(self.device)
            e.action_log_probs = old[i] * m
            if ref is not None:
                base = ref[i] * m
                if not a.algo.kl.use_loss:
                    e.kl = K.approx_kl_reference(e.action_log_probs, base, a.algo.kl.estimator) * m
                    e.info["kl"] = (e.kl.sum() / m.sum().clamp_min(1)).reshape(())
                else:
                    e.base_action_log_probs = base
            if e.kl is None:
                e.kl = torch.zeros_like(e.action_log_probs)
            if vals is not None:
                e.values = vals[i] * m
        return exps

    def _batch(self, items: list[Experience]) -> Experience:
        from ..rl.experience import make_experience_batch

        for it in items:
            it.info = {k: v for k, v in it.info.items() if isinstance(v, torch.Tensor) and v.dim() == 0}
        return make_experience_batch(items)

    @torch.no_grad()
    def compute_advantages(self, exps: list[Experience]) -> list[Experience]:
        """Group baselines / GAE / whitening over the whole rollout batch of this rank (batched per micro chunk)."""
        batches = []
        step = 64
        for s in range(0, len(exps), step):
            chunk = exps[s:s + step]
            b = self._batch(chunk)
            b.index = [i for e in chunk for i in e.index]
            batches.append(b)
        compute_advantages_and_returns(batches, self.args, self.kl_ctl.value, dist_group=self.group,
                                       distributed=self.world > 1)
        out = []
        from ..rl.experience import remove_padding_in_sequences, split_experience_batch

        for b in batches:
            idx = b.index
            singles = split_experience_batch(b)
            for s_, i in zip(singles, idx):
                s_.index = [i]
            out += remove_padding_in_sequences(singles)
        return out

    def train(self, exps: list[Experience]) -> dict:
        """PPO epochs over micro-batches of packed samples with gradient accumulation per optimizer step."""
        a = self.args
        micro = a.train.micro_batch_size
        per_step = max(micro, a.train.batch_size // self.world)
        status_acc: dict[str, float] = {}
        n_tok_total = 0.0
        eps_lo, eps_hi = a.actor.eps_clip_low_high
        self.actor.train()
        for _epoch in range(a.train.max_epochs):
            for s0 in range(0, len(exps), per_step):
                window = exps[s0:s0 + per_step]
                # global token-mean: normaliser = action tokens of the whole optimizer-step window over all ranks
                ntok = torch.stack([e.action_mask.sum() for e in window]).sum().float()
                if self.world > 1:
                    dist.all_reduce(ntok, group=self.group)
                for m0 in range(0, len(window), micro):
                    mb = window[m0:m0 + micro]
                    pb = pack_lists([e.sequences for e in mb], self.device)
                    logp_t, ent_t, aux = self.actor.forward_packed(pb, return_entropy=a.actor.entropy_coef is not None)
                    cu = pb.cu_list if pb.cu_list is not None else pb.cu_seqlens.tolist()   # host copy: no device sync
                    sel = torch.cat([torch.arange(cu[i], cu[i + 1] - 1, device=self.device) for i in range(len(mb))])
                    logp = logp_t[sel]
                    cat = lambda f: torch.cat([getattr(e, f) for e in mb])
                    mask = cat("action_mask").float()
                    w = mask * (self.world / ntok)
                    ref_lp = cat("base_action_log_probs") if mb[0].base_action_log_probs is not None else None
                    is_on = a.algo.advantage.is_correction_enable
                    out = K.ppo_loss(logp, cat("action_log_probs"), cat("advantages"), mask, ref_logp=ref_lp,
                                     rollout_logp=cat("rollout_log_probs"), weight=w, eps_low=eps_lo, eps_high=eps_hi,
                                     dual_clip=a.actor.dual_clip, kl_coef=self.kl_ctl.value if ref_lp is not None else 0.0,
                                     kl_estimator=a.algo.kl.estimator,
                                     is_mode=a.algo.advantage.is_correction_type if is_on else None,
                                     is_lo=a.algo.advantage.is_correction_threshold[0],
                                     is_hi=a.algo.advantage.is_correction_threshold[1])
                    loss = out["loss"]
                    if a.actor.entropy_coef:
                        loss = loss - a.actor.entropy_coef * (ent_t[sel] * w).sum()
                    if a.actor.aux_loss_coef:
                        loss = loss + a.actor.aux_loss_coef * aux
                    self.engine.backward(loss)
                    nt = mask.sum()
                    n_tok_total = n_tok_total + nt
                    for k in ("policy_loss", "clip_ratio", "ppo_kl", "vllm_kl"):
                        v = out[k].detach()
                        status_acc[k] = status_acc.get(k, 0.0) + (v * nt if k != "policy_loss" else v)
                self.engine.step()
        denom = max(float(n_tok_total), 1.0)
        st = {k: (float(v) / denom if k != "policy_loss" else float(v)) for k, v in status_acc.items()}
        st["actor_lr"] = self.engine.current_lr()
        st["actor_grad_norm"] = self.engine.grad_norm()
        return st

    def train_critic(self, exps: list[Experience]) -> dict:
        a = self.args
        micro = a.train.micro_batch_size
        per_step = max(micro, a.train.batch_size // self.world)
        tot = 0.0
        self.critic.train()
        for s0 in range(0, len(exps), per_step):
            window = exps[s0:s0 + per_step]
            ntok = torch.stack([e.action_mask.sum() for e in window]).sum().float()
            if self.world > 1:
                dist.all_reduce(ntok, group=self.group)
            for m0 in range(0, len(window), micro):
                mb = window[m0:m0 + micro]
                pb = pack_lists([e.sequences for e in mb], self.device)
                h, _ = self.critic(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
                v_t = self.critic.values(h)
                cu = pb.cu_list if pb.cu_list is not None else pb.cu_seqlens.tolist()   # host copy: no device sync
                sel = torch.cat([torch.arange(cu[i], cu[i + 1] - 1, device=self.device) for i in range(len(mb))])
                cat = lambda f: torch.cat([getattr(e, f) for e in mb])
                mask = cat("action_mask").float()
                loss = K.value_loss(v_t[sel], cat("values"), cat("returns"), mask, clip_eps=a.critic.value_clip,
                                    weight=mask * (self.world / ntok))
                self.critic_engine.backward(loss)
                tot += float(loss)
            self.critic_engine.step()
        return {"critic_loss": tot, "critic_lr": self.critic_engine.current_lr(),
                "critic_grad_norm": self.critic_engine.grad_norm()}

    def sync_weights(self):
        """Actor -> rollout weight hand-off. Trainer and rollout engine read the same buffer on this GPU, so after the
        optimizer step (which all-gathers updated shards into every rank's buffer) there is nothing left to move."""
        if self.zero3:
            self.engine.gather_full(self.rollout_model.flat)     # K-SYNC from the owners' parameter slices
            if self.tp_group is not None:
                self.rollout.update_weights(self.rollout_model.flat)
            return
        self.rollout.update_weights(self.model.flat)

    # ------------------------------------------------------------------ the RL step
    def rl_step(self, prompts: list[list[int]] | torch.Tensor) -> dict:
        """One synchronous RL step on this rank's prompts. `prompts` may be a pinned (P, L) CPU tensor."""
        ev = {k: torch.cuda.Event(enable_timing=True) for k in ("t0", "gen", "exp", "train", "sync")}
        ev["t0"].record()
        if isinstance(prompts, torch.Tensor):
            prompts = prompts.to(self.device, non_blocking=True).tolist()
        from ..utils.tracing import tracer

        with tracer.span("generation", cat="rl_step", step=self.global_step):
            exps = self.generate(prompts)
        ev["gen"].record()
        with tracer.span("make_experience", cat="rl_step", step=self.global_step):
            exps = self.make_experience(exps)
            exps = self.compute_advantages(exps)
        ev["exp"].record()
        status = {}
        with tracer.span("ppo_train", cat="rl_step", step=self.global_step):
            if self.critic is not None:
                status.update(self.train_critic(exps))
            status.update(self.train(exps))
        ev["train"].record()
        with tracer.span("broadcast", cat="rl_step", step=self.global_step):
            self.sync_weights()
        ev["sync"].record()
        torch.cuda.synchronize(self.device)
        self.timing = {"timing/generation": ev["t0"].elapsed_time(ev["gen"]) / 1e3,
                       "timing/make_experience": ev["gen"].elapsed_time(ev["exp"]) / 1e3,
                       "timing/ppo_train": ev["exp"].elapsed_time(ev["train"]) / 1e3,
                       "timing/broadcast": ev["train"].elapsed_time(ev["sync"]) / 1e3}
        self.timing["timing/step_total"] = sum(self.timing.values())
        status.update(self.timing)
        rw = torch.stack([e.rewards.to(self.device) for e in exps])
        status["reward"] = float(rw.mean())
        status["response_length"] = float(torch.stack([e.response_length for e in exps]).float().mean())
        status["num_samples"] = len(exps)
        status["gen_tokens"] = float(sum(float(e.response_length) for e in exps))
        self.global_step += 1
        return status
