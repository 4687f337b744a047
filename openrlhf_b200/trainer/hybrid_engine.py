"""Hybrid-engine RL worker driven SPMD: one process per GPU hosts every role that lives on that GPU and runs whole RL
steps on its own share of the prompts.

``HybridRLWorker`` IS the launcher's worker (``runtime.workers.RLWorker``: same constructor path, same engines, same
weight sync) plus ``rl_step``: generate -> rewards -> old / reference log-probs (+ values) -> advantages -> PPO epochs
over micro-batches -> weight sync, the unit the reference times in ``PPOTrainer.train_step``
(openrlhf/trainer/ppo_trainer.py:213-264). Under ``python -m openrlhf.cli.train_ppo_ray`` a controller drives the same
worker through RPCs instead (agents, remote rewards, dynamic filtering); under torchrun (``bench.py``, tests) every
rank calls ``rl_step`` itself and the ranks meet only in the collectives of the engines.

The reference's hybrid engine (``--train.colocate_all``: openrlhf/cli/train_ppo_ray.py:40-50,84-142) packs a vLLM
engine, a DeepSpeed actor, and optionally reference / critic / reward models onto the same GPUs as fractional Ray
actors and moves weights between them with CUDA IPC. Here the roles are plain objects of one process.
"""
from __future__ import annotations

import time
from types import SimpleNamespace
from typing import Callable

import torch
import torch.distributed as dist

from ..models.actor import Actor
from ..models.config import PRESETS, ModelConfig
from ..models.packing import pack_lists
from ..ops import rl as K
from ..rl.advantages import compute_advantages_and_returns
from ..rl.experience import Experience
from ..rl.kl_controller import FixedKLController
from ..rollout.engine import SamplingParams
from ..runtime.workers import RLWorker


def default_rl_args(**over) -> SimpleNamespace:
    """The flag tree of ``train_ppo_ray`` with its defaults (hybrid engine, packed samples, REINFORCE++-baseline
    without a KL term), then the dotted overrides, e.g. ``default_rl_args(**{"ds.zero_stage": 3})``."""
    from ..cli import flags as F
    from ..cli.train_ppo_ray import build_parser

    a = F.finalize(build_parser(), ["--train.colocate_all", "--ds.packing_samples", "--reward.remote_url", "function",
                                    "--algo.advantage.estimator", "reinforce_baseline", "--algo.kl.init_coef", "0",
                                    "--rollout.n_samples_per_prompt", "8", "--rollout.max_new_tokens", "2048",
                                    "--rollout.micro_batch_size", "8", "--train.micro_batch_size", "4",
                                    "--data.max_len", "4096", "--train.seed", "0"])
    a.algo.advantage.lambd = 0.95
    a.rollout.ignore_eos = False
    for k, v in over.items():
        node = a
        parts = k.split(".")
        for p in parts[:-1]:
            if not hasattr(node, p):
                setattr(node, p, SimpleNamespace())
            node = getattr(node, p)
        setattr(node, parts[-1], v)
    return a


class HybridRLWorker(RLWorker):
    def __init__(self, model_cfg: ModelConfig | str, args: SimpleNamespace | None = None, device=None,
                 reward_fn: Callable | None = None, max_steps: int = 1000, seed: int | None = None, group=None,
                 max_num_seqs: int = 256, num_pages: int | None = None, use_cuda_graph: bool = True,
                 with_critic: bool | None = None, use_symm: bool | None = None, reward_model=None,
                 reward_model_path: str | None = None):
        """model_cfg: a preset name / checkpoint directory, or a ModelConfig (random init). The process group, when
        there is more than one rank, is the default one (torchrun environment); `group` is accepted for older callers
        and must be None or the default group."""
        from ..cli.train_ppo_ray import validate

        a = args or default_rl_args()
        if isinstance(model_cfg, ModelConfig):
            name = f"_config_{id(model_cfg)}"
            PRESETS[name] = model_cfg
        else:
            name = model_cfg
        a.actor.model_name_or_path = name
        if seed is not None:
            a.train.seed = seed
        use_critic = with_critic if with_critic is not None else a.algo.advantage.estimator == "gae"
        a.critic.model_name_or_path = name if use_critic else None
        a.reward.model_name_or_path = reward_model_path
        if reward_model_path:
            a.reward.remote_url = None
        if getattr(a.actor, "eps_clip_low_high", None) is None:
            a.actor.eps_clip_low_high = (a.actor.eps_clip, a.actor.eps_clip)
        a.actor.eps_clip_low_high = tuple(a.actor.eps_clip_low_high)
        a.vllm.num_engines = a.vllm.num_engines or 1
        if int(getattr(a.ds, "ring_attn_size", 1) or 1) > 1:
            raise ValueError("context parallelism runs through the launcher's controller (train_ppo_ray), where the "
                             "members of a context-parallel group receive the same samples")
        assert group is None or group is dist.group.WORLD, "the SPMD worker spans the default process group"
        world = int(__import__("os").environ.get("WORLD_SIZE", "1"))
        a.actor.num_nodes, a.actor.num_gpus_per_node = 1, world
        roles = ["actor", "rollout"] + (["critic"] if use_critic else []) + \
                (["ref"] if a.algo.kl.init_coef > 0 else []) + (["reward"] if reward_model_path else [])
        del validate
        super().__init__(a, roles=tuple(roles), max_steps=max_steps, backend=None,
                         engine_opts={"max_num_seqs": max_num_seqs, "num_pages": num_pages,
                                      "use_cuda_graph": use_cuda_graph, "use_symm": use_symm})
        s = self.strategy
        self.world, self.rank = s.mesh.dp, s.mesh.dp_rank
        self.group = s.dp_group()
        self.cfg = self.actor.cfg
        self.model = self.actor.model
        self.engine = self.actor_engine
        self.symm = getattr(self.actor_engine, "symm", None)
        self.zero3 = self._rollout_source[0] == "zero3"
        self.tp_group = self._tp_groups[0]
        if self.tp_group is not None:
            self.rollout.spmd()             # every member issues the same generate() calls: no control channel
        self.reward_model = reward_model if reward_model is not None else self.reward
        self.reward_fn = reward_fn
        self.kl_ctl = FixedKLController(a.algo.kl.init_coef)
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
            cm = self.critic.model
            h, _ = cm(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
            v = cm.values(h)
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
                h, _ = self.critic.model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
                v_t = self.critic.model.values(h)
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
        """Actor -> rollout weight hand-off (``RLWorker.broadcast_to_vllm``): nothing to move when trainer and rollout
        engine read the same buffer, otherwise one launch of the copy kernel (ZeRO-3 slices -> full copy or
        tensor-parallel shard, full buffer -> tensor-parallel shard)."""
        self.broadcast_to_vllm()

    # ------------------------------------------------------------------ the RL step
    def rl_step(self, prompts: list[list[int]] | torch.Tensor) -> dict:
        """One synchronous RL step on this rank's prompts. `prompts` may be a pinned (P, L) CPU tensor."""
        on_gpu = self.device.type == "cuda"
        marks: dict = {}

        def mark(k):
            if on_gpu:
                marks[k] = torch.cuda.Event(enable_timing=True)
                marks[k].record()
            else:
                marks[k] = time.perf_counter()

        def between(a, b):
            return marks[a].elapsed_time(marks[b]) / 1e3 if on_gpu else marks[b] - marks[a]

        mark("t0")
        if isinstance(prompts, torch.Tensor):
            prompts = prompts.to(self.device, non_blocking=True).tolist()
        from ..utils.tracing import tracer

        with tracer.span("generation", cat="rl_step", step=self.global_step):
            exps = self.generate(prompts)
        mark("gen")
        with tracer.span("make_experience", cat="rl_step", step=self.global_step):
            exps = self.make_experience(exps)
            exps = self.compute_advantages(exps)
        mark("exp")
        status = {}
        with tracer.span("ppo_train", cat="rl_step", step=self.global_step):
            if self.critic is not None:
                status.update(self.train_critic(exps))
            status.update(self.train(exps))
        mark("train")
        with tracer.span("broadcast", cat="rl_step", step=self.global_step):
            self.sync_weights()
        mark("sync")
        if on_gpu:
            torch.cuda.synchronize(self.device)
        self.timing = {"timing/generation": between("t0", "gen"), "timing/make_experience": between("gen", "exp"),
                       "timing/ppo_train": between("exp", "train"), "timing/broadcast": between("train", "sync")}
        self.timing["timing/step_total"] = sum(self.timing.values())
        status.update(self.timing)
        rw = torch.stack([e.rewards.to(self.device) for e in exps])
        status["reward"] = float(rw.mean())
        status["response_length"] = float(torch.stack([e.response_length for e in exps]).float().mean())
        status["num_samples"] = len(exps)
        status["gen_tokens"] = float(sum(float(e.response_length) for e in exps))
        self.global_step += 1
        return status
