"""Controller-side experience maker: micro-batching of rollout samples, dispatch of the reward / actor / critic /
reference forwards to the worker group, per-token KL, and advantage computation
(openrlhf/trainer/ppo_utils/experience_maker.py:44-411)."""
from __future__ import annotations

import logging
import time

import torch

from ..models.utils import compute_approx_kl, masked_mean
from ..runtime.core import get
from ..utils.seqlen_balancing import get_minimum_num_micro_batch_size, get_seqlen_balanced_partitions
from .advantages import compute_advantages_and_returns
from .experience import Experience

logger = logging.getLogger(__name__)


class RemoteExperienceMaker:
    def __init__(self, group, kl_controller, strategy, tokenizer, has_critic: bool, has_ref: bool, has_reward: bool):
        from ..trainer.ppo_trainer import RoleGroups

        self.groups = group if isinstance(group, RoleGroups) else RoleGroups(group)
        self.group = self.groups.actor
        self.kl_ctl, self.strategy, self.args = kl_controller, strategy, strategy.args
        self.tokenizer = tokenizer
        self.has_critic, self.has_ref, self.has_reward = has_critic, has_ref, has_reward
        self.advantage_estimator = self.args.algo.advantage.estimator

    # ------------------------------------------------------------------ batching
    def split_rollout_samples(self, samples: list[Experience]) -> list[Experience]:
        """Assign prompt-order indices and concatenate into micro-batches: fixed size, or token-balanced partitions
        under --rollout.max_tokens_per_gpu when dynamic batching is on."""
        a = self.args
        for i, s in enumerate(samples):
            s.index = [i]
        pad = self.tokenizer.pad_token_id
        if a.train.dynamic_batch_enable:
            lens = [int(s.total_length.item()) for s in samples]
            dup = a.ds.ring_attn_size * a.ds.tensor_parallel_size
            world = a.actor.num_nodes * a.actor.num_gpus_per_node // dup
            n = get_minimum_num_micro_batch_size(lens, a.rollout.max_tokens_per_gpu, a.ds.ring_attn_size,
                                                 a.ds.tensor_parallel_size)
            n = min(max(-(-n // world) * world, world), len(samples))
            parts = get_seqlen_balanced_partitions(lens, n, equal_size=False)
            return [Experience.concat_experiences([samples[i] for i in p], pad) for p in parts]
        mb = a.rollout.micro_batch_size
        return [Experience.concat_experiences(samples[i:i + mb], pad) for i in range(0, len(samples), mb)]

    @torch.no_grad()
    def make_experience_batch(self, rollout_samples: list[Experience]) -> list[Experience]:
        batches = self.split_rollout_samples(rollout_samples)
        batches = self.make_experience(batches)
        return compute_advantages_and_returns(batches, self.args, self.kl_ctl.value)

    # ------------------------------------------------------------------ forwards
    def _forward(self, role: str, samples: list[Experience], sync: bool):
        kw = dict(sequences=[s.sequences for s in samples], action_mask=[s.action_mask for s in samples],
                  attention_mask=[s.attention_mask for s in samples], role=[role] * len(samples))
        if role != "critic" and any(any(m for m in (s.mm_train_inputs or [])) for s in samples):
            kw["mm_train_inputs"] = [s.mm_train_inputs for s in samples]      # per-sample image inputs of each batch
        g = self.groups.of(role)
        futs = g.async_run_method_batch("forward", **kw)
        if sync:
            get(futs)
            get(g.async_run_method("empty_cache"))
        return futs

    def _flatten(self, futs, role: str = "actor"):
        dup = self.groups.of(role).duplicate_actors
        return [x for chunk in get(futs)[::dup] for x in chunk]

    @torch.no_grad()
    def make_experience(self, samples: list[Experience]) -> list[Experience]:
        t0 = time.time()
        a = self.args
        colocated = a.train.colocate_all
        r_futs = None
        if samples[0].rewards is None:
            if not self.has_reward:
                raise ValueError("samples carry no rewards (reward function failed?) and no reward model is configured")
            r_futs = self.groups.reward.async_run_method_batch(
                "forward_reward", sequences=[s.sequences for s in samples],
                attention_mask=[s.attention_mask for s in samples], pad_sequence=[True] * len(samples))
            if colocated:
                get(r_futs)
        lp_futs = self._forward("actor", samples, colocated or a.train.colocate_actor_ref)
        v_futs = self._forward("critic", samples, colocated or a.train.colocate_critic_reward) if self.has_critic else None
        b_futs = self._forward("ref", samples, colocated or a.train.colocate_actor_ref) if self.has_ref else None
        logps = self._flatten(lp_futs, "actor")
        base = self._flatten(b_futs, "ref") if b_futs is not None else [None] * len(samples)
        vals = self._flatten(v_futs, "critic") if v_futs is not None else [None] * len(samples)
        if r_futs is not None:
            for s, r in zip(samples, self._flatten(r_futs, "reward")):
                s.rewards = r
                s.info["reward"] = r
        if not (len(samples) == len(logps) == len(base) == len(vals)):
            raise AssertionError("a worker returned a different number of micro-batches than it was sent")
        for s, lp, b, v in zip(samples, logps, base, vals):
            if b is not None and not a.algo.kl.use_loss:
                kl = compute_approx_kl(lp, b, kl_estimator=a.algo.kl.estimator)
                diff = lp.float() - b.float()
            else:
                kl = torch.zeros_like(lp)
                diff = torch.zeros_like(lp)
            s.action_log_probs = lp
            s.base_action_log_probs = b if a.algo.kl.use_loss else None
            s.values = v
            s.kl = kl
            s.info["kl"] = masked_mean(kl, s.action_mask, dim=-1)
            s.info["logprobs_diff"] = masked_mean(diff, s.action_mask, dim=-1)
        logger.info("experience making took %.1f s", time.time() - t0)
        return samples
