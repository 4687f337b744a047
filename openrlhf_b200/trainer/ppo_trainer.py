"""Single-controller RL trainers (sync): dataset preparation, the ``fit`` loop, one ``train_step`` (experience ->
balance -> append -> PPO epochs -> weight sync), evaluation with pass@k, periodic and best checkpoints, resume.

Behavioural counterpart of openrlhf/trainer/ppo_trainer.py:26-595, driving this framework's runtime
(``runtime.core.ActorGroup`` of ``RLWorker`` processes) instead of Ray actor groups.
"""
from __future__ import annotations

import logging
import os
import time

import torch

from ..datasets import PromptDataset
from ..datasets.utils import blending_datasets
from ..rl.experience import balance_experiences
from ..rl.experience_maker import RemoteExperienceMaker
from ..rl.kl_controller import AdaptiveKLController, FixedKLController
from ..rl.samples_generator import SamplesGenerator
from ..runtime.core import get
from ..utils.logging_utils import build_loggers
from ..utils.utils import get_tokenizer

logger = logging.getLogger(__name__)


def prepare_datasets(strategy, tokenizer):
    a = strategy.args

    def loader(spec, probs, split, shuffle):
        data = blending_datasets(spec, probs, strategy, a.train.seed, max_count=a.data.max_samples, dataset_split=split)
        data = data.select(range(min(a.data.max_samples, len(data))))
        ds = PromptDataset(data, tokenizer, strategy, input_template=a.data.input_template)
        return ds, strategy.setup_dataloader(ds, 1, True, shuffle, ds.collate_fn, drop_last=True,
                                             num_workers=a.data.dataloader_num_workers)

    prompts_ds, prompts_dl = loader(a.data.prompt_dataset, a.data.prompt_probs, a.data.prompt_split, True)
    eval_dl = None
    if getattr(a.eval, "dataset", None):
        _, eval_dl = loader(a.eval.dataset, None, a.eval.split, False)
    max_steps = (len(prompts_ds) * a.rollout.n_samples_per_prompt // a.train.batch_size * a.train.num_episodes
                 * a.train.max_epochs)
    return prompts_dl, eval_dl, max_steps


def compute_eval_metrics(eval_dataloader, samples_list, n_samples_per_prompt: int) -> dict:
    """pass@1 / pass@n per datasource plus response-length and truncation statistics."""
    if not samples_list:
        return {}
    source_of = {}
    for sources, prompts, _labels, _images in eval_dataloader:
        source_of.update(zip(prompts, sources))
    n = n_samples_per_prompt
    rewards = torch.tensor([float(s.rewards) for s in samples_list]).reshape(-1, n)
    per: dict[str, dict] = {}
    for g in range(rewards.shape[0]):
        ds = source_of.get(samples_list[g * n].prompts[0], "unknown")
        m = per.setdefault(ds, {"passn": 0.0, "pass1": 0.0, "count": 0, "len": [], "trunc": []})
        m["passn"] += float(rewards[g].max()) if n > 1 else 0.0
        m["pass1"] += float(rewards[g].mean())
        m["count"] += 1
        for s in samples_list[g * n:(g + 1) * n]:
            if s.response_length is not None:
                m["len"].append(float(s.response_length))
            if s.truncated is not None:
                m["trunc"].append(float(s.truncated))
    logs, all_len, all_tr = {}, [], []
    for ds, m in per.items():
        logs[f"eval_{ds}_pass{n}"] = m["passn"] / m["count"]
        logs[f"eval_{ds}_pass1"] = m["pass1"] / m["count"]
        if m["len"]:
            logs[f"eval_{ds}_response_length_mean"] = sum(m["len"]) / len(m["len"])
            all_len += m["len"]
        if m["trunc"]:
            logs[f"eval_{ds}_truncated_rate"] = sum(m["trunc"]) / len(m["trunc"])
            all_tr += m["trunc"]
    if all_len:
        logs["eval_response_length_mean"] = sum(all_len) / len(all_len)
    if all_tr:
        logs["eval_truncated_rate"] = sum(all_tr) / len(all_tr)
    logs["eval_num_samples"] = float(len(samples_list))
    return logs


class RoleGroups:
    """Which worker group serves which role. Under ``--train.colocate_all`` one group hosts everything; otherwise the
    launcher builds one group per placement (openrlhf/cli/train_ppo_ray.py:40-142) and the trainer addresses each
    role through its own group."""

    def __init__(self, actor, critic=None, ref=None, reward=None, rollout=None):
        self.actor = actor
        self.critic = critic if critic is not None else actor
        self.ref = ref if ref is not None else actor
        self.reward = reward if reward is not None else actor
        self.rollout = rollout               # None: the rollout engines live on the actor group's workers

    def of(self, role: str):
        return getattr(self, role)

    def distinct(self) -> list:
        seen, out = set(), []
        for g in (self.actor, self.critic, self.ref, self.reward, self.rollout):
            if g is not None and id(g) not in seen:
                seen.add(id(g))
                out.append(g)
        return out

    def shutdown(self):
        for g in self.distinct():
            g.shutdown()


class BasePPOTrainer:
    def __init__(self, strategy, group, has_critic: bool, has_ref: bool, has_reward: bool, tokenizer):
        self.groups = group if isinstance(group, RoleGroups) else RoleGroups(group)
        group = self.groups.actor
        self.strategy, self.args, self.group, self.tokenizer = strategy, strategy.args, group, tokenizer
        self.has_critic = has_critic
        a = self.args
        if a.algo.kl.target:
            self.kl_ctl = AdaptiveKLController(a.algo.kl.init_coef, a.algo.kl.target, a.algo.kl.horizon)
        else:
            self.kl_ctl = FixedKLController(a.algo.kl.init_coef)
        self.experience_maker = RemoteExperienceMaker(self.groups, self.kl_ctl, strategy, tokenizer, has_critic,
                                                      has_ref, has_reward)
        self.loggers = build_loggers(a, True)
        self.best_eval_metric_key = getattr(a.ckpt, "best_metric_key", "") or ""
        self.best_eval_metric_value = float("-inf")
        self._latest_eval_metric_value = None
        self.generate_kwargs = {"do_sample": True, "max_new_tokens": a.rollout.max_new_tokens, "max_len": a.data.max_len,
                                "temperature": a.rollout.temperature, "top_p": a.rollout.top_p,
                                "ignore_eos": getattr(a.rollout, "ignore_eos", False)}

    # ------------------------------------------------------------------ one RL step
    def train_step(self, rollout_samples, global_step: int):
        a = self.args
        t0 = time.time()
        experiences = self.experience_maker.make_experience_batch(rollout_samples)
        t_exp = time.time() - t0
        sample0 = None
        if rollout_samples:
            s = rollout_samples[0]
            sample0 = [self.tokenizer.decode(s.sequences[0].tolist(), skip_special_tokens=True),
                       float(s.rewards[0]) if s.rewards is not None else 0.0]
        stats = self._compute_rollout_stats(experiences)
        if a.train.dynamic_batch_enable:
            experiences = balance_experiences(experiences, a)
        get(self.group.async_run_method_batch("append", experience=experiences, role=["actor"] * len(experiences)))
        if self.has_critic:
            get(self.groups.critic.async_run_method_batch("append", experience=experiences,
                                                          role=["critic"] * len(experiences)))
        t1 = time.time()
        status = self.ppo_train(global_step)
        t_train = time.time() - t1
        t2 = time.time()
        self.broadcast_to_vllm()
        t_sync = time.time() - t2
        if "kl" in status:
            self.kl_ctl.update(status["kl"], a.rollout.batch_size * a.rollout.n_samples_per_prompt)
        status.update(stats)
        status["generated_samples"] = sample0
        status.update({"timing/make_experience": t_exp, "timing/ppo_train": t_train, "timing/broadcast": t_sync})
        return status, global_step + 1

    def ppo_train(self, global_step: int) -> dict:
        a = self.args
        status = {}
        sleep = getattr(a.ds, "enable_sleep", False)
        cg = self.groups.critic
        critic_futs = None
        if self.has_critic:
            if sleep:
                get(cg.async_run_method("reload_states", role="critic"))
            critic_futs = cg.async_run_method("fit", role="critic")
            if cg is self.group:              # same workers: the critic trains first, then the actor
                status.update(get(critic_futs)[0])
                critic_futs = None
                if sleep:
                    get(cg.async_run_method("offload_states", role="critic"))
        if global_step >= getattr(a.critic, "freezing_steps", 0) or not self.has_critic:
            if sleep:
                get(self.group.async_run_method("reload_states", role="actor"))
            status.update(get(self.group.async_run_method("fit", kl_ctl=self.kl_ctl.value, role="actor"))[0])
            if sleep:
                get(self.group.async_run_method("offload_states", role="actor"))
        if critic_futs is not None:           # critic on its own GPUs: it trained concurrently with the actor
            status.update(get(critic_futs)[0])
            if sleep:
                get(cg.async_run_method("offload_states", role="critic"))
        return status

    def broadcast_to_vllm(self):
        rg = self.groups.rollout
        if self.args.vllm.enable_sleep:
            get((rg or self.group).async_run_method("wake_up", tags=["weights"]))
        futs = self.group.async_run_method("broadcast_to_vllm")
        if rg is not None:                    # rollout engines on their own GPUs receive over the weight-update group
            futs = futs + rg.async_run_method("broadcast_to_vllm")
        get(futs)

    @staticmethod
    def _compute_rollout_stats(experiences) -> dict:
        rw = [e.info["reward"].float().reshape(-1) for e in experiences if "reward" in e.info]
        out = {}
        if rw:
            r = torch.cat(rw)
            out.update({"rollout/reward_mean": r.mean().item(), "rollout/reward_std": r.std().item() if len(r) > 1 else 0.0,
                        "rollout/num_samples": float(len(r))})
        ln = [e.response_length.float().reshape(-1) for e in experiences if e.response_length is not None]
        if ln:
            out["rollout/response_length_mean"] = torch.cat(ln).mean().item()
        tr = [e.truncated.float().reshape(-1) for e in experiences if e.truncated is not None]
        if tr:
            out["rollout/truncated_rate"] = torch.cat(tr).mean().item()
        return out

    # ------------------------------------------------------------------ checkpoints
    def _detect_eval_metric_key(self, metrics: dict):
        if self.best_eval_metric_key == "none":
            return None
        if self.best_eval_metric_key:
            return self.best_eval_metric_key if self.best_eval_metric_key in metrics else None
        for k in sorted(metrics):
            if k.endswith("_pass1"):
                self.best_eval_metric_key = k
                return k
        return None

    def _save(self, tag, client_states, metric_value, metric_key):
        futs = self.group.async_run_method("save_checkpoint", tag=tag, client_states=client_states, role="actor",
                                           metric_value=metric_value, metric_key=metric_key)
        get(futs)
        if self.has_critic:
            get(self.groups.critic.async_run_method("save_checkpoint", tag=tag, role="critic",
                                                    metric_value=metric_value, metric_key=metric_key))

    def save_best_checkpoint(self, eval_metrics: dict, global_step: int, client_states=None):
        if not eval_metrics:
            return
        key = self._detect_eval_metric_key(eval_metrics)
        if key is None:
            return
        value = eval_metrics[key]
        self._latest_eval_metric_value = value
        if value > self.best_eval_metric_value:
            self.best_eval_metric_value = value
            cs = dict(client_states or {})
            cs.update(best_eval_metric_key=key, best_eval_metric_value=value, checkpoint_metric_key=key)
            self._save(f"best_global_step{global_step}", cs, value, key)
            logger.info("saved best checkpoint at step %d (%s=%.4f)", global_step, key, value)

    def save_logs_and_checkpoints(self, global_step: int, logs_dict=None, client_states=None):
        a = self.args
        if global_step % a.logger.logging_steps == 0:
            for lg in self.loggers:
                lg.log_train(global_step, logs_dict or {})
        cs = client_states or {}
        if a.ckpt.save_steps > 0 and global_step % a.ckpt.save_steps == 0:
            self._save(f"global_step{global_step}", cs, self._latest_eval_metric_value,
                       cs.get("checkpoint_metric_key") or self.best_eval_metric_key or None)

    def init_checkpoint_states(self) -> dict:
        a = self.args
        if a.ckpt.load_enable and os.path.exists(os.path.join(a.ckpt.path, "_actor")):
            st = get(self.group.async_run_method("get_checkpoint_states"))[0]
            if st:
                return st
        return {"episode": 0, "global_step": 0, "total_consumed_prompts": 0, "data_loader_state_dict": {}}

    def restore_best_checkpoint_state(self, st: dict):
        if st.get("best_eval_metric_key"):
            self.best_eval_metric_key = st["best_eval_metric_key"]
            self.best_eval_metric_value = st.get("best_eval_metric_value", float("-inf"))


class PPOTrainer(BasePPOTrainer):
    """Synchronous trainer: generation and training alternate on the same workers."""

    def __init__(self, pretrain: str, strategy, group, rollout_engines, has_critic, has_ref, has_reward,
                 rollout_followers=None):
        tokenizer = get_tokenizer(pretrain, None, "left", strategy, use_fast=not strategy.args.data.disable_fast_tokenizer)
        super().__init__(strategy, group, has_critic, has_ref, has_reward, tokenizer)
        self.prompts_dataloader, self.eval_dataloader, self.max_steps = prepare_datasets(strategy, tokenizer)
        self.samples_generator = SamplesGenerator(rollout_engines, strategy, tokenizer, self.prompts_dataloader,
                                                  self.eval_dataloader, followers=rollout_followers)

    def get_max_steps(self) -> int:
        return self.max_steps

    def fit(self, global_step: int = 0) -> None:
        a = self.args
        st = self.init_checkpoint_states()
        self.restore_best_checkpoint_state(st)
        start_episode = st["episode"]
        if st["global_step"] > 0:
            global_step = st["global_step"]
        consumed = st["total_consumed_prompts"]
        if global_step:
            self.broadcast_to_vllm()
            if st.get("data_loader_state_dict") and hasattr(self.prompts_dataloader, "load_state_dict"):
                self.prompts_dataloader.load_state_dict(st["data_loader_state_dict"])
        for episode in range(start_episode, a.train.num_episodes):
            self.samples_generator.restart_epoch()
            while True:
                t0 = time.time()
                samples, pass_rate, n_prompts, exhausted = self.samples_generator.generate_samples(**self.generate_kwargs)
                t_gen = time.time() - t0
                consumed += n_prompts
                if not samples:
                    if exhausted:
                        break
                    continue
                status, global_step = self.train_step(samples, global_step)
                status["timing/generation"] = t_gen
                status["timing/step_total"] = sum(v for k, v in status.items() if k.startswith("timing/"))
                if a.algo.dynamic_filtering_enable:
                    status["dynamic_filtering_pass_rate"] = pass_rate
                logger.info("global step %d: %s", global_step, {k: v for k, v in status.items() if k != "generated_samples"})
                print(f"global step {global_step}: " + ", ".join(
                    f"{k}={v:.4g}" for k, v in status.items() if isinstance(v, (int, float))), flush=True)
                dl_state = self.prompts_dataloader.state_dict() if hasattr(self.prompts_dataloader, "state_dict") else {}
                cs = {"episode": episode, "global_step": global_step, "total_consumed_prompts": consumed,
                      "data_loader_state_dict": dl_state}
                self.save_logs_and_checkpoints(global_step, status, cs)
                if a.eval.steps > 0 and global_step % a.eval.steps == 0 and self.eval_dataloader:
                    kw = dict(self.generate_kwargs, temperature=a.eval.temperature,
                              n_samples_per_prompt=a.eval.n_samples_per_prompt)
                    self.save_best_checkpoint(self.evaluate(global_step, **kw), global_step, cs)
                if exhausted:
                    break
        for lg in self.loggers:
            lg.close()

    def evaluate(self, global_step: int, **gen) -> dict:
        t0 = time.time()
        samples = self.samples_generator.generate_eval_samples(**gen)
        logs = compute_eval_metrics(self.eval_dataloader, samples, gen["n_samples_per_prompt"])
        for lg in self.loggers:
            lg.log_eval(global_step, logs)
        logger.info("evaluation at step %d took %.1f s: %s", global_step, time.time() - t0, logs)
        return logs
