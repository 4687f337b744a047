"""CPU oracle determinism, trainer control flow with a fake worker group, environment handed to workers."""
import os
import sys
from types import SimpleNamespace

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))


def test_cpu_oracle_is_deterministic_and_on_policy():
    import cpu_oracle

    a = cpu_oracle.grpo_step(n_prompts=2, prompt_len=8, n=4, new_tokens=6)
    b = cpu_oracle.grpo_step(n_prompts=2, prompt_len=8, n=4, new_tokens=6)
    assert a["checksum"] == b["checksum"] and a["loss"] == b["loss"]
    # first step is on-policy and the reference equals the policy: the surrogate is -mean(advantage) and the KL is 0
    assert abs(a["kl_loss"]) < 1e-6 and a["grad_norm"] > 0 and a["samples"] == 8


class _FakeGroup:
    """Stands in for runtime.core.ActorGroup: records calls, answers instantly."""

    duplicate_actors = 1

    def __init__(self):
        self.calls = []

    def _fut(self, value):
        from openrlhf_b200.runtime.core import Future

        f = Future()
        f.set_result(value)
        return f

    def async_run_method(self, name, *a, **kw):
        self.calls.append(name)
        return [self._fut({"policy_loss": 0.0} if name == "fit" else None)]

    def async_run_method_batch(self, name, **kw):
        self.calls.append(name)
        return [self._fut([None])]


def _trainer(batches):
    from openrlhf_b200.trainer.ppo_trainer import PPOTrainer

    t = PPOTrainer.__new__(PPOTrainer)
    t.args = SimpleNamespace(train=SimpleNamespace(num_episodes=1, dynamic_batch_enable=False),
                             algo=SimpleNamespace(dynamic_filtering_enable=False),
                             eval=SimpleNamespace(steps=-1), ckpt=SimpleNamespace(load_enable=False, path="/nonexistent",
                                                                                   save_steps=-1),
                             logger=SimpleNamespace(logging_steps=1), vllm=SimpleNamespace(enable_sleep=False))
    t.group, t.has_critic, t.loggers = _FakeGroup(), False, []
    t.generate_kwargs, t.eval_dataloader, t.prompts_dataloader = {}, None, SimpleNamespace()
    t.best_eval_metric_key, t.best_eval_metric_value, t._latest_eval_metric_value = "", float("-inf"), None
    it = iter(batches)
    t.samples_generator = SimpleNamespace(restart_epoch=lambda: None, generate_samples=lambda **kw: next(it))
    trained = []
    t.train_step = lambda samples, step: (trained.append(len(samples)) or ({"timing/x": 0.0}, step + 1))
    return t, trained


def test_fit_trains_on_final_non_empty_batch_and_skips_empty_one():
    t, trained = _trainer([(["s1", "s2"], None, 2, False), (["s3"], None, 1, True)])
    t.fit()
    assert trained == [2, 1]            # the last batch arrives together with the exhaustion flag and is still used
    t, trained = _trainer([(["s1"], None, 1, False), ([], None, 0, True)])
    t.fit()
    assert trained == [1]               # an empty batch at exhaustion is not trained on


def test_worker_environment_and_user_overrides():
    from openrlhf_b200.runtime.core import ActorGroup, get

    os.environ["NCCL_DEBUG"] = "WARN"
    try:
        g = ActorGroup("worker_stubs.EnvWorker", 2, backend_env={"TOKENIZERS_PARALLELISM": "true"},
                       name="env")
        try:
            envs = get(g.async_run_method("env", ["RANK", "WORLD_SIZE", "MASTER_ADDR", "NCCL_DEBUG",
                                                  "TOKENIZERS_PARALLELISM"]), 60)
        finally:
            g.shutdown()
    finally:
        del os.environ["NCCL_DEBUG"]
    assert [e["RANK"] for e in envs] == ["0", "1"] and all(e["WORLD_SIZE"] == "2" for e in envs)
    assert all(e["MASTER_ADDR"] == "127.0.0.1" for e in envs)
    assert all(e["NCCL_DEBUG"] == "WARN" for e in envs)          # the user's setting reaches the workers
    assert all(e["TOKENIZERS_PARALLELISM"] == "true" for e in envs)
