"""``python -m openrlhf.cli.train_ppo_ray``: PPO / REINFORCE++(-baseline) / GRPO / Dr.GRPO / RLOO training under a single
controller. Flag-compatible with openrlhf/cli/train_ppo_ray.py:198-717 (the module keeps its name for launch-script
compatibility; the workers are this framework's runtime processes, one per GPU, not Ray actors).

Placement: with ``--train.colocate_all`` (hybrid engine) every GPU worker hosts all roles and the rollout engine reads
the buffer the actor's optimizer writes. Without it, rollout engines get their own GPUs after the trainer GPUs and
receive weights by NCCL broadcast from the actor.
"""
from __future__ import annotations

import argparse
import os

from ..runtime.core import ActorGroup, get
from ..utils.strategy import get_strategy
from . import flags as F

B = F.BOOL

RL_FLAGS = [
    # placement
    ("--ref.num_nodes", int, 1), ("--ref.num_gpus_per_node", int, 8), ("--reward.num_nodes", int, 1),
    ("--reward.num_gpus_per_node", int, 8), ("--actor.num_nodes", int, 1), ("--actor.num_gpus_per_node", int, 8),
    ("--critic.num_nodes", int, 1), ("--critic.num_gpus_per_node", int, 8), ("--train.colocate_actor_ref", B, False),
    ("--train.colocate_critic_reward", B, False), ("--train.colocate_all", B, False),
    # rollout engine
    ("--vllm.num_engines", int, None), ("--vllm.tensor_parallel_size", int, 1), ("--vllm.sync_backend", str, "nccl"),
    ("--vllm.sync_with_ray", B, False), ("--vllm.enable_prefix_caching", B, False), ("--vllm.enforce_eager", B, False),
    ("--vllm.enable_sleep", B, False), ("--vllm.gpu_memory_utilization", float, 0.95), ("--vllm.max_num_seqs", int, 256),
    ("--vllm.quantization", str, None),
    # algorithm
    ("--algo.advantage.is_correction_enable", B, False),
    ("--algo.advantage.is_correction_threshold", float, [0.5, 5.0], {"nargs": 2}),
    ("--algo.advantage.is_correction_type", str, "tis", {"choices": ["tis", "icepop", "seq-mask-tis"]}),
    ("--algo.advantage.estimator", str, "gae",
     {"choices": ["gae", "reinforce", "rloo", "reinforce_baseline", "group_norm", "dr_grpo"]}),
    ("--algo.advantage.lambd", float, 1), ("--algo.advantage.gamma", float, 1), ("--algo.advantage.no_std_norm", B, False),
    ("--algo.kl.target", float, None), ("--algo.kl.horizon", int, 10000), ("--algo.kl.init_coef", float, 0.01),
    ("--algo.kl.estimator", str, "k1", {"choices": ["k1", "k2", "k3"]}), ("--algo.kl.use_loss", B, False),
    ("--algo.dynamic_filtering_enable", B, False), ("--algo.dynamic_filtering_range", float, (0, 1), {"nargs": 2}),
    # training loop
    ("--train.async_enable", B, False), ("--train.async_queue_size", int, 1), ("--train.partial_rollout_enable", B, False),
    ("--train.enable_ema", B, False), ("--train.ema_beta", float, 0.992), ("--train.dynamic_batch_enable", B, False),
    ("--train.max_tokens_per_gpu", int, 16192), ("--train.num_episodes", int, 1), ("--train.max_epochs", int, 1),
    ("--train.micro_batch_size", int, 1), ("--train.batch_size", int, 128), ("--train.seed", int, 42),
    ("--train.full_determinism_enable", B, False), ("--train.agent_func_path", str, None),
    # rollout
    ("--rollout.max_tokens_per_gpu", int, None), ("--rollout.batch_size", int, 1024),
    ("--rollout.vllm_generate_batch_size", int, None), ("--rollout.micro_batch_size", int, 1),
    ("--rollout.max_new_tokens", int, None), ("--rollout.top_p", float, 1.0), ("--rollout.temperature", float, 1.0),
    ("--rollout.n_samples_per_prompt", int, 1),
    # models
    ("--actor.gradient_checkpointing_enable", B, False), ("--actor.gradient_checkpointing_reentrant", B, False),
    ("--actor.eps_clip", float, 0.2), ("--actor.eps_clip_low_high", float, None, {"nargs": 2}),
    ("--actor.dual_clip", float, None), ("--actor.policy_loss_type", str, "ppo", {"choices": ["ppo", "gspo"]}),
    ("--actor.aux_loss_coef", float, 0), ("--actor.entropy_coef", float, None), ("--actor.model_name_or_path", str, None),
    ("--actor.freeze_visual_encoder", B, False), ("--critic.value_clip", float, 0.5), ("--critic.freezing_steps", int, -1),
    ("--critic.save_value_network", B, False), ("--critic.model_name_or_path", str, None),
    ("--reward.normalize_enable", B, False), ("--reward.clip_range", float, (-10, 10), {"nargs": 2}),
    ("--reward.overlong_buffer_len", float, None), ("--reward.overlong_penalty_factor", float, 1),
    ("--reward.stop_properly_penalty_coef", float, None), ("--reward.model_name_or_path", str, None),
    ("--reward.remote_url", str, None), ("--reward.offload", B, False), ("--ref.offload", B, False),
    ("--ref.model_name_or_path", str, None), ("--ds.enable_sleep", B, False),
    # data / eval
    ("--data.disable_fast_tokenizer", B, False), ("--data.dataloader_num_workers", int, 0), ("--data.max_len", int, 2048),
    ("--data.max_samples", int, int(1e8)), ("--data.prompt_dataset", str, None), ("--data.prompt_probs", str, None),
    ("--data.prompt_split", str, "train"), ("--data.input_key", str, "input"), ("--data.label_key", str, None),
    ("--data.input_template", str, None), ("--data.apply_chat_template", B, False), ("--data.image_key", str, "images"),
    ("--data.max_images_per_prompt", int, 0), ("--eval.dataset", str, None), ("--eval.split", str, "train"),
    ("--eval.temperature", float, 0.6), ("--eval.n_samples_per_prompt", int, 4), ("--eval.steps", int, -1),
    # checkpoints
    ("--ckpt.save_steps", int, -1), ("--ckpt.path", str, "./ckpt/checkpoints_ppo_ray"), ("--ckpt.save_hf", B, False),
    ("--ckpt.disable_ds", B, False), ("--ckpt.max_num", int, 3), ("--ckpt.max_mem", float, float("inf")),
    ("--ckpt.load_enable", B, False), ("--ckpt.best_metric_key", str, ""), ("--ckpt.output_dir", str, "./ckpt"),
    ("--rollout.ignore_eos", B, False),
]


def build_parser():
    p = argparse.ArgumentParser()
    F.add_flags(p, RL_FLAGS, F.logger_flags("openrlhf_train_ppo", "ppo"), F.ENGINE,
                F.optimizer_flags("actor.", 1e-6), F.optimizer_flags("critic.", 9e-6))
    return p


def validate(args):
    """Derived settings and cross-flag checks (openrlhf/cli/train_ppo_ray.py:593-717)."""
    a = args
    if a.actor.eps_clip_low_high is None:
        a.actor.eps_clip_low_high = (a.actor.eps_clip, a.actor.eps_clip)
    a.actor.eps_clip_low_high = tuple(a.actor.eps_clip_low_high)
    if a.train.agent_func_path:
        a.reward.remote_url = "agent"
    if a.algo.advantage.estimator != "gae":
        a.critic.model_name_or_path = None
    elif a.critic.model_name_or_path is None:
        a.critic.model_name_or_path = (a.actor.model_name_or_path if a.reward.remote_url
                                       else a.reward.model_name_or_path.split(",")[0])
    if a.algo.advantage.estimator in ("rloo", "reinforce_baseline", "group_norm", "dr_grpo"):
        assert a.rollout.n_samples_per_prompt > 1, f"{a.algo.advantage.estimator} requires n_samples_per_prompt > 1"
    if a.data.max_images_per_prompt > 0:
        assert a.critic.model_name_or_path is None, "VLM training does not support a critic model; use a critic-free estimator"
    if a.reward.remote_url and isinstance(a.reward.remote_url, str):
        a.reward.remote_url = a.reward.remote_url.split(",")
    if a.data.input_template and "{}" not in a.data.input_template:
        print("[Warning] '{}' not in --data.input_template; set to None")
        a.data.input_template = None
    if a.data.input_template and "\\n" in a.data.input_template:
        print("[Warning] input_template contains \\n characters instead of newline.")
    if a.ds.ring_attn_size > 1 and not a.ds.packing_samples:
        print("[Warning] --ds.ring_attn_size > 1 requires --ds.packing_samples.")
        a.ds.packing_samples = True
    if a.train.dynamic_batch_enable:
        if not a.ds.packing_samples:
            print("[Warning] --train.dynamic_batch_enable works on packed samples; enabling --ds.packing_samples.")
            a.ds.packing_samples = True
        if a.rollout.max_tokens_per_gpu is None:
            a.rollout.max_tokens_per_gpu = a.train.max_tokens_per_gpu
    if a.vllm.num_engines is None:
        a.vllm.num_engines = a.actor.num_nodes * a.actor.num_gpus_per_node if a.train.colocate_all else 1
    assert a.vllm.num_engines > 0, "a rollout engine is required"
    if a.vllm.enable_sleep and not a.train.colocate_all:
        print("--vllm.enable_sleep needs --train.colocate_all; disabled.")
        a.vllm.enable_sleep = False
    if a.train.async_enable:
        assert not a.vllm.enable_sleep, "async training is not supported with --vllm.enable_sleep"
    if a.train.partial_rollout_enable:
        assert a.train.async_enable, "--train.partial_rollout_enable requires --train.async_enable"
    if a.eval.dataset:
        assert a.reward.remote_url or a.train.agent_func_path, \
            "--eval.dataset requires --reward.remote_url (remote RM / reward_func.py) or --train.agent_func_path"
    if a.algo.kl.use_loss and a.algo.kl.estimator not in ("k2", "k3"):
        print(f"Recommend --algo.kl.estimator k2 or k3 when the KL is used as a loss (got {a.algo.kl.estimator})")
    if not a.algo.kl.use_loss and a.algo.kl.estimator != "k1":
        print(f"Recommend --algo.kl.estimator k1 when the KL is a reward penalty (got {a.algo.kl.estimator})")
    if not a.rollout.vllm_generate_batch_size:
        a.rollout.vllm_generate_batch_size = a.rollout.batch_size
    if a.rollout.vllm_generate_batch_size > a.rollout.batch_size:
        assert a.train.async_enable, "over-sampling (--rollout.vllm_generate_batch_size > --rollout.batch_size) requires --train.async_enable"
    if a.algo.dynamic_filtering_enable:
        lo, hi = a.algo.dynamic_filtering_range
        assert lo < hi, "dynamic_filtering_range[0] must be less than dynamic_filtering_range[1]"
        assert a.reward.remote_url or a.train.agent_func_path, "dynamic filtering needs a remote reward or an agent"
        assert a.rollout.n_samples_per_prompt > 1, "dynamic filtering needs n_samples_per_prompt > 1"
    eff = a.actor.num_nodes * a.actor.num_gpus_per_node // a.ds.ring_attn_size // a.ds.tensor_parallel_size
    assert a.rollout.n_samples_per_prompt * a.rollout.batch_size // a.rollout.micro_batch_size >= eff, \
        "The number of sample batches must be greater than or equal to the effective number of actor processes."
    return a


def train(args):
    from ..trainer.ppo_trainer import PPOTrainer
    from ..trainer.ppo_trainer_async import PPOTrainerAsync

    a = args
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "true")
    strategy = get_strategy(a)                      # controller-side copy: flags + CPU helpers, no process group
    n_train = a.actor.num_nodes * a.actor.num_gpus_per_node
    has_critic = a.critic.model_name_or_path is not None
    has_ref = a.algo.kl.init_coef > 0
    has_reward = bool(a.reward.model_name_or_path) and not a.reward.remote_url
    import torch

    backend = "nccl" if torch.cuda.is_available() else "gloo"
    # one worker per GPU; under --train.colocate_all every worker carries every role (hybrid engine)
    roles = ["actor", "rollout"] + (["critic"] if has_critic else []) + (["ref"] if has_ref else []) + \
            (["reward"] if has_reward else [])
    if not a.train.colocate_all:
        print("[Info] roles are placed on the same GPU workers; pass --train.colocate_all to make it explicit.")
    group = ActorGroup("openrlhf_b200.runtime.workers.RLWorker", n_train,
                       init_kwargs={"args": a, "roles": tuple(roles), "max_steps": 1000, "backend": backend},
                       duplicate_actors=a.ds.ring_attn_size * a.ds.tensor_parallel_size, name="rl")
    engines = group.workers[:: max(1, a.vllm.tensor_parallel_size)][: a.vllm.num_engines] or group.workers
    cls = PPOTrainerAsync if a.train.async_enable else PPOTrainer
    trainer = cls(a.actor.model_name_or_path, strategy, group, engines, has_critic, has_ref, has_reward)
    try:
        trainer.fit()
        get(group.async_run_method("save_model", role="actor"))
        if has_critic and a.critic.save_value_network:
            get(group.async_run_method("save_model", role="critic"))
    finally:
        group.shutdown()


if __name__ == "__main__":
    train(validate(F.finalize(build_parser())))
