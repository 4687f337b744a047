"""``python -m openrlhf.cli.train_ppo_ray``: PPO / REINFORCE++(-baseline) / GRPO / Dr.GRPO / RLOO training under a single
controller. Flag-compatible with openrlhf/cli/train_ppo_ray.py:198-717 (the module keeps its name for launch-script
compatibility; the workers are this framework's runtime processes, one per GPU, not Ray actors).

Placement (``plan_placement``): with ``--train.colocate_all`` (hybrid engine) every GPU worker hosts all roles, the
rollout engine reads the buffer the actor's optimizer writes (or is refreshed from the ZeRO-3 / tensor-parallel shards by
one copy kernel), and ``--vllm.tensor_parallel_size`` consecutive workers form one engine. Without it every role group
gets its own GPUs and its own process-group world; the rollout engines receive weights from trainer rank 0 over a
separate weight-update group, and ``--train.async_enable`` then overlaps generation with training.
"""
from __future__ import annotations

import argparse
import os

from ..runtime.core import ActorGroup, WorkerDied, get
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
    # not a reference flag: how often a job whose worker died is restarted from its last checkpoint inside this process
    ("--train.max_restarts", int, 0),
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


def plan_placement(a, has_critic: bool, has_ref: bool, has_reward: bool) -> list[dict]:
    """Which worker groups to start, on which GPUs, with which roles (openrlhf/cli/train_ppo_ray.py:40-142).

    ``--train.colocate_all``: one group of ``actor.num_nodes x actor.num_gpus_per_node`` workers hosts every role, and
    ``--vllm.tensor_parallel_size`` consecutive workers form one rollout engine (hybrid engine).
    Otherwise each role gets its own GPUs in the order actor, critic, reference, reward, rollout engines, where
    ``--train.colocate_actor_ref`` puts the reference model on the actor's workers and
    ``--train.colocate_critic_reward`` the reward model on the critic's. Returns a list of
    {"name", "roles", "gpus", "serves"} entries; "serves" names the roles the trainer addresses through that group."""
    n_actor = a.actor.num_nodes * a.actor.num_gpus_per_node
    tp = max(1, a.vllm.tensor_parallel_size)
    if a.train.colocate_all:
        if n_actor % tp:
            raise ValueError(f"--vllm.tensor_parallel_size {tp} does not divide the {n_actor} hybrid-engine workers")
        if a.vllm.num_engines * tp != n_actor:
            print(f"[Info] hybrid engine: {n_actor // tp} rollout engines x TP {tp} on the {n_actor} workers "
                  f"(--vllm.num_engines {a.vllm.num_engines} adjusted)")
            a.vllm.num_engines = n_actor // tp
        roles = ["actor", "rollout"] + (["critic"] if has_critic else []) + (["ref"] if has_ref else []) + \
                (["reward"] if has_reward else [])
        return [{"name": "rl", "roles": tuple(roles), "gpus": list(range(n_actor)), "serves": tuple(roles)}]
    groups, nxt = [], 0

    def take(n):
        nonlocal nxt
        ids = list(range(nxt, nxt + n))
        nxt += n
        return ids

    actor_roles = ["actor"] + (["ref"] if has_ref and a.train.colocate_actor_ref else [])
    groups.append({"name": "actor", "roles": tuple(actor_roles), "gpus": take(n_actor), "serves": tuple(actor_roles)})
    if has_critic:
        cr = ["critic"] + (["reward"] if has_reward and a.train.colocate_critic_reward else [])
        groups.append({"name": "critic", "roles": tuple(cr), "gpus": take(a.critic.num_nodes * a.critic.num_gpus_per_node),
                       "serves": tuple(cr)})
    if has_ref and not a.train.colocate_actor_ref:
        groups.append({"name": "ref", "roles": ("ref",), "gpus": take(a.ref.num_nodes * a.ref.num_gpus_per_node),
                       "serves": ("ref",)})
    if has_reward and not (has_critic and a.train.colocate_critic_reward):
        groups.append({"name": "reward", "roles": ("reward",),
                       "gpus": take(a.reward.num_nodes * a.reward.num_gpus_per_node), "serves": ("reward",)})
    groups.append({"name": "rollout", "roles": ("rollout",), "gpus": take(a.vllm.num_engines * tp),
                   "serves": ("rollout",)})
    return groups


# Environment of the controller and, by inheritance, of every worker process it starts; a value the user exported wins
# (the reference passes the same defaults to its actors: openrlhf/cli/train_ppo_ray.py, runtime_env of ray.init).
ENV_DEFAULTS = {"TOKENIZERS_PARALLELISM": "true", "NCCL_DEBUG": "WARN"}


def apply_env_defaults(environ=None) -> dict:
    environ = os.environ if environ is None else environ
    for key, value in ENV_DEFAULTS.items():
        environ.setdefault(key, value)
    return {k: environ[k] for k in ENV_DEFAULTS}


def train(args):
    import torch

    a = args
    apply_env_defaults()
    strategy = get_strategy(a)                      # controller-side copy: flags + CPU helpers, no process group
    has_critic = a.critic.model_name_or_path is not None
    has_ref = a.algo.kl.init_coef > 0
    has_reward = bool(a.reward.model_name_or_path) and not a.reward.remote_url
    on_gpu = torch.cuda.is_available()
    backend = "nccl" if on_gpu else "gloo"
    plan = plan_placement(a, has_critic, has_ref, has_reward)
    need = max(max(g["gpus"]) for g in plan) + 1
    if on_gpu and need > torch.cuda.device_count():
        raise ValueError(f"the placement needs {need} GPUs on this node but {torch.cuda.device_count()} are visible; "
                         "pass --train.colocate_all (hybrid engine) or lower the per-role GPU counts")
    if a.train.async_enable and a.train.colocate_all and on_gpu:
        print("[Info] --train.async_enable with --train.colocate_all time-slices the same GPUs; give the rollout "
              "engines their own GPUs (drop --train.colocate_all) for generation to overlap with training.")
    dup_train = a.ds.ring_attn_size * a.ds.tensor_parallel_size
    tp = max(1, a.vllm.tensor_parallel_size)
    # Recovery: a dead worker (process exit, missed heartbeats) surfaces as WorkerDied from a future. The reference
    # leaves the restart to the user (relaunch with --ckpt.load_enable, openrlhf/trainer/ppo_trainer.py:429-442);
    # with --train.max_restarts N the controller does that itself: it stops every worker of the job, builds the
    # worker groups again and resumes from the last checkpoint (what was done since that checkpoint is repeated).
    restarts_left = int(getattr(a.train, "max_restarts", 0) or 0)
    while True:
        try:
            return _run_job(a, strategy, plan, on_gpu, backend, dup_train, tp, has_critic, has_ref, has_reward)
        except WorkerDied as e:
            if restarts_left <= 0:
                raise
            if not (a.ckpt.path and a.ckpt.save_steps and a.ckpt.save_steps > 0):
                print("[Warning] a worker died and --train.max_restarts is set, but the job writes no checkpoints "
                      "(--ckpt.path / --ckpt.save_steps): nothing to resume from", flush=True)
                raise
            restarts_left -= 1
            print(f"[Warning] worker died ({e}); restarting the job from its last checkpoint "
                  f"({restarts_left} restarts left)", flush=True)
            a.ckpt.load_enable = True


def _run_job(a, strategy, plan, on_gpu, backend, dup_train, tp, has_critic, has_ref, has_reward):
    """Build the worker groups of one placement plan, train, save; always stops the workers it started."""
    import copy

    from ..runtime.core import free_port
    from ..trainer.ppo_trainer import PPOTrainer, RoleGroups
    from ..trainer.ppo_trainer_async import PPOTrainerAsync

    made: dict[str, ActorGroup] = {}
    try:
        for g in plan:
            ga = a
            if g["name"] in ("ref", "reward", "rollout"):
                # inference-only worlds of their own size: no ring-attention / tensor-parallel training mesh there
                ga = copy.deepcopy(a)
                ga.ds.ring_attn_size = ga.ds.tensor_parallel_size = 1
            dup = dup_train if ga is a else 1
            made[g["name"]] = ActorGroup("openrlhf_b200.runtime.workers.RLWorker", len(g["gpus"]),
                                         init_kwargs={"args": ga, "roles": g["roles"], "max_steps": 1000,
                                                      "backend": backend},
                                         gpu_ids=g["gpus"] if on_gpu else None, duplicate_actors=dup, name=g["name"])
        by_role = {r: made[g["name"]] for g in plan for r in g["serves"]}
        main = by_role["actor"]
        rollout_group = by_role["rollout"]
        groups = RoleGroups(main, by_role.get("critic"), by_role.get("ref"), by_role.get("reward"),
                            rollout_group if rollout_group is not main else None)
        if rollout_group is not main:
            # weight-update group: trainer rank 0 + every rollout rank, next to the two training / rollout worlds
            port, n = free_port(), 1 + len(rollout_group)
            futs = [main.workers[0].call("setup_sync_group", "127.0.0.1", port, 0, n, backend)]
            futs += [w.call("setup_sync_group", "127.0.0.1", port, 1 + i, n, backend)
                     for i, w in enumerate(rollout_group.workers)]
            get(futs)
        engines = rollout_group.workers[::tp]
        followers = [w for i, w in enumerate(rollout_group.workers) if i % tp]
        cls = PPOTrainerAsync if a.train.async_enable else PPOTrainer
        trainer = cls(a.actor.model_name_or_path, strategy, groups, engines, has_critic, has_ref, has_reward,
                      rollout_followers=followers)
        trainer.fit()
        get(main.async_run_method("save_model", role="actor"))
        if has_critic and a.critic.save_value_network:
            get(groups.critic.async_run_method("save_model", role="critic"))
    finally:
        for g in made.values():
            g.shutdown()


if __name__ == "__main__":
    train(validate(F.finalize(build_parser())))
