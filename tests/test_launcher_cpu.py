"""The RL launcher end to end on CPU worker processes (gloo): every parallelism / placement flag either takes effect or
raises. The rollout engine, the ZeRO engines and the models run their PyTorch restatements here; the same command lines
run on GPUs in tests/test_cli_gpu.py and tests/dist_scripts/."""
import json
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

COMMON = [
    "--vllm.gpu_memory_utilization", "0.3", "--data.prompt_dataset", "synthetic://prompts?n=64&len=24&vocab=2000",
    "--data.input_key", "input", "--data.label_key", "label", "--rollout.batch_size", "8", "--rollout.max_new_tokens", "12",
    "--data.max_len", "128", "--train.batch_size", "16", "--train.micro_batch_size", "4", "--rollout.micro_batch_size", "8",
    "--train.max_epochs", "1", "--train.num_episodes", "1", "--data.max_samples", "16", "--ds.packing_samples",
    "--actor.adam.lr", "1e-5", "--reward.remote_url", "examples/python/reward_func.py",
    "--algo.advantage.estimator", "reinforce_baseline", "--rollout.n_samples_per_prompt", "4",
]


def _launch(extra, tmp_path, expect_ok=True, timeout=900):
    out_dir = str(tmp_path / "out")
    cmd = [sys.executable, "-m", "openrlhf.cli.train_ppo_ray", *COMMON, *extra, "--ckpt.output_dir", out_dir]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2",
               CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    log = r.stdout + r.stderr
    if expect_ok:
        assert r.returncode == 0, log[-3000:]
        assert "global step 2" in r.stdout, log[-3000:]
        assert os.path.exists(os.path.join(out_dir, "config.json")), log[-2000:]
    return r, log, out_dir


def _metric(log, step, key):
    line = next(ln for ln in log.splitlines() if ln.startswith(f"global step {step}:"))
    return float(re.search(rf"\b{re.escape(key)}=([-+0-9.e]+)", line).group(1))


def test_zero3_for_actor_critic_reference_on_two_workers(tmp_path):
    _, log, _ = _launch(["--actor.num_gpus_per_node", "2", "--critic.num_gpus_per_node", "2", "--train.colocate_all",
                         "--actor.model_name_or_path", "tiny-qwen2", "--ds.zero_stage", "3",
                         "--algo.kl.init_coef", "0.01", "--algo.advantage.estimator", "gae",
                         "--rollout.n_samples_per_prompt", "2"], tmp_path)
    assert _metric(log, 2, "critic_grad_norm") > 0 and _metric(log, 2, "actor_grad_norm") > 0


def test_tensor_parallel_rollout_engine_under_the_controller(tmp_path):
    """Two workers form ONE rollout engine (--vllm.tensor_parallel_size 2): the controller talks to the leader, the
    follower mirrors it; the engine's shards are filled from the ZeRO-3 slices. Rollout log-probs must agree with the
    trainer's, which they only do if both members sampled and cached identically."""
    _, log, _ = _launch(["--actor.num_gpus_per_node", "2", "--train.colocate_all", "--vllm.tensor_parallel_size", "2",
                         "--actor.model_name_or_path", "tiny-qwen2-gqa", "--ds.zero_stage", "3",
                         "--algo.kl.init_coef", "0", "--algo.advantage.is_correction_enable"], tmp_path)
    assert "1 rollout engines x TP 2" in log
    assert abs(_metric(log, 1, "vllm_kl")) < 1e-3       # first step is on-policy: rollout and trainer log-probs agree


def test_separate_rollout_gpus_with_async_training_and_weight_update_group(tmp_path):
    _, log, _ = _launch(["--actor.num_gpus_per_node", "2", "--vllm.num_engines", "2", "--train.async_enable",
                         "--actor.model_name_or_path", "tiny-qwen2", "--ds.zero_stage", "3", "--algo.kl.init_coef", "0",
                         "--algo.advantage.is_correction_enable"], tmp_path)
    # step 2's samples come from engines on other workers that received the updated weights over the sync group
    assert abs(_metric(log, 2, "vllm_kl")) < 5e-2


def test_placement_plan_matches_the_flags():
    from openrlhf_b200.cli import flags as F
    from openrlhf_b200.cli.train_ppo_ray import build_parser, plan_placement, validate

    def plan(extra):
        a = validate(F.finalize(build_parser(), ["--actor.model_name_or_path", "m", "--reward.model_name_or_path", "r",
                                                 "--rollout.batch_size", "64", *extra]))
        return plan_placement(a, True, True, True)

    hybrid = plan(["--train.colocate_all", "--actor.num_gpus_per_node", "8", "--vllm.tensor_parallel_size", "2"])
    assert len(hybrid) == 1 and hybrid[0]["gpus"] == list(range(8)) and set(hybrid[0]["roles"]) == {
        "actor", "critic", "ref", "reward", "rollout"}
    sep = plan(["--actor.num_gpus_per_node", "2", "--critic.num_gpus_per_node", "2", "--ref.num_gpus_per_node", "1",
                "--reward.num_gpus_per_node", "1", "--vllm.num_engines", "1", "--vllm.tensor_parallel_size", "2"])
    assert [(g["name"], g["gpus"]) for g in sep] == [("actor", [0, 1]), ("critic", [2, 3]), ("ref", [4]),
                                                     ("reward", [5]), ("rollout", [6, 7])]
    shared = plan(["--actor.num_gpus_per_node", "2", "--critic.num_gpus_per_node", "2", "--train.colocate_actor_ref",
                   "--train.colocate_critic_reward", "--vllm.num_engines", "2"])
    assert [(g["name"], g["roles"]) for g in shared] == [("actor", ("actor", "ref")), ("critic", ("critic", "reward")),
                                                         ("rollout", ("rollout",))]
    with pytest.raises(ValueError):
        plan(["--train.colocate_all", "--actor.num_gpus_per_node", "3", "--vllm.tensor_parallel_size", "2"])


def test_unsupported_combinations_raise(tmp_path):
    r, log, _ = _launch(["--actor.num_gpus_per_node", "2", "--train.colocate_all", "--actor.model_name_or_path",
                         "tiny-qwen2", "--ds.zero_stage", "3", "--ds.adam_offload", "--algo.kl.init_coef", "0"],
                        tmp_path, expect_ok=False, timeout=300)
    assert r.returncode != 0 and "adam_offload is available with ZeRO stages 1 / 2" in log
    # a tensor-parallel rollout engine needs a worker count it divides
    r, log, _ = _launch(["--actor.num_gpus_per_node", "3", "--train.colocate_all", "--vllm.tensor_parallel_size", "2",
                         "--actor.model_name_or_path", "tiny-qwen2-gqa", "--algo.kl.init_coef", "0"], tmp_path,
                        expect_ok=False, timeout=300)
    assert r.returncode != 0 and "does not divide" in log


def test_checkpoint_resume_continues_from_the_saved_step(tmp_path):
    ck = str(tmp_path / "ckpt")
    base = ["--actor.num_gpus_per_node", "1", "--train.colocate_all", "--actor.model_name_or_path", "tiny-qwen2",
            "--ds.zero_stage", "2", "--algo.kl.init_coef", "0", "--ckpt.path", ck, "--ckpt.save_steps", "1",
            "--ds.adam_offload"]
    r, log, _ = _launch(base + ["--data.max_samples", "8"], tmp_path, expect_ok=False)   # one step, checkpointed
    assert r.returncode == 0 and "global step 1" in r.stdout, log[-3000:]
    assert os.path.exists(os.path.join(ck, "_actor", "latest"))
    r, log, _ = _launch(base + ["--data.max_samples", "16", "--ckpt.load_enable"], tmp_path, expect_ok=False)
    assert r.returncode == 0, log[-3000:]
    steps = [int(m) for m in re.findall(r"^global step (\d+):", r.stdout, flags=re.M)]
    assert steps and steps[0] == 2, steps                               # resumed after step 1, not from scratch


def test_worker_death_restarts_the_job_from_its_last_checkpoint(tmp_path):
    """--train.max_restarts: a worker process that dies in the middle of the run (here: killed on the host by its own
    reward function, once, during the third rollout) surfaces as WorkerDied in the controller, which stops all
    workers, starts them again and resumes from the last checkpoint; the run then finishes all its steps."""
    marker = tmp_path / "died_once"
    counter = tmp_path / "calls"
    reward = tmp_path / "reward_func.py"
    reward.write_text(
        "import os, torch\n"
        f"MARKER, COUNTER = {str(marker)!r}, {str(counter)!r}\n"
        "def reward_func(queries, prompts, labels, **kw):\n"
        "    fd = os.open(COUNTER, os.O_WRONLY | os.O_CREAT | os.O_APPEND)   # one byte per call, from any thread\n"
        "    os.write(fd, b'x'); os.close(fd)\n"
        "    n = os.path.getsize(COUNTER)\n"
        "    if n > 70 and not os.path.exists(MARKER):      # 32 samples per rollout: inside the third one\n"
        "        open(MARKER, 'w').write('x')\n"
        "        os._exit(17)                               # the worker process ends here, on the host\n"
        "    return {'rewards': torch.tensor([float(len(q) % 2) for q in queries]), 'scores': torch.zeros(len(queries)),\n"
        "            'extra_logs': {}}\n")
    ck = str(tmp_path / "ckpt")
    common = [c for c in COMMON]
    common[common.index("--reward.remote_url") + 1] = str(reward)
    common[common.index("--data.max_samples") + 1] = "32"            # four rollouts of 8 prompts
    cmd = [sys.executable, "-m", "openrlhf.cli.train_ppo_ray", *common, "--actor.num_gpus_per_node", "1",
           "--train.colocate_all", "--actor.model_name_or_path", "tiny-qwen2", "--ds.zero_stage", "2",
           "--algo.kl.init_coef", "0", "--ckpt.path", ck, "--ckpt.save_steps", "1", "--train.max_restarts", "1",
           "--ckpt.output_dir", str(tmp_path / "out")]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2",
               CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    log = r.stdout + r.stderr
    assert r.returncode == 0, log[-4000:]
    assert marker.exists() and "restarting the job from its last checkpoint" in log, log[-4000:]
    steps = [int(m) for m in re.findall(r"^global step (\d+):", r.stdout, flags=re.M)]
    # steps before the death, then the resumed run continues after the last checkpointed step up to the last one
    assert steps[-1] == 4 and steps.count(1) == 1 and len(steps) >= 4, steps
    assert os.path.exists(os.path.join(str(tmp_path / "out"), "config.json"))


def test_worker_environment_defaults_yield_to_the_user():
    from openrlhf_b200.cli.train_ppo_ray import apply_env_defaults

    assert apply_env_defaults({}) == {"TOKENIZERS_PARALLELISM": "true", "NCCL_DEBUG": "WARN"}
    user = {"NCCL_DEBUG": "INFO", "TOKENIZERS_PARALLELISM": "false", "OTHER": "1"}
    assert apply_env_defaults(user) == {"TOKENIZERS_PARALLELISM": "false", "NCCL_DEBUG": "INFO"} and user["OTHER"] == "1"
