"""End-to-end runs of the RL launcher on one GPU: controller, worker process, rollout engine, experience maker,
training and checkpoint, through the same command line the example scripts use."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

COMMON = [
    "--actor.num_nodes", "1", "--actor.num_gpus_per_node", "1", "--ref.num_nodes", "1", "--ref.num_gpus_per_node", "1",
    "--train.colocate_all", "--vllm.num_engines", "1", "--vllm.tensor_parallel_size", "1",
    "--vllm.gpu_memory_utilization", "0.3", "--actor.model_name_or_path", "tiny-qwen2",
    "--data.prompt_dataset", "synthetic://prompts?n=64&len=24&vocab=2000", "--data.input_key", "input",
    "--data.label_key", "label", "--rollout.batch_size", "8", "--rollout.max_new_tokens", "32", "--data.max_len", "128",
    "--train.batch_size", "16", "--train.micro_batch_size", "4", "--rollout.micro_batch_size", "8",
    "--train.max_epochs", "1", "--train.num_episodes", "1", "--data.max_samples", "16", "--ds.zero_stage", "2",
    "--ds.packing_samples", "--actor.adam.lr", "1e-5",
]

VARIANTS = {
    "reinforce_baseline_reward_func": [
        "--vllm.enable_sleep", "--reward.remote_url", "examples/python/reward_func.py",
        "--algo.advantage.estimator", "reinforce_baseline", "--rollout.n_samples_per_prompt", "4",
        "--algo.kl.init_coef", "1e-3", "--algo.kl.use_loss", "--algo.kl.estimator", "k2"],
    "gae_with_critic": [
        "--vllm.enable_sleep", "--reward.remote_url", "examples/python/reward_func.py",
        "--critic.num_nodes", "1", "--critic.num_gpus_per_node", "1",
        "--algo.advantage.estimator", "gae", "--rollout.n_samples_per_prompt", "2", "--critic.adam.lr", "1e-5"],
    "vlm_reinforce_baseline": [
        "--actor.model_name_or_path", "tiny-qwen2-vl", "--actor.freeze_visual_encoder",
        "--data.prompt_dataset", "synthetic://vlm_prompts?n=64&len=24&vocab=2000&image=56",
        "--data.image_key", "images", "--data.max_images_per_prompt", "1",
        "--reward.remote_url", "examples/python/reward_func.py",
        "--algo.advantage.estimator", "reinforce_baseline", "--rollout.n_samples_per_prompt", "4",
        "--algo.kl.init_coef", "1e-3", "--algo.kl.use_loss", "--algo.kl.estimator", "k2"],
    "async_multiturn_agent": [
        "--train.agent_func_path", "examples/python/agent_func.py", "--train.async_enable",
        "--algo.advantage.estimator", "group_norm", "--rollout.n_samples_per_prompt", "4"],
}


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_train_ppo_ray_end_to_end(variant, tmp_path):
    out_dir = str(tmp_path / "out")
    cmd = [sys.executable, "-m", "openrlhf.cli.train_ppo_ray", *COMMON, *VARIANTS[variant], "--ckpt.output_dir", out_dir]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "global step 1" in r.stdout, tail
    assert os.path.exists(os.path.join(out_dir, "config.json")), tail
    assert any(f.endswith(".safetensors") for f in os.listdir(out_dir)), tail


def _run(args, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return r.stdout + r.stderr


SPMD = ["--data.max_len", "128", "--train.batch_size", "16", "--train.micro_batch_size", "4", "--train.max_epochs", "1",
        "--ds.zero_stage", "2", "--ds.packing_samples", "--adam.lr", "1e-4"]


def test_sft_lora_then_combiner(tmp_path):
    lora_dir, merged = str(tmp_path / "lora"), str(tmp_path / "merged")
    _run(["-m", "openrlhf.cli.train_sft", "--model.model_name_or_path", "tiny-qwen2",
          "--data.dataset", "synthetic://sft?n=64&len=48&vocab=2000", "--data.input_key", "input",
          "--data.output_key", "output", *SPMD, "--ds.lora.rank", "8", "--ds.lora.alpha", "16",
          "--ckpt.output_dir", lora_dir])
    assert os.listdir(lora_dir)
    _run(["-m", "openrlhf.cli.lora_combiner", "--model_path", "tiny-qwen2", "--lora_path", lora_dir,
          "--output_path", merged])
    assert os.path.exists(os.path.join(merged, "config.json"))


def test_rm_then_dpo(tmp_path):
    rm_dir, dpo_dir = str(tmp_path / "rm"), str(tmp_path / "dpo")
    data = ["--data.dataset", "synthetic://preference?n=64&len=48&vocab=2000", "--data.prompt_key", "prompt",
            "--data.chosen_key", "chosen", "--data.rejected_key", "rejected"]
    log = _run(["-m", "openrlhf.cli.train_rm", "--model.model_name_or_path", "tiny-qwen2", *data, *SPMD,
                "--ckpt.output_dir", rm_dir])
    assert "acc" in log
    import json

    cfg = json.load(open(os.path.join(rm_dir, "config.json")))
    assert cfg.get("value_head_prefix") == "score"            # the trained reward model carries its head's name
    _run(["-m", "openrlhf.cli.train_dpo", "--model.model_name_or_path", "tiny-qwen2", "--ref.model_name_or_path",
          "tiny-qwen2", *data, *SPMD, "--model.beta", "0.1", "--ckpt.output_dir", dpo_dir])
    assert os.path.exists(os.path.join(dpo_dir, "config.json"))
