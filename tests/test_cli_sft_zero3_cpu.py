"""train_sft CLI end to end on two CPU ranks (gloo) with --ds.zero_stage 3: training steps, sharded optimizer
checkpoints, HF export of the gathered weights, and resume."""
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(out, extra=()):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29773", "-m", "openrlhf.cli.train_sft", "--model.model_name_or_path",
           "tiny-llama", "--data.dataset", "synthetic://sft?n=64&len=32&vocab=1000", "--data.input_key", "input",
           "--data.output_key", "output", "--data.max_len", "64", "--train.batch_size", "16",
           "--train.micro_batch_size", "4", "--train.max_epochs", "1", "--ds.zero_stage", "3", "--ds.packing_samples",
           "--adam.lr", "1e-3", "--ckpt.output_dir", out, "--ckpt.save_steps", "2", "--ckpt.path",
           os.path.join(out, "ckpt"), *extra]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout + r.stderr


def test_sft_cli_zero3_two_ranks(tmp_path):
    out = str(tmp_path / "sft")
    log = _run(out)
    assert "step 4" in log and "grad_norm" in log
    assert os.path.exists(os.path.join(out, "model.safetensors")) and os.path.exists(os.path.join(out, "config.json"))
    files = os.listdir(os.path.join(out, "ckpt", "global_step4"))
    assert {"manifest.json", "shard_00000.safetensors", "shard_00001.safetensors"} <= set(files), files
    # the exported weights are the trained ones: they load back and differ from the seed-0 initialisation
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.hf_io import load_pretrained
    from openrlhf_b200.models.transformer import TransformerLM
    trained = load_pretrained(out, device="cpu")
    init = TransformerLM(PRESETS["tiny-llama"], device="cpu", seed=42)
    a = torch.cat([p.detach().float().flatten() for _, p in trained.named_specs()])
    b = torch.cat([p.detach().float().flatten() for _, p in init.named_specs()])
    assert a.shape == b.shape and torch.isfinite(a).all() and (a - b).abs().max() > 1e-4
    # resume from the sharded checkpoint
    log2 = _run(out, ("--ckpt.load_enable",))
    assert "Loaded the checkpoint" in log2
