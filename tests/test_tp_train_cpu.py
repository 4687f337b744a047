"""Tensor-parallel training on CPU ranks (gloo): engine-level parity with unsharded training for tp = 2 alone and
with data parallelism, and the SFT launcher end to end with --ds.tensor_parallel_size 2."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, port, tail_args, timeout=900):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(port), *tail_args]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", TP_TEST_CPU="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout + r.stderr


@pytest.mark.parametrize("nproc", [2, 4])
def test_tp_training_matches_unsharded(nproc):
    out = _torchrun(nproc, 29820 + nproc, [os.path.join(ROOT, "tests", "dist_scripts", "tp_train.py")])
    assert "TP_TRAIN_OK" in out


def test_sft_cli_tensor_parallel(tmp_path):
    out_dir = str(tmp_path / "sft_tp")
    log = _torchrun(2, 29831, [
        "-m", "openrlhf.cli.train_sft", "--model.model_name_or_path", "tiny-llama", "--data.dataset",
        "synthetic://sft?n=64&len=32&vocab=1000", "--data.input_key", "input", "--data.output_key", "output",
        "--data.max_len", "64", "--train.batch_size", "8", "--train.micro_batch_size", "4", "--train.max_epochs", "1",
        "--ds.zero_stage", "2", "--ds.tensor_parallel_size", "2", "--ds.packing_samples", "--adam.lr", "1e-3",
        "--ckpt.output_dir", out_dir, "--ckpt.save_steps", "4", "--ckpt.path", os.path.join(out_dir, "ckpt")])
    assert "grad_norm" in log
    # both tp ranks consumed the same 64 samples in batches of 8: 8 optimizer steps, not 4
    assert "step 8" in log
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.hf_io import load_pretrained
    from openrlhf_b200.models.transformer import TransformerLM

    trained = load_pretrained(out_dir, device="cpu")          # the export is the full (unsharded) HF layout
    cfg = PRESETS["tiny-llama"]
    assert trained.cfg.num_attention_heads == cfg.num_attention_heads
    assert trained.p("layers.0.qkv.weight").shape == (cfg.qkv_size, cfg.hidden_size)
    init = TransformerLM(cfg, device="cpu", seed=42)
    a = torch.cat([p.detach().float().flatten() for _, p in trained.named_specs()])
    b = torch.cat([p.detach().float().flatten() for _, p in init.named_specs()])
    assert torch.isfinite(a).all() and (a - b).abs().max() > 1e-4
    files = os.listdir(os.path.join(out_dir, "ckpt", "global_step8"))
    assert {"tp_00", "tp_01"} <= set(files), files


def test_shard_plan_round_trip_with_value_head():
    """full -> tp shards (copy plan) -> full (the inverse used for HF export) is the identity, value head included."""
    from openrlhf_b200.models.config import ModelConfig
    from openrlhf_b200.models.transformer import build_param_specs
    from openrlhf_b200.parallel.reshard import build_plan, run_plan_reference, tp_param_specs

    cfg = ModelConfig("qwen2", 512, 128, 256, 2, 4, 2, head_dim=64, attention_bias=True)
    specs = build_param_specs(cfg, with_lm_head=False, with_value_head=True)
    total = specs[-1].offset + specs[-1].numel
    full = torch.arange(total, dtype=torch.float32)
    back = torch.full((total,), -1.0)
    tp = 2
    for r in range(tp):
        entries, size = build_plan(cfg, r, tp, with_lm_head=False, with_value_head=True)
        shard = torch.zeros(size)
        run_plan_reference(entries, [full], shard)
        names = [s.name for s in tp_param_specs(cfg, r, tp, with_lm_head=False, with_value_head=True)]
        assert "value_head.weight" in names and "lm_head.weight" not in names
        for e in entries:
            dst = back.as_strided((e.rows, e.row_elems), (e.src_ld, 1), e.src_off)
            dst.copy_(shard.as_strided((e.rows, e.row_elems), (e.dst_ld, 1), e.dst_off))
    for s in specs:          # every parameter element was restored (alignment gaps between parameters stay untouched)
        assert torch.equal(back[s.offset:s.offset + s.numel], full[s.offset:s.offset + s.numel]), s.name
