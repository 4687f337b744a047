"""Multi-GPU tests: run the scripts of tests/dist_scripts under torchrun when at least two GPUs are visible."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(script, nproc=2, env=None, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "dist_scripts", script)]
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_symm_optimizer_step_matches_nccl():
    out = _run("zero_symm_vs_nccl.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "zero_symm_vs_nccl ok" in out


def test_fused_tp_gemms():
    out = _run("tp_gemm.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "tp_gemm ok" in out


def test_context_parallel_attention():
    out = _run("cp_attention.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "CP_ATTENTION_OK" in out


def test_context_parallel_model():
    out = _run("cp_model.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "CP_MODEL_OK" in out


def test_expert_parallel_moe():
    out = _run("ep_moe.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "EP_MOE_OK" in out


def test_expert_parallel_model():
    out = _run("ep_model.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "EP_MODEL_OK" in out


def test_vocab_parallel_logprob():
    out = _run("vocab_parallel.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "VOCAB_PARALLEL_OK" in out


def test_zero3_matches_zero2():
    out = _run("zero3_vs_zero2.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "ZERO3_OK" in out


def test_tensor_parallel_rollout_engine():
    out = _run("tp_rollout.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "TP_ROLLOUT_OK" in out


def test_hybrid_worker_zero3_and_tp_rollout():
    out = _run("hybrid_modes.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "HYBRID_MODES_OK" in out


def test_tensor_parallel_training():
    out = _run("tp_train.py", env={"NCCL_NVLS_ENABLE": "0"})
    assert "TP_TRAIN_OK" in out


def test_rl_launcher_with_tensor_parallel_training(tmp_path):
    r = subprocess.run(["bash", os.path.join(HERE, "dist_scripts", "cli_ppo_tp.sh"), str(tmp_path / "out")],
                       capture_output=True, text=True, timeout=900, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0 and "CLI_PPO_TP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    assert "global step 1" in r.stdout
