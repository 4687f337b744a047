"""CPU fp32 oracle and timed CPU baseline: one GRPO step of a tiny Llama-architecture policy (2 layers, hidden 64,
4 heads, 2 KV heads, FFN 176, vocab 1024) exactly as the first benchmark config describes it: 8 prompts x 64 tokens
(ids uniform in [3, 1024), seed 0), n = 4 sampled responses of exactly 64 tokens at temperature 1, reward = fraction of
even token ids, group-normalised advantages, clipped PPO loss (eps 0.2) on packed samples, k3 KL to the reference
policy at beta 0.01, one Adam step at lr 1e-5. Everything is plain PyTorch on CPU (the PyTorch restatements of the
operators), which is what the GPU kernels are compared against.

    python baseline/cpu_oracle.py            # prints a JSON line with the metrics and the step time
"""
from __future__ import annotations

import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from openrlhf_b200.models.config import PRESETS  # noqa: E402
from openrlhf_b200.models.packing import pack_lists  # noqa: E402
from openrlhf_b200.models.transformer import TransformerLM  # noqa: E402
from openrlhf_b200.ops import rl as K  # noqa: E402
from openrlhf_b200.rl.advantages import group_baseline  # noqa: E402


@torch.no_grad()
def sample(model, prompts: torch.Tensor, n: int, new_tokens: int, gen: torch.Generator) -> torch.Tensor:
    """Ancestral sampling at temperature 1 by full recomputation (no KV cache: this is the oracle, not the engine)."""
    seqs = prompts.repeat_interleave(n, dim=0)
    for _ in range(new_tokens):
        pb = pack_lists(list(seqs), "cpu")
        h, _ = model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        last = (pb.cu_seqlens[1:] - 1).long()
        probs = torch.softmax(model.logits(h[last]).float(), -1)
        nxt = torch.multinomial(probs, 1, generator=gen)
        seqs = torch.cat([seqs, nxt], dim=1)
    return seqs


def grpo_step(seed: int = 0, n_prompts: int = 8, prompt_len: int = 64, n: int = 4, new_tokens: int = 64):
    cfg = PRESETS["tiny-llama"]
    torch.manual_seed(seed)
    policy = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=seed)
    ref = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=None)
    ref.flat.copy_(policy.flat)
    ref.requires_grad_(False)
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(3, cfg.vocab_size, (n_prompts, prompt_len), generator=g)
    t0 = time.perf_counter()
    seqs = sample(policy, prompts, n, new_tokens, g)
    t_gen = time.perf_counter() - t0
    resp = seqs[:, prompt_len:]
    rewards = (resp % 2 == 0).float().mean(-1)
    adv_seq, _ = group_baseline(rewards, n, "group_norm")
    pb = pack_lists(list(seqs), "cpu")
    T = seqs.shape[1]
    mask = torch.zeros(seqs.shape[0], T - 1)
    mask[:, prompt_len - 1:] = 1

    def logps(model):
        h, _ = model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        lp, _ = model.logprobs(h, pb.labels)
        return lp.view(seqs.shape[0], T)[:, :-1]

    with torch.no_grad():
        old = logps(policy)
        base = logps(ref)
    new = logps(policy)
    adv = adv_seq[:, None].expand_as(mask) * mask
    out = K.ppo_loss(new, old, adv, mask, ref_logp=base, eps_low=0.2, eps_high=0.2, kl_coef=0.01, kl_estimator="k3")
    out["loss"].backward()
    opt = torch.optim.Adam(policy.parameters(), lr=1e-5)
    opt.step()
    t_total = time.perf_counter() - t0
    gnorm = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in policy.parameters() if p.grad is not None))
    return {"loss": float(out["loss"]), "policy_loss": float(out["policy_loss"]), "kl_loss": float(out["kl_loss"]),
            "reward_mean": float(rewards.mean()), "grad_norm": float(gnorm), "samples": int(seqs.shape[0]),
            "generation_s": t_gen, "step_s": t_total, "samples_per_s": seqs.shape[0] / t_total,
            "checksum": float(policy.flat.double().sum())}


if __name__ == "__main__":
    print(json.dumps(grpo_step()))
