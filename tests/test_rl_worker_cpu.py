"""The RL launcher's worker on CPU: gradient accumulation must not change the optimizer step, and the whitening
statistics of the SPMD worker are global over ranks."""
import copy
from types import SimpleNamespace

import torch

from dist_helpers import run_gloo_ranks


def _args(extra=()):
    from openrlhf_b200.cli import flags as F
    from openrlhf_b200.cli.train_ppo_ray import build_parser, validate

    argv = ["--actor.model_name_or_path", "tiny-llama", "--reward.remote_url", "none", "--algo.advantage.estimator",
            "reinforce", "--algo.kl.init_coef", "0", "--ds.packing_samples", "--actor.adam.lr", "1e-3",
            "--actor.num_gpus_per_node", "1", "--data.max_len", "64", "--rollout.batch_size", "8",
            "--actor.lr_scheduler", "constant", *extra]
    return validate(F.finalize(build_parser(), argv))


def _experiences(n, seed=0):
    from openrlhf_b200.rl.experience import Experience

    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        T = 6 + 5 * (i % 4)                       # uneven lengths: micro-batches carry different token counts
        P = 3
        seq = torch.randint(3, 1000, (1, T), generator=g)
        am = torch.zeros(1, T - 1, dtype=torch.bool)
        am[0, P - 1:] = True
        out.append(Experience(sequences=seq, attention_mask=torch.ones(1, T, dtype=torch.long), action_mask=am,
                              action_log_probs=-torch.rand(1, T - 1, generator=g) * 3,
                              advantages=torch.randn(1, T - 1, generator=g),
                              rollout_log_probs=torch.zeros(1, T - 1),
                              response_length=torch.tensor([T - P]), total_length=torch.tensor([float(T)]),
                              truncated=torch.tensor([False]), info={}))
    return out


def _fit(micro, batch):
    from openrlhf_b200.runtime.workers import RLWorker

    a = _args(["--train.micro_batch_size", str(micro), "--train.batch_size", str(batch)])
    w = RLWorker(a, roles=("actor",), max_steps=10, backend="gloo")
    assert w.strategy.accumulated_gradient == batch // micro
    for e in _experiences(8):
        w.append(copy.deepcopy(e), role="actor")
    st = w.fit(role="actor")
    return st, w.actor.model.flat[: w.actor.model.total_numel].float().clone()


def test_gradient_accumulation_matches_one_big_batch():
    st1, flat1 = _fit(micro=8, batch=8)          # one micro-batch per optimizer step
    st4, flat4 = _fit(micro=2, batch=8)          # four uneven micro-batches accumulated
    assert abs(st1["actor_grad_norm"] - st4["actor_grad_norm"]) <= 1e-4 * max(1.0, st1["actor_grad_norm"]), (st1, st4)
    # bf16 parameters and Adam's first step (lr * sign of the gradient): elements whose gradient is at rounding level
    # may move the other way, everything else must move identically
    differs = ((flat1 - flat4).abs() > 1e-4).float().mean().item()
    assert differs < 0.02, differs


def _whiten_rank(rank, world):
    from openrlhf_b200.rl.advantages import compute_advantages_and_returns
    from openrlhf_b200.rl.experience import Experience

    g = torch.Generator().manual_seed(100 + rank)
    A = 7
    exps = []
    for i in range(2):
        am = torch.ones(2, A, dtype=torch.bool)
        exps.append(Experience(sequences=torch.zeros(2, A + 1, dtype=torch.long), action_mask=am,
                               attention_mask=torch.ones(2, A + 1, dtype=torch.long), kl=torch.zeros(2, A),
                               rewards=torch.randn(2, generator=g) * (1 + 3 * rank) + rank,
                               response_length=torch.full((2,), A), total_length=torch.full((2,), A + 1.0),
                               index=[2 * i, 2 * i + 1], info={}))
    args = SimpleNamespace(algo=SimpleNamespace(advantage=SimpleNamespace(estimator="reinforce", gamma=1.0, lambd=1.0,
                                                                           no_std_norm=False)),
                           rollout=SimpleNamespace(n_samples_per_prompt=1),
                           reward=SimpleNamespace(clip_range=(-10.0, 10.0), overlong_buffer_len=None,
                                                  stop_properly_penalty_coef=None))
    raw = torch.cat([e.rewards for e in exps])
    compute_advantages_and_returns(exps, args, 0.0, dist_group=None, distributed=True)
    adv = torch.cat([e.advantages[:, -1] for e in exps])
    # with estimator "reinforce", gamma 1 and no KL every action token of a sample carries the sample's reward, so the
    # whitened advantage is (reward - mean) / std with the statistics of ALL ranks' tokens
    return raw, adv


def test_whitening_statistics_are_global_over_ranks():
    res = run_gloo_ranks(_whiten_rank, 2)
    raw = torch.cat([r[0] for r in res])
    adv = torch.cat([r[1] for r in res])
    mean, var = raw.mean(), raw.var(unbiased=False)
    expect = (raw - mean) * torch.rsqrt(var.clamp_min(1e-8))
    assert torch.allclose(adv, expect, atol=1e-4), (adv, expect)
