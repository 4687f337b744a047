"""CPU tests of the host-side RL core: experience batching/balancing, loss aggregation invariances, advantage
estimators, partitioners, flag tree, sampler resume, KL controllers, length penalties."""
import math
from types import SimpleNamespace

import pytest
import torch

from openrlhf_b200.models.loss import (DPOLoss, LogExpLoss, PairWiseLoss, PolicyLoss, SFTLoss, ValueLoss,
                                       aggregate_loss)
from openrlhf_b200.models.utils import compute_approx_kl, compute_reward, log_probs_from_logits, masked_mean
from openrlhf_b200.rl.experience import (Experience, balance_experiences, make_experience_batch,
                                         remove_padding_in_sequences, split_experience_batch)
from openrlhf_b200.utils.config import hierarchize
from openrlhf_b200.utils.loss_utils import get_loss_batch_info, iter_grad_accum_global_norm
from openrlhf_b200.utils.seqlen_balancing import (get_minimum_num_micro_batch_size, get_seqlen_balanced_partitions,
                                                  karmarkar_karp)


def _exp(index, length):
    return Experience(sequences=torch.full((1, length), index, dtype=torch.long),
                      attention_mask=torch.ones((1, length), dtype=torch.long),
                      action_mask=torch.ones((1, length - 1), dtype=torch.bool),
                      total_length=torch.tensor([length]), prompts=[f"sample-{index}"])


@pytest.mark.parametrize("count", [4, 5, 9])
def test_balance_experiences_keeps_every_sample(count):
    args = SimpleNamespace(actor=SimpleNamespace(num_nodes=1, num_gpus_per_node=4),
                           ds=SimpleNamespace(ring_attn_size=1, tensor_parallel_size=1))
    outs = balance_experiences([_exp(i, count - i + 1) for i in range(count)], args)
    sizes = [len(b.sequences) for b in outs]
    assert len(outs) == 4 and all(s > 0 for s in sizes) and sum(sizes) == count
    assert sorted(p for b in outs for p in b.prompts) == sorted(f"sample-{i}" for i in range(count))
    tok = [int(b.total_length.sum()) for b in outs]
    assert max(tok) - min(tok) <= count + 1


def test_split_batch_roundtrip_and_padding_strip():
    a = Experience(sequences=torch.tensor([[1, 2, 3, 0], [4, 5, 6, 7]]), attention_mask=torch.tensor([[1, 1, 1, 0], [1, 1, 1, 1]]),
                   action_mask=torch.tensor([[0, 1, 0], [0, 1, 1]]).bool(), rewards=torch.tensor([1.0, 2.0]),
                   total_length=torch.tensor([3, 4]), prompts=["a", "b"], info={"x": torch.tensor([0.5, 0.7])})
    items = remove_padding_in_sequences(split_experience_batch(a))
    assert items[0].sequences.tolist() == [1, 2, 3] and items[0].action_mask.tolist() == [False, True]
    assert items[1].sequences.tolist() == [4, 5, 6, 7]
    b = make_experience_batch(items)
    assert b.sequences.tolist() == [[1, 2, 3, 0], [4, 5, 6, 7]] and b.rewards.tolist() == [1.0, 2.0]
    assert b.prompts == ["a", "b"]
    c = Experience.concat_experiences([a, a], pad_token_id=9)
    assert c.sequences.shape == (4, 4) and c.rewards.shape == (4,) and len(c.prompts) == 4


def test_aggregate_loss_is_invariant_to_dp_sharding():
    torch.manual_seed(0)
    loss = torch.randn(6, 9)
    mask = (torch.rand(6, 9) > 0.4).float()
    mask[2] = 0
    ntok = mask.sum()
    nseq = (mask.sum(-1) > 0).sum().float()
    for token_level in (True, False):
        whole = aggregate_loss(loss, mask, token_level, 1, ntok, nseq)
        parts = [aggregate_loss(loss[s], mask[s], token_level, 2, ntok, nseq) for s in (slice(0, 3), slice(3, 6))]
        assert torch.allclose(whole, sum(parts) / 2, atol=1e-6)
    # no normalisers: plain masked means; fully masked rows do not count in sample mode
    assert torch.allclose(aggregate_loss(loss, mask, True), (loss * mask).sum() / mask.sum())
    rows = [(loss[i] * mask[i]).sum() / mask[i].sum() for i in range(6) if mask[i].sum() > 0]
    assert torch.allclose(aggregate_loss(loss, mask, False), torch.stack(rows).mean(), atol=1e-6)


def test_policy_loss_metrics_and_variants():
    torch.manual_seed(1)
    lp = -torch.rand(4, 7); old = lp + 0.2 * torch.randn(4, 7); adv = torch.randn(4, 7)
    roll = old + 0.05 * torch.randn(4, 7)
    mask = (torch.rand(4, 7) > 0.2).float()
    ntok, nseq = mask.sum(), (mask.sum(-1) > 0).sum().float()
    pl = PolicyLoss(0.2, 0.3, enable_vllm_is_correction=True, vllm_is_truncated_threshold=[0.5, 2.0])
    loss, clip, kl, vkl = pl(lp, old, adv, mask, roll, batch_num_tokens=ntok, global_batch_size=nseq)
    ratio = (lp - old).clamp(-20, 20).exp()
    s1, s2 = ratio * adv, ratio.clamp(0.8, 1.3) * adv
    ref = (-(torch.min(s1, s2)) * (old - roll).exp().clamp(0.5, 2.0) * mask).sum() / ntok
    assert torch.allclose(loss, ref, atol=1e-6)
    assert torch.allclose(kl, masked_mean(-(lp - old), mask)) and torch.allclose(vkl, masked_mean(roll - old, mask))
    assert torch.allclose(clip, masked_mean((s2 < s1).float(), mask))
    # dp sharding equivalence
    halves = [pl(lp[s], old[s], adv[s], mask[s], roll[s], 2, ntok, nseq)[0] for s in (slice(0, 2), slice(2, 4))]
    assert torch.allclose(loss, sum(halves) / 2, atol=1e-6)
    # gspo is a sequence-level ratio with sample-level aggregation
    g = PolicyLoss(0.2, 0.2, policy_loss_type="gspo")
    gl, *_ = g(lp, old, adv, mask)
    seq_ratio = (((lp - old) * mask).sum(-1) / mask.sum(-1).clamp(min=1)).exp()[:, None] * mask
    t1, t2 = seq_ratio * adv, seq_ratio.clamp(0.8, 1.2) * adv
    assert torch.allclose(gl, aggregate_loss(-torch.min(t1, t2), mask, False), atol=1e-6)
    # seq-mask-tis drops whole sequences
    sm = PolicyLoss(0.2, 0.2, enable_vllm_is_correction=True, vllm_is_truncated_threshold=[0.99, 1.01],
                    vllm_is_correction_type="seq-mask-tis")
    assert sm(lp, old, adv, mask, old.clone())[0].abs() > 0
    with pytest.raises(ValueError):
        PolicyLoss(vllm_is_correction_type="nope")
    with pytest.raises(AssertionError):
        PolicyLoss(dual_clip=0.5)


def test_grad_accum_window_normalisation_equals_one_global_mean():
    torch.manual_seed(2)
    micro = [((torch.rand(2, n) > 0.3).float(), torch.randn(2, n)) for n in (3, 9, 5, 7)]
    got = 0.0
    for (mask, loss), info in iter_grad_accum_global_norm(iter(micro), object(), 4, lambda it: it[0]):
        got = got + aggregate_loss(loss, mask, True, info["dp_size"], info["batch_num_tokens"], info["global_batch_size"]) / 4
    want = sum((l * m).sum() for m, l in micro) / sum(m.sum() for m, _ in micro)
    assert torch.allclose(got, want, atol=1e-6)
    per_micro = sum((l * m).sum() / m.sum() for m, l in micro) / 4
    assert not torch.allclose(per_micro, want, atol=1e-4)
    info = get_loss_batch_info(object(), micro[0][0])
    assert info["dp_size"] == 1 and float(info["batch_num_tokens"]) == float(micro[0][0].sum())


def test_other_losses():
    c, r = torch.tensor([1.0, 0.2]), torch.tensor([0.5, 0.9])
    assert torch.allclose(PairWiseLoss()(c, r), -torch.nn.functional.logsigmoid(c - r).mean())
    assert torch.allclose(PairWiseLoss()(c, r, torch.tensor([0.1, 0.1])), -torch.nn.functional.logsigmoid(c - r - 0.1).mean())
    assert torch.allclose(LogExpLoss()(c, r), torch.log(1 + torch.exp(r - c)).mean())
    pc, pr, rc, rr = torch.tensor([-1.0]), torch.tensor([-2.0]), torch.tensor([-1.5]), torch.tensor([-1.8])
    loss, cw, rj = DPOLoss(0.1)(pc, pr, rc, rr)
    z = (pc - pr) - (rc - rr)
    assert torch.allclose(loss, -torch.nn.functional.logsigmoid(0.1 * z).mean()) and torch.allclose(cw, 0.1 * (pc - rc))
    assert torch.allclose(DPOLoss(0.1, ipo=True)(pc, pr, rc, rr)[0], ((z - 5.0) ** 2).mean())
    v, ov, ret, m = torch.randn(3, 5), torch.randn(3, 5), torch.randn(3, 5), torch.ones(3, 5)
    vc = ov + (v - ov).clamp(-0.2, 0.2)
    assert torch.allclose(ValueLoss(0.2)(v, ov, ret, m), 0.5 * torch.max((vc - ret) ** 2, (v - ret) ** 2).mean(), atol=1e-6)
    lp = -torch.rand(2, 4); lm = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 1.0]])
    assert torch.allclose(SFTLoss()(lp, lm), (-lp * lm).sum() / 6)


def test_model_utils():
    a, b = torch.tensor([[-1.0, -2.0]]), torch.tensor([[-1.5, -1.0]])
    d = a - b
    assert torch.allclose(compute_approx_kl(a, b, "k1"), d)
    assert torch.allclose(compute_approx_kl(a, b, "k2"), d * d / 2)
    assert torch.allclose(compute_approx_kl(a, b, "k3"), torch.exp(-d) - 1 + d)
    kl = torch.tensor([[0.1, 0.2, 0.3, 0.0]]); mask = torch.tensor([[1, 1, 1, 0]])
    rew = compute_reward(torch.tensor([20.0]), 0.5, kl, mask, (-10, 10))
    assert torch.allclose(rew, torch.tensor([[-0.05, -0.1, -0.15 + 10.0, 0.0]]))
    logits = torch.randn(3, 5, 11); y = torch.randint(0, 11, (3, 5))
    ref = torch.log_softmax(logits / 0.7, -1).gather(-1, y[..., None]).squeeze(-1)
    assert torch.allclose(log_probs_from_logits(logits, y, 0.7), ref, atol=1e-5)


def test_advantage_estimators_match_naive():
    from openrlhf_b200.rl.advantages import compute_advantages_and_returns
    torch.manual_seed(3)
    n, P, A = 4, 3, 6
    def make(est):
        exps = []
        idx = list(range(P * n))
        for b in range(0, P * n, 6):
            ii = idx[b:b + 6]
            mask = torch.ones(len(ii), A); mask[:, -1] = 0
            exps.append(Experience(sequences=torch.zeros(len(ii), A + 1, dtype=torch.long), action_mask=mask.bool(),
                                   rewards=torch.tensor([float((i * 7) % 5) for i in ii]), kl=0.1 * torch.ones(len(ii), A),
                                   values=torch.randn(len(ii), A) if est == "gae" else None,
                                   response_length=torch.full((len(ii),), 5.0), index=ii, info={}))
        return exps
    for est in ("group_norm", "rloo", "reinforce_baseline", "dr_grpo", "reinforce", "gae"):
        args = SimpleNamespace(algo=SimpleNamespace(advantage=SimpleNamespace(estimator=est, gamma=1.0, lambd=0.95, no_std_norm=False)),
                               rollout=SimpleNamespace(n_samples_per_prompt=n, max_new_tokens=8),
                               reward=SimpleNamespace(clip_range=(-10, 10), overlong_buffer_len=None, stop_properly_penalty_coef=None),
                               data=SimpleNamespace(max_len=16))
        exps = make(est)
        raw = torch.cat([e.rewards for e in exps]).reshape(P, n)
        vals = [e.values.clone() if e.values is not None else None for e in exps]
        compute_advantages_and_returns(exps, args, kl_value=0.2)
        if est == "group_norm":
            shaped = (raw - raw.mean(-1, keepdim=True)) / (raw.std(-1, keepdim=True) + 1e-9)
        elif est == "rloo":
            shaped = raw - (raw.sum(-1, keepdim=True) - raw) / (n - 1)
        elif est in ("reinforce_baseline", "dr_grpo"):
            shaped = raw - raw.mean(-1, keepdim=True)
        else:
            shaped = raw
        shaped = shaped.reshape(-1)
        adv_all = torch.cat([e.advantages for e in exps]); mask_all = torch.cat([e.action_mask.float() for e in exps])
        # naive recomputation
        rows = []
        k = 0
        for e, v in zip(exps, vals):
            for j in range(len(e.index)):
                r = torch.full((A,), -0.2 * 0.1); r[A - 2] += shaped[e.index[j]]; r[A - 1] = 0
                if est == "gae":
                    vv = v[j] * e.action_mask[j].float(); out = torch.zeros(A); last = 0.0
                    for t in reversed(range(A)):
                        nv = vv[t + 1] if t < A - 1 else 0.0
                        last = r[t] + nv - vv[t] + 0.95 * last; out[t] = last
                else:
                    out = torch.flip(torch.cumsum(torch.flip(r, [0]), 0), [0])
                rows.append(out)
        naive = torch.stack(rows)
        if est in ("gae", "reinforce", "reinforce_baseline"):
            mean = (naive * mask_all).sum() / mask_all.sum()
            var = (((naive - mean) ** 2) * mask_all).sum() / mask_all.sum()
            naive = (naive - mean) * var.clamp(min=1e-8).rsqrt()
        assert torch.allclose(adv_all * mask_all, naive * mask_all, atol=1e-4), est
        assert "return" in exps[0].info and exps[0].kl is None
        if n > 1:
            assert "group_reward_std" in exps[0].info


def test_partitioners():
    import random
    random.seed(0)
    for _ in range(20):
        lens = [random.randint(1, 4000) for _ in range(random.randint(8, 40))]
        k = random.randint(2, 8)
        parts = get_seqlen_balanced_partitions(lens, k, equal_size=False)
        assert sorted(i for p in parts for i in p) == list(range(len(lens))) and all(parts)
        sums = [sum(lens[i] for i in p) for p in parts]
        assert max(sums) - min(sums) <= max(lens)
    lens = list(range(1, 17))
    parts = karmarkar_karp(lens, 4, equal_size=True)
    assert all(len(p) == 4 for p in parts)
    assert get_minimum_num_micro_batch_size([5, 5, 5, 5], 10, 1, 1) == 2
    assert get_minimum_num_micro_batch_size([5, 5, 5, 5], 5, 2, 2) == 1
    with pytest.raises(AssertionError):
        get_seqlen_balanced_partitions([1, 2], 3, False)


def test_hierarchize_and_sampler_and_controllers():
    import argparse
    from openrlhf_b200.rl.kl_controller import AdaptiveKLController, FixedKLController
    from openrlhf_b200.rl.length_penalty import apply_overlong_penalty, apply_stop_properly_penalty
    from openrlhf_b200.utils.distributed_sampler import DistributedSampler
    ns = argparse.Namespace(**{"actor.adam.lr": 1e-6, "actor.eps_clip": 0.2, "seed": 1, "ds.lora.rank": 0})
    h = hierarchize(ns)
    assert h.actor.adam.lr == 1e-6 and h.actor.eps_clip == 0.2 and h.seed == 1 and h.ds.lora.rank == 0
    s = DistributedSampler(list(range(10)), num_replicas=2, rank=1, shuffle=False)
    assert list(s) == [1, 3, 5, 7, 9]
    s.set_epoch(0, consumed_samples=4)
    assert list(s) == [5, 7, 9] and len(s) == 3
    a = DistributedSampler(list(range(7)), num_replicas=2, rank=0, shuffle=True, seed=3)
    b = DistributedSampler(list(range(7)), num_replicas=2, rank=1, shuffle=True, seed=3)
    assert len(list(a)) == len(list(b)) == 4
    c = AdaptiveKLController(0.1, target=1.0, horizon=100)
    c.update(2.0, 10)
    assert math.isclose(c.value, 0.1 * (1 + 0.2 * 10 / 100))
    f = FixedKLController(0.3); f.update(5, 5); assert f.value == 0.3
    e = Experience(rewards=torch.tensor([1.0, 1.0, 1.0]), response_length=torch.tensor([10.0, 95.0, 120.0]),
                   truncated=torch.tensor([False, False, True]), info={})
    assert apply_overlong_penalty([e], 100, 20, 1.0) == 2
    assert torch.allclose(e.rewards, torch.tensor([1.0, 1 - 15 / 20, 0.0]))
    assert apply_stop_properly_penalty([e], -0.5) == 1 and e.rewards[2] == -0.5
