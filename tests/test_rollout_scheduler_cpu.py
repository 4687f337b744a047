"""Rollout-engine scheduler on CPU tensors (the PyTorch restatements of the kernels): waves and preemption when the KV
demand exceeds the page pool, chunked prefill, the prefix cache for multi-turn requests, per-request nucleus settings."""
import pytest
import torch

from openrlhf_b200.models.config import ModelConfig
from openrlhf_b200.models.transformer import TransformerLM
from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams


@pytest.fixture(autouse=True)
def _invariant_checks(monkeypatch):
    """Every engine step of these tests re-checks the page / slot bookkeeping against the device state."""
    import openrlhf_b200.rollout.engine as E

    monkeypatch.setattr(E, "_DEBUG", True)


@pytest.fixture(scope="module")
def model():
    return TransformerLM(ModelConfig.from_pretrained("tiny-qwen2"), device="cpu", dtype=torch.float32, seed=0)


@pytest.fixture(scope="module")
def prompts():
    g = torch.Generator().manual_seed(0)
    return [torch.randint(3, 2000, (n,), generator=g).tolist() for n in (5, 300, 17, 140, 260, 33)]


def _same(a, b, n=1):
    for x, y in zip(a, b):
        for j in range(n):
            assert x.outputs[j].token_ids == y.outputs[j].token_ids, (len(x.prompt_token_ids), j)
            la, lb = torch.tensor(x.outputs[j].logprob_values), torch.tensor(y.outputs[j].logprob_values)
            assert (la - lb).abs().max() < 1e-3


def test_kv_demand_three_times_the_pool_gives_identical_greedy_outputs(model, prompts):
    sp = SamplingParams(temperature=0.0, max_tokens=150, n=2, ignore_eos=True)
    big = RolloutEngine(model, max_num_seqs=16, max_model_len=512, num_pages=80)
    ref = big.generate(prompts, sp)
    assert big.stats["preemptions"] == 0 and big.stats["prefill_chunks"] == 1
    # all contexts together need about 40 pages; 13 usable pages force waves, preemption with recomputation, and
    # (with a 128-token prefill budget) chunked prefill of the longer prompts and of the preempted samples
    small = RolloutEngine(model, max_num_seqs=16, max_model_len=512, num_pages=14, max_prefill_tokens=128)
    out = small.generate(prompts, sp)
    assert small.stats["preemptions"] >= 1 and small.stats["prefill_chunks"] > 6
    _same(ref, out, 2)
    assert small.blocks.num_free() == 14 - 1            # every page came back (one backs inactive rows)
    assert not small.has_unfinished()


def test_single_sequence_too_long_for_the_pool_raises(model):
    eng = RolloutEngine(model, max_num_seqs=4, max_model_len=512, num_pages=3)
    with pytest.raises(RuntimeError):
        eng.generate([list(range(3, 403))], SamplingParams(temperature=0.0, max_tokens=8))


def test_prefix_cache_serves_the_second_turn_of_a_conversation(model, prompts):
    plain = RolloutEngine(model, max_num_seqs=16, max_model_len=512, num_pages=80)
    pc = RolloutEngine(model, max_num_seqs=16, max_model_len=512, num_pages=80, enable_prefix_caching=True)
    sp1 = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    o1 = pc.generate(prompts, sp1)
    _same(plain.generate(prompts, sp1), o1)
    # multi-turn agents re-send the growing conversation: prompt + response + the next user turn
    turn2 = [list(o.prompt_token_ids) + o.outputs[0].token_ids + [7, 8, 9] for o in o1]
    before = pc.stats["prefill_tokens"]
    sp2 = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    o2 = pc.generate(turn2, sp2)
    computed = pc.stats["prefill_tokens"] - before
    total = sum(len(t) for t in turn2)
    whole_pages = sum((len(t) - 4) // 128 * 128 for t in turn2)       # pages of turn 1 that were complete
    assert computed == total - whole_pages and pc.stats["prefix_hit_tokens"] >= whole_pages
    _same(plain.generate(turn2, sp2), o2)
    # a weight update invalidates the cache and returns its pages
    pc.update_weights(model.flat)
    assert pc.blocks.num_free() == 80 - 1 and not pc._cache
    _same(plain.generate(turn2, sp2), pc.generate(turn2, sp2))


def test_nucleus_settings_are_per_request(model, prompts):
    eng = RolloutEngine(model, max_num_seqs=8, max_model_len=256, num_pages=24)
    sps = [SamplingParams(temperature=1.0, top_k=1, max_tokens=6, ignore_eos=True),      # top-1 == greedy
           SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True),
           SamplingParams(temperature=1.0, top_p=1e-6, max_tokens=6, ignore_eos=True)]   # nucleus of one token
    out = eng.generate([prompts[0]] * 3, sps)
    assert out[0].outputs[0].token_ids == out[1].outputs[0].token_ids == out[2].outputs[0].token_ids


def test_fixed_length_rows_decode_in_long_bursts_with_identical_outputs(model, prompts):
    """Rows that ignore EOS can only finish at their token limit, so the engine runs them in bursts of up to eight
    check intervals once nothing waits for admission or prefill; rows that may stop on EOS start with short bursts
    that grow while no row finishes. Same tokens and log-probs either way, far fewer host round trips."""
    sp_fixed = SamplingParams(temperature=0.0, max_tokens=90, n=1, ignore_eos=True)
    sp_eos = SamplingParams(temperature=0.0, max_tokens=90, n=1, ignore_eos=False)
    calls = {}
    outs = {}
    for name, sp in (("fixed", sp_fixed), ("eos", sp_eos)):
        eng = RolloutEngine(model, max_num_seqs=8, max_model_len=512, num_pages=40, check_interval=4,
                            eos_token_id=-1)            # no token is ever the EOS: both runs generate 90 tokens
        for i, p in enumerate(prompts[:4]):
            eng.add_request(i, p, sp)
        n, done = 0, []
        while eng.has_unfinished():
            done += eng.step()
            n += 1
        calls[name] = n
        outs[name] = sorted(done, key=lambda o: o.request_id)
        assert eng.decode_steps >= 90 - 1
    _same(outs["fixed"], outs["eos"])
    # 90 tokens: rows that may stop on EOS start with bursts of 4 steps and grow to 8 and 16 while nobody finishes
    # (4 + 4 + 8 + 8 + 16 ...: about nine calls); rows that cannot stop early run 32 steps at a time from the start
    assert 7 <= calls["eos"] <= 12 and calls["fixed"] <= 6 and calls["fixed"] < calls["eos"], calls
