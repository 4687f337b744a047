"""Model-level GPU tests: CUDA forward/backward against the CPU fp32 restatement, rollout-vs-trainer parity."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny():
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.transformer import TransformerLM
    cfg = PRESETS["tiny-qwen2"]
    m = TransformerLM(cfg, device="cuda", seed=3)
    return cfg, m


def test_forward_backward_matches_cpu_reference():
    from openrlhf_b200.models.packing import pack_lists
    from openrlhf_b200.models.transformer import TransformerLM
    cfg, m = _tiny()
    ref = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=None)
    ref.flat.copy_(m.flat.float().cpu())
    torch.manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab_size, (n,)) for n in (37, 150, 64)]
    pb = pack_lists(seqs, "cuda")
    h, _ = m(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
    logp, ent = m.logprobs(h, pb.labels, 0.9, True)
    w = torch.randn_like(logp)
    (logp * w).sum().backward()
    pc = pack_lists(seqs, "cpu")
    hr, _ = ref(pc.input_ids, pc.position_ids, pc.cu_seqlens, pc.max_seqlen)
    lr, er = ref.logprobs(hr, pc.labels, 0.9, True)
    (lr * w.cpu()).sum().backward()
    assert (logp.cpu() - lr).abs().max() < 0.08, (logp.cpu() - lr).abs().max()
    assert (ent.cpu() - er).abs().max() < 0.08
    for name in ("layers.0.qkv.weight", "layers.1.down.weight", "embed.weight", "norm.weight"):
        g, gr = m.p(name).grad.float().cpu(), ref.p(name).grad
        denom = gr.abs().max().item() + 1e-6
        assert (g - gr).abs().max().item() / denom < 0.08, (name, (g - gr).abs().max().item(), denom)


def test_rollout_matches_trainer_logprobs_and_greedy():
    from openrlhf_b200.models.packing import pack_lists
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    cfg, m = _tiny()
    eng = RolloutEngine(m, max_num_seqs=8, max_model_len=512, num_pages=64, seed=1)
    torch.manual_seed(1)
    prompts = [torch.randint(3, cfg.vocab_size, (n,)).tolist() for n in (5, 130, 77)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=140, n=1, logprobs=1, ignore_eos=True))
    _lib.check_status()
    for p, o in zip(prompts, outs):
        toks = o.outputs[0].token_ids
        assert len(toks) == 140
        seq = torch.tensor(p + toks)
        pb = pack_lists([seq], "cuda")
        with torch.no_grad():
            h, _ = m(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
            logits = m.logits(h).float()
        pred = logits[len(p) - 1:-1]
        lp = torch.log_softmax(pred, -1)
        chosen = lp.gather(-1, torch.tensor(toks, device="cuda")[:, None]).squeeze(-1)
        # greedy tokens are (near-)argmax of the trainer's logits and log-probs agree
        assert (lp.max(-1).values - chosen).max() < 0.05
        assert (chosen.cpu() - torch.tensor(o.outputs[0].logprob_values)).abs().max() < 0.05
    # sampled generation with n > 1 shares the prompt pages and yields distinct continuations
    outs = eng.generate([prompts[1]], SamplingParams(temperature=1.0, max_tokens=20, n=4, logprobs=1, ignore_eos=True))
    conts = {tuple(c.token_ids) for c in outs[0].outputs}
    assert len(conts) > 1 and all(len(c.token_ids) == 20 for c in outs[0].outputs)
    assert eng.blocks.num_free() == eng.num_pages - 1


def test_rl_step_smoke():
    import __graft_entry__ as ge
    ge.smoke()


def test_engine_sleep_wake_keeps_graphs_and_results():
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    cfg, m = _tiny()
    eng = RolloutEngine(m, max_num_seqs=4, max_model_len=256, num_pages=16, seed=1)
    p = [torch.randint(3, cfg.vocab_size, (9,)).tolist()]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    a = eng.generate(p, sp)[0].outputs[0].token_ids
    free0 = torch.cuda.mem_get_info()[0]
    n_graphs = len(eng.graphs)
    eng.sleep()
    assert eng.arena is None or torch.cuda.mem_get_info()[0] > free0
    eng.wake_up()
    b = eng.generate(p, sp)[0].outputs[0].token_ids
    assert a == b and (eng.arena is None or len(eng.graphs) == n_graphs)
