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


def test_moe_model_trains_and_rolls_out():
    """Qwen3-MoE family on the GPU: grouped expert GEMMs in training (finite loss / gradients for router and
    experts), the generic decode path (qk-norm + MoE) in the rollout engine, and trainer / rollout log-prob agreement
    for most tokens (a routing flip between the two batch shapes may move an individual token)."""
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.packing import pack_lists
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    cfg = PRESETS["tiny-qwen3-moe"]
    m = TransformerLM(cfg, device="cuda", seed=5, init_std=0.05)
    torch.manual_seed(0)
    seqs = [torch.randint(3, cfg.vocab_size, (n,)) for n in (90, 300)]
    pb = pack_lists(seqs, "cuda")
    h, aux = m(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
    logp, _ = m.logprobs(h, pb.labels)
    (-logp.mean() + 0.01 * aux).backward()
    _lib.check_status()
    assert torch.isfinite(logp).all() and float(aux) > 0
    for name in ("layers.0.router.weight", "layers.1.experts.gate_up", "layers.0.experts.down", "layers.0.qkv.weight"):
        g = m.p(name).grad
        assert g is not None and torch.isfinite(g).all() and g.float().abs().sum() > 0, name
    eng = RolloutEngine(m, max_num_seqs=4, max_model_len=256, num_pages=16, seed=1)
    prompt = torch.randint(3, cfg.vocab_size, (40,)).tolist()
    out = eng.generate([prompt], SamplingParams(temperature=1.0, max_tokens=48, n=2, logprobs=1, ignore_eos=True))
    _lib.check_status()
    diffs = []
    for c in out[0].outputs:
        seq = torch.tensor(prompt + c.token_ids)
        p1 = pack_lists([seq], "cuda")
        with torch.no_grad():
            hh, _ = m(p1.input_ids, p1.position_ids, p1.cu_seqlens, p1.max_seqlen)
            lp, _ = m.logprobs(hh, p1.labels)
        diffs.append((lp[len(prompt) - 1:-1].cpu() - torch.tensor(c.logprob_values)).abs())
    d = torch.cat(diffs)
    assert d.median() < 0.02 and (d < 0.1).float().mean() > 0.9, (d.median(), (d < 0.1).float().mean())


def test_rl_step_with_critic_and_kl():
    """Full PPO flavour of the hybrid worker on a tiny model: actor, reference, critic and a reward model (scalar head
    on the last token), GAE and a KL penalty."""
    from openrlhf_b200.trainer.hybrid_engine import HybridRLWorker, default_rl_args
    args = default_rl_args(**{"rollout.n_samples_per_prompt": 2, "rollout.max_new_tokens": 8, "train.micro_batch_size": 2,
                              "train.batch_size": 4, "data.max_len": 64, "algo.advantage.estimator": "gae",
                              "algo.kl.init_coef": 0.05})
    args.rollout.ignore_eos = True
    from openrlhf_b200.models.model import get_llm_for_sequence_regression
    rm = get_llm_for_sequence_regression("tiny-qwen2", "reward", device="cuda", seed=7, init_value_head=True)
    w = HybridRLWorker("tiny-qwen2", args, device="cuda", reward_model=rm, max_num_seqs=8, num_pages=32)
    prompts = [torch.randint(3, w.cfg.vocab_size, (12,)).tolist() for _ in range(2)]
    st = w.rl_step(prompts)
    assert "critic_loss" in st and st["num_samples"] == 4
    for k in ("policy_loss", "critic_loss", "actor_grad_norm", "critic_grad_norm"):
        assert torch.isfinite(torch.tensor(float(st[k]))), (k, st[k])


def test_vlm_trains_and_rolls_out():
    """Qwen2-VL family on the GPU: the vision tower and the language model train through the same GEMM kernels
    (gradients reach the tower), the fused RoPE + attention kernels take the per-token multimodal rotary rows, and the
    rollout engine's prefill with images plus its offset decode positions reproduce the trainer's log-probs."""
    import dataclasses

    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    cfg = dataclasses.replace(PRESETS["tiny-qwen2-vl"])
    m = TransformerLM(cfg, device="cuda", seed=7, init_std=0.05)
    torch.manual_seed(0)
    IMG, VS, VE = cfg.image_token_id, cfg.vision_start_token_id, cfg.vision_end_token_id

    def doc(grids, n_text):
        ids = torch.randint(3, 2000, (n_text,)).tolist()
        for t, h, w in grids:
            ids += [VS] + [IMG] * (t * h * w // 4) + [VE] + torch.randint(3, 2000, (5,)).tolist()
        npatch = sum(t * h * w for t, h, w in grids)
        return ids, torch.randn(npatch, 1176).bfloat16(), torch.tensor(grids)

    d0, d1 = doc([(1, 4, 4), (1, 4, 8)], 20), doc([(1, 8, 8)], 7)
    ids = torch.tensor(d0[0] + d1[0], device="cuda")
    cu_list = [0, len(d0[0]), len(d0[0]) + len(d1[0])]
    pv, thw = torch.cat([d0[1], d1[1]]).cuda(), torch.cat([d0[2], d1[2]])
    emb, pos = m.multimodal_inputs(ids, cu_list, pv, thw)
    cu = torch.tensor(cu_list, dtype=torch.int32, device="cuda")
    h, _ = m(ids, pos, cu, max(len(d0[0]), len(d1[0])), inputs_embeds=emb)
    logp, _ = m.logprobs(h, torch.roll(ids, -1))
    (-logp.mean()).backward()
    _lib.check_status()
    assert torch.isfinite(logp).all()
    for name in ("visual.patch_embed.weight", "visual.blocks.1.mlp.fc1.weight", "visual.merger.mlp.2.weight",
                 "layers.0.qkv.weight"):
        g = m.p(name).grad
        assert g is not None and torch.isfinite(g).all() and g.float().abs().sum() > 0, name
    # fp32 PyTorch restatement of the same forward on the CPU
    mc = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=None)
    mc.flat.copy_(m.flat.float().cpu())
    with torch.no_grad():
        e2, p2 = mc.multimodal_inputs(ids.cpu(), cu_list, pv.float().cpu(), thw)
        h2, _ = mc(ids.cpu(), p2, cu.cpu(), max(len(d0[0]), len(d1[0])), inputs_embeds=e2)
        ref, _ = mc.logprobs(h2, torch.roll(ids.cpu(), -1))
    assert (logp.detach().float().cpu() - ref).abs().max() < 0.15

    # rollout: prompt with one image, greedy; the trainer's log-probs of the generated tokens must agree
    eng = RolloutEngine(m, max_num_seqs=4, max_model_len=512, num_pages=16, seed=1)
    prompt, ppv, pthw = d1
    out = eng.generate([prompt, d0[0][:20]], SamplingParams(temperature=0.0, max_tokens=24, logprobs=1, ignore_eos=True),
                       multi_modal_data=[{"pixel_values": ppv, "image_grid_thw": pthw}, None])
    _lib.check_status()
    toks = out[0].outputs[0].token_ids
    seq = torch.tensor(prompt + toks, device="cuda")
    with torch.no_grad():
        e, p = m.multimodal_inputs(seq, [0, seq.numel()], ppv.cuda(), pthw)
        hh, _ = m(seq, p, torch.tensor([0, seq.numel()], dtype=torch.int32, device="cuda"), seq.numel(), inputs_embeds=e)
        lp, _ = m.logprobs(hh, torch.roll(seq, -1))
    got = torch.tensor(out[0].outputs[0].logprob_values)
    assert (lp[len(prompt) - 1:-1].cpu() - got).abs().max() < 0.05
    # the text-only request in the same batch decodes with plain positions
    t2 = out[1].outputs[0].token_ids
    s2 = torch.tensor(d0[0][:20] + t2, device="cuda")
    from openrlhf_b200.models.packing import pack_lists
    pb = pack_lists([s2], "cuda")
    with torch.no_grad():
        h3, _ = m(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        lp3, _ = m.logprobs(h3, pb.labels)
    assert (lp3[19:-1].cpu() - torch.tensor(out[1].outputs[0].logprob_values)).abs().max() < 0.05


def test_rollout_fp8_decode_tracks_bf16_trainer():
    """fp8 (per-tensor e4m3) projection weights in the decode loop: samples stay close to the bf16 trainer's
    distribution (log-prob gap of the sampled tokens well below the gap between unrelated tokens)."""
    from openrlhf_b200.models.packing import pack_lists
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    cfg, m = _tiny()
    eng = RolloutEngine(m, max_num_seqs=8, max_model_len=512, num_pages=32, seed=1, quantization="fp8")
    torch.manual_seed(2)
    prompts = [torch.randint(3, cfg.vocab_size, (n,)).tolist() for n in (40, 130)]
    outs = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=64, n=1, logprobs=1, ignore_eos=True))
    _lib.check_status()
    assert len(eng.fp8) == 4 * cfg.num_hidden_layers
    gaps = []
    for p, o in zip(prompts, outs):
        toks = o.outputs[0].token_ids
        seq = torch.tensor(p + toks)
        pb = pack_lists([seq], "cuda")
        with torch.no_grad():
            h, _ = m(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
            lp, _ = m.logprobs(h, pb.labels)
        gaps.append((lp[len(p) - 1:-1].cpu() - torch.tensor(o.outputs[0].logprob_values)).abs())
    g = torch.cat(gaps)
    assert g.mean() < 0.1 and g.max() < 1.0, (g.mean().item(), g.max().item())
    # weights changed -> the e4m3 copies follow
    s0 = eng.fp8[(0, "qkv")].w_scale.item()
    m.p("layers.0.qkv.weight").data.mul_(2.0)
    eng.update_weights(m.flat)
    assert abs(eng.fp8[(0, "qkv")].w_scale.item() / s0 - 2.0) < 0.05
    m.p("layers.0.qkv.weight").data.div_(2.0)


def test_decode_chain_matches_plain_launches():
    """The fused decode layers launched as a programmatic-dependent-launch chain (kernel prologues and the first
    weight tiles of every GEMM overlap the predecessor) against the same engine with plain stream-ordered launches:
    identical greedy tokens and log-probs over several hundred steps with rows of different lengths."""
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    cfg, m = _tiny()
    torch.manual_seed(5)
    prompts = [torch.randint(3, cfg.vocab_size, (n,)).tolist() for n in (3, 64, 129, 200, 17, 255, 90, 140, 33, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=300, n=1, logprobs=1, ignore_eos=True)
    outs = []
    for pdl in (True, False):
        eng = RolloutEngine(m, max_num_seqs=16, max_model_len=768, num_pages=80, seed=1, decode_pdl=pdl)
        outs.append(eng.generate(prompts, sp))
        _lib.check_status()
    for a, b in zip(*outs):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
        assert a.outputs[0].logprob_values == b.outputs[0].logprob_values
