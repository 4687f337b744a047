"""Each CUDA op against the PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, rtol=2e-2, atol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= rtol * ref + atol, f"max err {err} vs ref scale {ref}"


@pytest.mark.parametrize("T,H", [(333, 1536), (2000, 1536), (1031, 2048), (700, 3584), (600, 5120), (513, 72)])
def test_rmsnorm_fwd_bwd(T, H):
    """Covers the block-per-row kernels (few rows, or wide rows in the backward) and the warp-per-row kernels."""
    from openrlhf_b200.ops import functional as F, reference as R
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = F.rmsnorm(x, w, 1e-6)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(); wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    yr.backward(dy.float())
    _close(y, yr); _close(x.grad, xr.grad); _close(w.grad, wr.grad, rtol=3e-2, atol=0.3)


def test_rope_and_swiglu_and_embedding():
    from openrlhf_b200.ops import functional as F, reference as R
    torch.manual_seed(0)
    T, Hq, Hkv, D = 257, 12, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    tab = F.rope_table(D, 1e6, 4096, "cuda")
    out = F.rope(qkv, pos, tab, Hq + Hkv, D)
    ref = R.rope(qkv.detach(), pos, tab, Hq + Hkv, D)
    _close(out, ref)
    g = torch.randn_like(out); out.backward(g)
    # rotation is orthogonal: the backward of a rotation is the inverse rotation
    back = R.rope(qkv.grad, pos, tab, Hq + Hkv, D)
    _close(back, g, rtol=3e-2, atol=3e-2)
    gu = torch.randn(T, 2 * 8960, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.swiglu(gu); dy = torch.randn_like(y); y.backward(dy)
    gr = gu.detach().float().requires_grad_(); yr = torch.nn.functional.silu(gr[:, :8960]) * gr[:, 8960:]; yr.backward(dy.float())
    _close(y, yr); _close(gu.grad, gr.grad)
    table = torch.randn(1000, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (T,), device="cuda")
    e = F.embedding(ids, table); de = torch.randn_like(e); e.backward(de)
    tr = table.detach().float().requires_grad_(); er = tr[ids]; er.backward(de.float())
    _close(e, er); _close(table.grad, tr.grad)


def test_linear_autograd():
    from openrlhf_b200.ops import functional as F
    torch.manual_seed(0)
    T, K, N = 515, 1536, 2048
    x = (0.5 * torch.randn(T, K, device="cuda")).to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(N, K, device="cuda")).to(torch.bfloat16).requires_grad_()
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(T, N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.linear(x, w, b, res); dy = torch.randn_like(y); y.backward(dy)
    xr, wr, br, rr = [t.detach().float().requires_grad_() for t in (x, w, b, res)]
    yr = xr @ wr.t() + br + rr; yr.backward(dy.float())
    _close(y, yr); _close(x.grad, xr.grad); _close(w.grad, wr.grad); _close(b.grad, br.grad, atol=0.3); _close(res.grad, rr.grad)


def test_fused_logprob_fwd_bwd():
    from openrlhf_b200.ops import functional as F
    torch.manual_seed(0)
    T, H, V = 300, 512, 4096
    h = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = torch.randint(0, V, (T,), device="cuda")
    logp, ent = F.fused_logprob(h, w, y, temperature=0.7, want_entropy=True, chunk=128)
    g = torch.randn(T, device="cuda")
    logp.backward(g)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = hr @ wr.t()
    lr = torch.log_softmax(logits / 0.7, -1).gather(-1, y[:, None]).squeeze(-1)
    p = torch.softmax(logits, -1); er = torch.logsumexp(logits, -1) - (p * logits).sum(-1)
    lr.backward(g)
    _close(logp, lr, atol=3e-2); _close(ent, er, atol=3e-2)
    _close(h.grad, hr.grad, rtol=4e-2, atol=4e-2); _close(w.grad, wr.grad, rtol=4e-2, atol=4e-2)


@pytest.mark.parametrize("T,H,V,temp,chunk", [(130, 256, 5000, 1.0, 128), (1, 128, 264, 0.5, 128),
                                              (257, 320, 1000, 1.3, 128), (1300, 256, 5000, 0.9, 2048)])
def test_fused_logprob_ragged_vocabulary_and_edge_labels(T, H, V, temp, chunk):
    """Vocabulary sizes that are not multiples of the 256-column tile (the last tile is partly outside), token counts
    that are not multiples of 128 and labels on the first / last column, against the fp32 PyTorch computation."""
    from openrlhf_b200.ops import functional as F
    torch.manual_seed(1)
    h = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.08 * torch.randn(V, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = torch.randint(0, V, (T,), device="cuda")
    y[0] = V - 1
    y[-1] = 0
    logp, ent = F.fused_logprob(h, w, y, temperature=temp, want_entropy=True, chunk=chunk)   # >= 1024: CTA pairs
    g = torch.randn(T, device="cuda")
    logp.backward(g)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = hr @ wr.t()
    lr = torch.log_softmax(logits / temp, -1).gather(-1, y[:, None]).squeeze(-1)
    p = torch.softmax(logits, -1); er = torch.logsumexp(logits, -1) - (p * logits).sum(-1)
    lr.backward(g)
    _close(logp, lr, atol=3e-2); _close(ent, er, atol=3e-2)
    _close(h.grad, hr.grad, rtol=4e-2, atol=4e-2); _close(w.grad, wr.grad, rtol=4e-2, atol=4e-2)
    logp2, none = F.fused_logprob(h.detach(), w.detach(), y, temperature=temp, want_entropy=False)
    assert none is None
    _close(logp2, lr.detach(), atol=3e-2)


@pytest.mark.parametrize("B,Hq,Hkv,splits", [(3, 12, 2, 1), (5, 32, 8, 1), (4, 28, 4, 3), (2, 16, 2, 2)])
def test_paged_decode(B, Hq, Hkv, splits):
    from openrlhf_b200.ops import _lib, reference as R
    from openrlhf_b200.ops.attention import paged_decode
    torch.manual_seed(0)
    D, page, num_pages, max_pages = 128, 128, 64, 8
    k_cache = torch.randn(num_pages * page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.randn(num_pages * page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(num_pages, device="cuda")[: B * max_pages].reshape(B, max_pages).int()
    seq_lens = torch.tensor([1, 127, 128, 129, 700, 1000][:B], device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    scale = 1 / math.sqrt(D)
    out = paged_decode(q, k_cache, v_cache, perm, seq_lens, scale, splits=splits)
    _lib.check_status()
    ref = R.paged_decode_attention(q, k_cache, v_cache, perm, seq_lens, scale)
    _close(out, ref, rtol=2e-2, atol=2e-2)


def test_rope_kvwrite():
    from openrlhf_b200.ops import functional as F, reference as R
    from openrlhf_b200.ops.attention import rope_kvwrite
    torch.manual_seed(0)
    T, Hq, Hkv, D = 37, 12, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 2000, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(512, device="cuda")[:T].int()
    tab = F.rope_table(D, 1e6, 4096, "cuda")
    q_out = torch.empty(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(512, Hkv, D, device="cuda", dtype=torch.bfloat16); vc = torch.zeros_like(kc)
    rope_kvwrite(qkv, pos, slots, tab, q_out, kc, vc, Hq, Hkv)
    ref = R.rope(qkv, pos, tab, Hq + Hkv, D)
    _close(q_out.reshape(T, -1), ref[:, : Hq * D])
    _close(kc[slots.long()].reshape(T, -1), ref[:, Hq * D:(Hq + Hkv) * D])
    _close(vc[slots.long()].reshape(T, -1), ref[:, (Hq + Hkv) * D:])


def test_sampler_greedy_and_distribution():
    import ctypes
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops.sampling import sample
    torch.manual_seed(0)
    B, V = 64, 1024
    logits = torch.randn(B, V, device="cuda").to(torch.bfloat16)
    tok, lp = sample(logits, temperature=0.0)
    assert torch.equal(tok, logits.float().argmax(-1))
    ref_lp = torch.log_softmax(logits.float(), -1).gather(-1, tok[:, None]).squeeze(-1)
    _close(lp, ref_lp, atol=1e-3)
    # distribution check on a tiny vocabulary: empirical frequencies match softmax
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-30.0] * 4], device="cuda").repeat(4096, 1)
    tok, lp = sample(z, temperature=1.0, seed=123, step=7)
    freq = torch.bincount(tok, minlength=8).float() / tok.numel()
    p = torch.softmax(z[0], -1)
    assert (freq - p).abs().max().item() < 0.03
    _close(lp, torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1), atol=1e-3)
    # top-p keeps only the head of the distribution
    tok, lp = sample(z, temperature=1.0, top_p=0.6, seed=5, step=1)
    assert int(tok.max()) <= 1
    tok, _ = sample(z, temperature=1.0, top_k=1, seed=5, step=2)
    assert int(tok.max()) == 0


def test_sampler_large_vocab_distribution():
    """Inverse-CDF draw over a bf16 vocabulary that spans all warp segments: bucketed frequencies follow softmax."""
    from openrlhf_b200.ops.sampling import sample
    torch.manual_seed(1)
    V, R = 20011, 16384
    row = (torch.randn(V, device="cuda") * 2.0).to(torch.bfloat16)
    z = row[None, :].repeat(R, 1)
    tok, lp = sample(z, temperature=0.8, seed=11, step=3)
    p = torch.softmax(row.float() / 0.8, -1)
    _close(lp, torch.log(p)[tok], atol=2e-3)
    buckets = (torch.arange(V, device="cuda") * 16 // V)           # 16 contiguous index ranges (cross warp segments)
    want = torch.zeros(16, device="cuda").index_add_(0, buckets, p)
    got = torch.bincount(buckets[tok], minlength=16).float() / R
    assert (got - want).abs().max().item() < 0.02, (got - want).abs().max().item()
    # different steps give different draws, same (seed, step) the same draw
    t2, _ = sample(z, temperature=0.8, seed=11, step=3)
    t3, _ = sample(z, temperature=0.8, seed=11, step=4)
    assert torch.equal(tok, t2) and not torch.equal(tok, t3)


def test_rl_kernels_match_reference():
    from openrlhf_b200.ops import rl as K
    torch.manual_seed(0)
    B, A = 9, 77
    mask = (torch.rand(B, A, device="cuda") > 0.2).float(); mask[:, 0] = 1
    logp = -torch.rand(B, A, device="cuda"); old = logp + 0.3 * torch.randn(B, A, device="cuda")
    adv = torch.randn(B, A, device="cuda"); ref = logp + 0.2 * torch.randn(B, A, device="cuda")
    roll = old + 0.1 * torch.randn(B, A, device="cuda")
    for kw in [dict(), dict(dual_clip=3.0), dict(kl_coef=0.05, kl_estimator="k3"), dict(is_mode="tis", is_lo=0.5, is_hi=2.0),
               dict(is_mode="icepop", is_lo=0.8, is_hi=1.2, kl_coef=0.1, kl_estimator="k2")]:
        lp_c = logp.clone().requires_grad_(); lp_r = logp.clone().requires_grad_()
        out_c = K.ppo_loss(lp_c, old, adv, mask, ref_logp=ref, rollout_logp=roll, **kw)
        out_r = K.ppo_loss_reference(lp_r, old, adv, mask, ref_logp=ref, rollout_logp=roll, **kw)
        out_c["loss"].backward(); out_r["loss"].backward()
        for k in ("loss", "policy_loss", "kl_loss", "clip_ratio", "ppo_kl", "vllm_kl"):
            _close(out_c[k], out_r[k], rtol=1e-3, atol=1e-4)
        _close(lp_c.grad, lp_r.grad, rtol=1e-3, atol=1e-5)
    vals = torch.randn(B, A, device="cuda"); r = torch.randn(B, device="cuda"); kl = torch.rand(B, A, device="cuda")
    for use_v in (True, False):
        a1, r1, s1 = K.gae_advantages(vals if use_v else None, kl, r, mask, beta=0.1, gamma=0.99, lambd=0.95, clip=(-10, 10))
        a2, r2, s2 = K.gae_advantages_reference(vals if use_v else None, kl, r, mask, beta=0.1, gamma=0.99, lambd=0.95, clip=(-10, 10))
        _close(a1, a2, rtol=1e-3, atol=1e-4); _close(r1, r2, rtol=1e-3, atol=1e-4); _close(s1, s2, rtol=1e-3, atol=1e-4)
    w1 = K.masked_whiten(adv.clone(), mask); w2 = K.masked_whiten_reference(adv.clone(), mask)
    _close(w1 * mask, w2 * mask, rtol=1e-3, atol=1e-4)
    v = vals.clone().requires_grad_(); v2 = vals.clone().requires_grad_()
    l1 = K.value_loss(v, vals + 0.3, r1, mask, clip_eps=0.2); l2 = K.value_loss_reference(v2, vals + 0.3, r1, mask, clip_eps=0.2)
    l1.backward(); l2.backward()
    _close(l1, l2, rtol=1e-3, atol=1e-5); _close(v.grad, v2.grad, rtol=1e-3, atol=1e-6)


@pytest.mark.parametrize("Hq,Hkv,lens", [(4, 2, [1, 127, 128, 129, 300]), (12, 2, [513, 40]), (8, 8, [1024]),
                                         (7, 1, [700, 129, 5, 256])])
def test_attn_fwd_tcgen05(Hq, Hkv, lens):
    from openrlhf_b200.ops import _lib, reference as R
    from openrlhf_b200.ops.attention import attn_fwd_tcgen05
    torch.manual_seed(0)
    T, D = sum(lens), 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out, lse = attn_fwd_tcgen05(q, k, v, cu, scale)
    _lib.check_status()
    ref = R.attention_varlen(q, k, v, cu, scale)
    _close(out, ref, rtol=2e-2, atol=2e-2)
    # log-sum-exp against a direct computation for the first sequence / head 0
    L = lens[0]
    s = (q[:L, 0].float() @ k[:L, 0].float().t()) * scale
    s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    _close(lse[0, :L], torch.logsumexp(s, -1), rtol=1e-2, atol=1e-2)


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("Hq,Hkv,lens", [(4, 2, [100, 200]), (12, 2, [513, 40, 128]), (7, 1, [700, 129, 5, 256]),
                                         (2, 2, [1, 127, 129])])
def test_attention_autograd_matches_reference(Hq, Hkv, lens):
    """Forward and backward (tcgen05 kernels) against fp32 PyTorch autograd of the same op."""
    from openrlhf_b200.ops import _lib, functional as F, reference as R
    torch.manual_seed(0)
    T, D = sum(lens), 128
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    out = F.attention_varlen(q, k, v, cu, max(lens))
    g = torch.randn_like(out)
    out.backward(g)
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = R.attention_varlen(qr, kr, vr, cu, 1 / math.sqrt(D))
    ref.backward(g.float())
    _close(out, ref)
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        assert torch.isfinite(a).all(), name
        assert _rel_err(a, b) < 2e-2, (name, _rel_err(a, b))
        _close(a, b, rtol=5e-2, atol=5e-2)


def test_rope_attention_fused_matches_reference():
    """Fused rotary + attention autograd function: output and the gradient of the un-rotated fused qkv."""
    from openrlhf_b200.ops import _lib, functional as F, reference as R
    from openrlhf_b200.ops.attention import rope_attention
    torch.manual_seed(1)
    Hq, Hkv, D, lens = 6, 2, 128, [300, 77, 130]
    T = sum(lens)
    W = (Hq + 2 * Hkv) * D
    x = torch.randn(T, W, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).to("cuda", torch.int32)
    table = F.rope_table(D, 10000.0, 512, "cuda")
    scale = 1 / math.sqrt(D)
    out = rope_attention(x * 1.0, pos, table, cu, Hq, Hkv, scale)
    g = torch.randn_like(out)
    out.backward(g)
    _lib.check_status()
    xr = x.detach().float().requires_grad_()
    r = R.rope(xr, pos, table.float(), Hq + Hkv, D)
    ref = R.attention_varlen(r[:, : Hq * D].view(T, Hq, D), r[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D),
                             r[:, (Hq + Hkv) * D:].view(T, Hkv, D), cu, scale).reshape(T, Hq * D)
    ref.backward(g.float())
    _close(out, ref, rtol=3e-2, atol=3e-2)
    assert _rel_err(x.grad, xr.grad) < 2e-2, _rel_err(x.grad, xr.grad)


@pytest.mark.parametrize("tp,src_world", [(1, 1), (2, 1), (2, 4)])
def test_reshard_plan_kernel(tp, src_world):
    """Weight-sync copy plan executed by the CUDA kernel (sources = local buffers standing in for peer shards)
    against the PyTorch executor of the same plan."""
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.transformer import build_param_specs
    from openrlhf_b200.parallel.reshard import ReshardPlan, build_plan, run_plan_reference
    cfg = PRESETS["tiny-llama"]
    specs = build_param_specs(cfg)
    size = specs[-1].offset + (specs[-1].numel + 127) // 128 * 128
    flat = torch.randn(size, device="cuda").to(torch.bfloat16)
    shard, srcs = None, [flat]
    if src_world > 1:
        shard = (size + src_world * 256 - 1) // (src_world * 256) * 256
        padded = torch.cat([flat, torch.zeros(shard * src_world - size, device="cuda", dtype=torch.bfloat16)])
        srcs = [padded[r * shard:(r + 1) * shard].clone() for r in range(src_world)]
    for tp_rank in range(tp):
        entries, dsize = build_plan(cfg, tp_rank, tp, src_world, shard)
        want = torch.zeros(dsize, dtype=torch.bfloat16)
        run_plan_reference(entries, [s.cpu() for s in srcs], want)
        got = torch.zeros(dsize, device="cuda", dtype=torch.bfloat16)
        ReshardPlan(entries, "cuda").run([s.data_ptr() for s in srcs], got)
        torch.cuda.synchronize()
        assert torch.equal(got.cpu(), want)
        # the same plan under a block budget (a copy that shares the GPU with compute kernels): fewer blocks, each
        # with several loads in flight, identical result
        for budget in (1, 37, 296):
            got.zero_()
            ReshardPlan(entries, "cuda").run([s.data_ptr() for s in srcs], got, max_ctas=budget)
            torch.cuda.synchronize()
            assert torch.equal(got.cpu(), want), budget


@pytest.mark.parametrize("T,H,I,E,k", [(300, 128, 128, 8, 2), (1000, 256, 192, 16, 4)])
def test_moe_grouped_matches_expert_loop(T, H, I, E, k):
    """Grouped tcgen05 GEMM MoE block against the per-expert loop (fp32 reference for the gradients)."""
    from openrlhf_b200.models import moe
    from openrlhf_b200.ops import _lib
    torch.manual_seed(0)
    x = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    rw = (torch.randn(E, H, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    gu = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    dn = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y, aux = moe.moe_forward_grouped(x, rw, gu, dn, k, True)
    g = torch.randn_like(y)
    (y.float() * g.float()).sum().backward()
    _lib.check_status()
    got = [t.grad.float().clone() for t in (x, gu, dn)]
    for t in (x, rw, gu, dn):
        t.grad = None
    y2, aux2 = moe.moe_forward(x, rw, gu, dn, k, True, expert_range=(0, E))
    (y2.float() * g.float()).sum().backward()
    ref = [t.grad.float() for t in (x, gu, dn)]
    rel = lambda a, b: ((a - b).norm() / b.norm().clamp_min(1e-6)).item()
    assert rel(y.float(), y2.float()) < 2e-2, rel(y.float(), y2.float())
    assert abs(aux.item() - aux2.item()) < 1e-4
    for name, a, b in zip(("dx", "dgate_up", "ddown"), got, ref):
        assert rel(a, b) < 3e-2, (name, rel(a, b))


@pytest.mark.parametrize("T,E,k,norm", [(257, 8, 2, True), (1000, 128, 8, True), (64, 60, 4, False)])
def test_moe_router_kernel(T, E, k, norm):
    """Fused router (softmax, top-k, renorm) and its backward against PyTorch fp32."""
    from openrlhf_b200.models.moe import _RouteFn
    torch.manual_seed(0)
    logits = torch.randn(T, E, device="cuda", requires_grad=True)
    w, idx, probs = _RouteFn.apply(logits, k, norm)
    ref_l = logits.detach().clone().requires_grad_()
    rp = torch.softmax(ref_l, -1)
    rw, ridx = rp.topk(k, -1)
    if norm:
        rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(idx.sort(-1).values, ridx.sort(-1).values)
    _close(probs, rp, rtol=1e-4, atol=1e-6)
    _close(w.gather(1, idx.argsort(-1)), rw.gather(1, ridx.argsort(-1)), rtol=1e-4, atol=1e-6)
    gw, gp = torch.randn_like(w), torch.randn_like(probs)
    # same pairing of weights and upstream gradients on both sides: order by expert index
    (w.gather(1, idx.argsort(-1)) * gw).sum().add((probs * gp).sum()).backward()
    (rw.gather(1, ridx.argsort(-1)) * gw).sum().add((rp * gp).sum()).backward()
    _close(logits.grad, ref_l.grad, rtol=1e-3, atol=1e-5)


def test_nf4_kernels_match_cpu_restatement():
    from openrlhf_b200.ops import nf4
    torch.manual_seed(0)
    w = (torch.randn(64 * 4097) * 0.03).bfloat16()
    w[64:128] = 0
    codes, absmax = nf4.quantize(w.cuda())
    rc, ra = nf4.quantize(w.float())
    assert torch.equal(codes.cpu(), rc) and torch.allclose(absmax.cpu(), ra)
    d = nf4.dequantize(codes, absmax)
    assert torch.equal(d.cpu(), nf4.dequantize(rc, ra, torch.bfloat16))
