"""Kernel micro-benchmarks: ``python -m bench.kernels --kernel gemm --m 8192 --n 8960 --k 1536``.

Times one kernel with CUDA events (3 warm-up launches, L2 flushed between timed launches by writing a 256 MiB
buffer) and prints achieved FLOP/s or bytes/s next to the measured peaks in MEASURED_PEAKS.json when that file is
present. The same command line is what the ncu summaries under ``profiles/`` were captured with."""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "of measured"
    except OSError:
        return 6650.0, 1590.0, "of fallback"


FLUSH = True
GRAPH = 0
CHAIN = False


def _time(fn, iters: int, flush: bool | None = None) -> float:
    flush = FLUSH if flush is None else flush
    if GRAPH > 0:
        # back-to-back launches inside one CUDA graph: per-launch device time without host launch latency and with
        # warm instruction / descriptor caches (the situation inside the captured decode loop)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        import contextlib

        from openrlhf_b200.ops import _lib
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g), (_lib.decode_chain() if CHAIN else contextlib.nullcontext()):
            for _ in range(GRAPH):
                fn()
        g.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) * 1e-3 / GRAPH
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e-3)
    return sorted(ts)[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=["gemm", "gemm_fp8", "gemm_splitk", "gemm_swiglu", "decode_attn", "attn_fwd", "attn_bwd", "logprob", "logprob_bwd",
                                                         "rmsnorm", "adamw", "decode_step", "decode_gemms", "sample", "ppo_loss", "gae"])
    ap.add_argument("--top-p", type=float, default=1.0, help="sample: nucleus threshold (1.0: plain Gumbel-max pass)")
    ap.add_argument("--model", default="qwen2.5-1.5b", help="decode_step: model preset")
    ap.add_argument("--layers", type=int, default=0, help="decode_step: cut the preset to this many layers (0: all)")
    ap.add_argument("--pdl", action="store_true", help="decode_step: launch the fused layers as a dependent-launch chain")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8960)
    ap.add_argument("--k", type=int, default=1536)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"], help="nt: fwd, nn: dgrad, tn: wgrad")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=1550)
    ap.add_argument("--hq", type=int, default=12)
    ap.add_argument("--hkv", type=int, default=2)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--bn", type=int, default=0, help="GEMM tile width (0: heuristic)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--graph", type=int, default=0, help="time N back-to-back launches inside one CUDA graph")
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between timed launches")
    ap.add_argument("--chain", action="store_true",
                    help="with --graph: record the launches as a programmatic-dependent-launch chain (decode loop)")
    a = ap.parse_args()
    global FLUSH, GRAPH, CHAIN
    FLUSH = not a.no_flush
    GRAPH = a.graph
    CHAIN = a.chain
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops import functional as F
    from openrlhf_b200.ops.attention import attn_bwd_tcgen05, attn_fwd_tcgen05, paged_decode
    from openrlhf_b200.ops.gemm import gemm, gemm_splitk

    hbm, tf, tag = _peaks()
    dev = "cuda"
    if a.kernel == "gemm_fp8":
        from openrlhf_b200.ops.fp8 import gemm_e4m3, quantize_e4m3
        M, N, K = a.m, a.n, a.k
        A = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        B = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        (aq, sa), (bq, sb) = quantize_e4m3(A), quantize_e4m3(B)
        t = _time(lambda: gemm_e4m3(aq, sa, bq, sb, bn=a.bn), a.iters)
        fl = 2.0 * M * N * K
        print(f"gemm_fp8 M{M} N{N} K{K} bn{a.bn}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s "
              f"({fl / t / 1e12 / tf:.2f} {tag} bf16 peak; nominal fp8 peak is twice the bf16 one)")
    elif a.kernel == "gemm_swiglu":
        # --n is the intermediate size I: y[M, I] = swiglu(x[M, K] @ w[2I, K]^T), fused vs GEMM + separate kernel
        from openrlhf_b200.ops.gemm import gemm_swiglu
        M, I, K = a.m, a.n, a.k
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(2 * I, K, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * M * 2 * I * K
        import openrlhf_b200.ops.gemm as G

        ref_y = None
        for pair in ("0", "1"):
            G.PAIR_KERNEL = pair
            yy, gg = gemm_swiglu(x, w, want_gate_up=True, bn=a.bn)
            if ref_y is not None:
                print(f"cta_group::2 vs single-CTA: max |dy| {(yy.float() - ref_y[0].float()).abs().max().item():.3g}, "
                      f"max |d gate_up| {(gg.float() - ref_y[1].float()).abs().max().item():.3g}")
            ref_y = (yy, gg)
            t = _time(lambda: gemm_swiglu(x, w, want_gate_up=True, bn=a.bn), a.iters)
            print(f"gemm_swiglu M{M} I{I} K{K} fused (y + gate_up), {'CTA pairs' if pair == '1' else 'single CTA'}: "
                  f"{t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s ({fl / t / 1e12 / tf:.2f} {tag} bf16 peak)")
        G.PAIR_KERNEL = "0"
        for name, fn in (("fused (y only)", lambda: gemm_swiglu(x, w, bn=a.bn)),
                         ("fused (y + gate_up)", lambda: gemm_swiglu(x, w, want_gate_up=True, bn=a.bn)),
                         ("gemm + swiglu kernel", lambda: F.swiglu(gemm(x, w, bn=a.bn)))):
            t = _time(fn, a.iters)
            print(f"gemm_swiglu M{M} I{I} K{K} bn{a.bn} {name}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s "
                  f"({fl / t / 1e12 / tf:.2f} {tag} bf16 peak)")
    elif a.kernel in ("gemm", "gemm_splitk"):
        M, N, K = a.m, a.n, a.k
        a_mn, b_mn = a.layout == "tn", a.layout in ("nn", "tn")
        A = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
        B = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
        if a.kernel == "gemm":
            fn = lambda: gemm(A, B, a_mn=a_mn, b_mn=b_mn, bn=a.bn)
        else:
            # distinct weight matrices in turn, more than L2 holds: every launch streams its weights from HBM, as the
            # layers of a decode step do
            Bs = [B] + [torch.randn_like(B) for _ in range(max(0, (300 << 20) // (2 * N * K)))]
            turn = [0]

            def fn():
                turn[0] += 1
                return gemm_splitk(A, Bs[turn[0] % len(Bs)], a.splits, bn=a.bn)
        t = _time(fn, a.iters)
        fl = 2.0 * M * N * K
        byt = 2.0 * (M * K + N * K + M * N)
        print(f"{a.kernel} M{M} N{N} K{K} {a.layout} bn{a.bn} splits{a.splits}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s "
              f"({fl / t / 1e12 / tf:.2f} {tag} bf16 peak), {byt / t / 1e9:.0f} GB/s ({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
        if a.kernel == "gemm":
            import openrlhf_b200.ops.gemm as G

            G.PAIR_KERNEL = "1"                      # the same GEMM on CTA pairs (tcgen05.mma.cta_group::2)
            if G._use_pair_kernel(M, N, K, 1, 0, a.bn):
                ref = gemm(A, B, a_mn=a_mn, b_mn=b_mn, bn=a.bn).float()
                G.PAIR_KERNEL = "0"
                one = gemm(A, B, a_mn=a_mn, b_mn=b_mn, bn=a.bn).float()
                G.PAIR_KERNEL = "1"
                err = (ref - one).abs().max().item()
                t2 = _time(fn, a.iters)
                print(f"cta_group::2 kernel: {t2 * 1e6:.1f} us, {fl / t2 / 1e12:.0f} TFLOP/s ({fl / t2 / 1e12 / tf:.2f} {tag} "
                      f"bf16 peak), max |diff| vs single-CTA kernel {err:.3g}")
            G.PAIR_KERNEL = "0"
            # the library GEMM on the same operands, same process, same timing loop
            At, Bt = (A.t() if a_mn else A), (B if b_mn else B.t())
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            tl = _time(lambda: torch.matmul(At, Bt, out=out), a.iters)
            print(f"torch.matmul same operands: {tl * 1e6:.1f} us, {fl / tl / 1e12:.0f} TFLOP/s; this kernel / library "
                  f"= {tl / t:.2f}x")
    elif a.kernel == "decode_attn":
        B_, Hq, Hkv, ctx = a.batch, a.hq, a.hkv, a.ctx
        per = ctx // 128 + 1
        kv = torch.randn(2, (B_ * per + 8) * 128, Hkv, 128, device=dev, dtype=torch.bfloat16)
        bt = torch.arange(B_ * per, device=dev, dtype=torch.int32).reshape(B_, per)
        sl = torch.full((B_,), ctx, device=dev, dtype=torch.int32)
        q = torch.randn(B_, Hq, 128, device=dev, dtype=torch.bfloat16)
        t = _time(lambda: paged_decode(q, kv[0], kv[1], bt, sl, 1 / math.sqrt(128), splits=a.splits), a.iters)
        byt = B_ * ctx * 2 * Hkv * 128 * 2
        print(f"decode_attn B{B_} Hq{Hq} Hkv{Hkv} ctx{ctx} splits{a.splits}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s "
              f"({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
    elif a.kernel == "sample":
        # sampler of the rollout engine over [batch, vocabulary] bf16 logits (--n: vocabulary size)
        from openrlhf_b200.ops.sampling import sample
        B, V = a.batch, a.n
        logits = torch.randn(max(B, (300 << 20) // (2 * V) + B), V, device=dev, dtype=torch.bfloat16)   # > L2
        toks = torch.zeros(B, dtype=torch.int64, device=dev)
        lps = torch.zeros(B, dtype=torch.float32, device=dev)
        turn = [0]

        def fn():
            turn[0] = (turn[0] + B) % (logits.shape[0] - B + 1)
            return sample(logits[turn[0]:turn[0] + B], temperature=1.0, top_k=-1, top_p=a.top_p, seed=1, step=turn[0],
                          out_tokens=toks, out_logprobs=lps)
        t = _time(fn, a.iters)
        byt = 2.0 * B * V
        print(f"sample B{B} V{V} top_p{a.top_p}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s of logits "
              f"({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
    elif a.kernel == "ppo_loss":
        # fused clipped-surrogate loss + k3 KL + metrics over [sequences, action tokens] fp32 (--m x --n), forward and
        # backward (the backward is a scale of the dlogp the forward kernel already wrote)
        from openrlhf_b200.ops.rl import ppo_loss
        Bq, A = a.m, a.n
        logp = (-torch.rand(Bq, A, device=dev)).requires_grad_()
        old = logp.detach() + 0.05 * torch.randn(Bq, A, device=dev)
        ref = logp.detach() + 0.05 * torch.randn(Bq, A, device=dev)
        adv = torch.randn(Bq, A, device=dev)
        mask = (torch.rand(Bq, A, device=dev) > 0.1).float()

        def fn():
            logp.grad = None
            out = ppo_loss(logp, old, adv, mask, ref_logp=ref, kl_coef=0.001, kl_estimator="k3")
            out["loss"].backward()
        t = _time(fn, a.iters)
        byt = 4.0 * Bq * A * 7          # five inputs read, dlogp written and read once more by the backward scale
        print(f"ppo_loss fwd+bwd B{Bq} A{A}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s ({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
    elif a.kernel == "gae":
        # reward shaping + GAE scan over [sequences, action tokens] fp32 (--m x --n)
        from openrlhf_b200.ops.rl import gae_advantages
        Bq, A = a.m, a.n
        values, kl = torch.randn(Bq, A, device=dev), 0.01 * torch.randn(Bq, A, device=dev)
        mask = torch.ones(Bq, A, device=dev)
        rew = torch.randn(Bq, device=dev)
        t = _time(lambda: gae_advantages(values, kl, rew, mask, beta=0.01, gamma=1.0, lambd=0.95), a.iters)
        byt = 4.0 * Bq * A * 5
        print(f"gae B{Bq} A{A}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s ({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
    elif a.kernel == "decode_gemms":
        # the four projections of one decoder layer at decode batch size, launched exactly as the rollout engine
        # launches them (split-K into the fp32 workspace / SwiGLU epilogue), over distinct weights in turn so that
        # every launch streams from HBM; use --graph N (and --chain) for the in-graph situation
        import dataclasses

        from openrlhf_b200.models.config import PRESETS
        from openrlhf_b200.ops.gemm import gemm_swiglu
        from openrlhf_b200.rollout.engine import gemm_to_workspace
        cfg = dataclasses.replace(PRESETS[a.model])
        H, I, B = cfg.hidden_size, cfg.intermediate_size, a.batch
        shapes = {"qkv": (cfg.qkv_size, H), "o": (H, cfg.q_size), "gate_up": (2 * I, H), "down": (H, I)}
        for name, (N, K) in shapes.items():
            x = torch.randn(B, K, device=dev, dtype=torch.bfloat16)
            ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
                  for _ in range(1 + (300 << 20) // (2 * N * K))]
            turn = [0]

            def fn():
                turn[0] += 1
                w = ws[turn[0] % len(ws)]
                if name == "gate_up":
                    return gemm_swiglu(x, w, bn=128)
                return gemm_to_workspace(x, w)
            t = _time(fn, a.iters)
            byt = 2.0 * N * K
            outs = torch.empty(B, N, device=dev, dtype=torch.bfloat16)

            def lib_fn():
                turn[0] += 1
                return torch.matmul(x, ws[turn[0] % len(ws)].t(), out=outs)
            t_lib = _time(lib_fn, a.iters)
            print(f"decode_gemms {a.model} B{B} {name} N{N} K{K}: {t * 1e6:.1f} us, weights {byt / t / 1e9:.0f} GB/s "
                  f"({byt / t / 1e9 / hbm:.2f} {tag} HBM), chain {CHAIN}, graph {GRAPH}; torch.matmul (no SwiGLU, bf16 "
                  f"output): {t_lib * 1e6:.1f} us")
            del ws
    elif a.kernel == "decode_step":
        # the rollout engine's whole decode step (CUDA graph of one token for `batch` sequences at context `ctx`),
        # through the public engine API; host work of the scheduler is included, amortised over its 32-step bursts
        import dataclasses

        from openrlhf_b200.models.config import PRESETS
        from openrlhf_b200.models.transformer import TransformerLM
        from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
        cfg = dataclasses.replace(PRESETS[a.model])
        if a.layers:
            cfg.num_hidden_layers = a.layers
        m = TransformerLM(cfg, device=dev, seed=0)
        B, ctx, bursts = a.batch, a.ctx, max(2, a.iters)
        chunks = (B * ctx + 16383) // 16384          # rows that finish their prefill early decode during the others'
        interval = 4                                 # bursts of 4 steps while rows still prefill, 8 x 4 afterwards
        new = interval * (8 * (bursts + 5) + chunks + 4)
        eng = RolloutEngine(m, max_num_seqs=B, max_model_len=ctx + new + 128,
                            num_pages=B * ((ctx + new) // 128 + 2) + 8, seed=1, decode_pdl=a.pdl,
                            check_interval=interval)
        g = torch.Generator().manual_seed(0)
        sp = SamplingParams(temperature=1.0, max_tokens=new, n=1, ignore_eos=True)
        for i in range(B):
            eng.add_request(i, torch.randint(3, cfg.vocab_size, (ctx,), generator=g).tolist(), sp)
        new_steps = 0
        for _ in range(chunks + 8):  # chunked prefill of every row, graph capture, then three warm-up bursts
            eng.step()
            decoding = sum(1 for r in eng.rows if r is not None and r.prefilled < 0)
            new_steps += 1 if decoding == B else 0
            if new_steps == 3:
                break
        assert new_steps == 3, "the rows did not all reach the decode phase"
        torch.cuda.synchronize()
        d0 = eng.decode_steps
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        for _ in range(bursts):
            eng.step()
        e_.record()
        torch.cuda.synchronize()
        _lib.check_status()
        n = eng.decode_steps - d0
        t = s_.elapsed_time(e_) * 1e-3 / n
        wbytes = (m.flat.numel() - (0 if cfg.tie_word_embeddings else cfg.vocab_size * cfg.hidden_size)) * 2
        kvbytes = 2 * cfg.num_hidden_layers * B * (ctx + interval * 8 * 3 + n // 2) * cfg.kv_size * 2
        print(f"decode_step {a.model} layers{cfg.num_hidden_layers} B{B} ctx{ctx}: {t * 1e3:.3f} ms per step over {n} "
              f"steps, {(wbytes + kvbytes) / t / 1e9:.0f} GB/s of weights + KV ({(wbytes + kvbytes) / t / 1e9 / hbm:.2f} "
              f"{tag} HBM), launches per graph {eng.graph_launches}, dependent-launch chain {a.pdl}")
    elif a.kernel == "attn_fwd":
        T, Hq, Hkv, L = a.m, a.hq, a.hkv, a.ctx
        qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device=dev, dtype=torch.bfloat16)
        q = qkv[:, : Hq * 128].view(T, Hq, 128)
        k = qkv[:, Hq * 128:(Hq + Hkv) * 128].view(T, Hkv, 128)
        v = qkv[:, (Hq + Hkv) * 128:].view(T, Hkv, 128)
        cu = torch.arange(0, T + 1, L, device=dev, dtype=torch.int32)
        t = _time(lambda: attn_fwd_tcgen05(q, k, v, cu, 1 / math.sqrt(128)), a.iters)
        fl = 4.0 * (T // L) * (L * (L + 128) / 2) * Hq * 128
        print(f"attn_fwd T{T} seq{L} Hq{Hq} Hkv{Hkv}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s "
              f"({fl / t / 1e12 / tf:.2f} {tag} bf16 peak)")
    elif a.kernel == "attn_bwd":
        T, Hq, Hkv, L = a.m, a.hq, a.hkv, a.ctx
        qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device=dev, dtype=torch.bfloat16)
        q = qkv[:, : Hq * 128].view(T, Hq, 128)
        k = qkv[:, Hq * 128:(Hq + Hkv) * 128].view(T, Hkv, 128)
        v = qkv[:, (Hq + Hkv) * 128:].view(T, Hkv, 128)
        cu = torch.arange(0, T + 1, L, device=dev, dtype=torch.int32)
        out, lse = attn_fwd_tcgen05(q, k, v, cu, 1 / math.sqrt(128))
        dout = torch.randn_like(out)
        t = _time(lambda: attn_bwd_tcgen05(q, k, v, out, dout, lse, cu, 1 / math.sqrt(128)), a.iters)
        fl = 10.0 * (T // L) * (L * (L + 128) / 2) * Hq * 128
        print(f"attn_bwd T{T} seq{L} Hq{Hq} Hkv{Hkv}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s "
              f"({fl / t / 1e12 / tf:.2f} {tag} bf16 peak; includes delta, zeroing and the fp32->bf16 pass)")
    elif a.kernel == "logprob":
        T, V, H = a.m, a.n, a.k
        h = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        w = (0.02 * torch.randn(V, H, device=dev)).to(torch.bfloat16)
        y = torch.randint(0, V, (T,), device=dev)
        with torch.no_grad():
            t = _time(lambda: F.fused_logprob(h, w, y), a.iters)
        fl = 2.0 * T * V * H
        print(f"logprob T{T} V{V} H{H}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s ({fl / t / 1e12 / tf:.2f} {tag} bf16 peak)")
    elif a.kernel == "logprob_bwd":
        T, V, H = a.m, a.n, a.k
        h = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = (0.02 * torch.randn(V, H, device=dev)).to(torch.bfloat16).requires_grad_()
        w.main_grad = torch.zeros(V, H, device=dev, dtype=torch.float32)
        y = torch.randint(0, V, (T,), device=dev)
        g = torch.randn(T, device=dev)

        def step():
            lp, _ = F.fused_logprob(h, w, y)
            lp.backward(g)
            h.grad = None

        t = _time(step, a.iters)
        fl = 8.0 * T * V * H              # forward, recomputation, dH and dW GEMMs
        print(f"logprob fwd+bwd T{T} V{V} H{H}: {t * 1e6:.1f} us, {fl / t / 1e12:.0f} TFLOP/s ({fl / t / 1e12 / tf:.2f} {tag} bf16 peak)")
    elif a.kernel == "rmsnorm":
        T, H = a.m, a.k
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            t = _time(lambda: F.rmsnorm(x, w, 1e-6), a.iters)
        byt = 4.0 * T * H
        print(f"rmsnorm T{T} H{H}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s ({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
        # backward: reads x and dy, writes dx (the fp32 weight gradient is H floats)
        import ctypes

        dy, dx = torch.randn_like(x), torch.empty_like(x)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        dw = torch.zeros(H, device=dev)
        L = _lib.lib()
        bwd = lambda: L.b200_rmsnorm_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), None, _lib.ptr(dx),
                                         _lib.ptr(dw), ctypes.c_int(T), ctypes.c_int(H), _lib.stream_ptr())
        t = _time(bwd, a.iters)
        byt = 6.0 * T * H
        print(f"rmsnorm_bwd T{T} H{H}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s ({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
    elif a.kernel == "adamw":
        import ctypes

        n = a.m * a.k
        ms, m1, v1, g = (torch.randn(n, device=dev) for _ in range(4))
        pb = torch.empty(n, device=dev, dtype=torch.bfloat16)
        L = _lib.lib()
        fn = lambda: L.b200_adamw(_lib.ptr(ms), _lib.ptr(m1), _lib.ptr(v1), _lib.ptr(g), _lib.ptr(pb),
                                  ctypes.c_longlong(n), None, ctypes.c_float(1e-5), ctypes.c_float(0.9),
                                  ctypes.c_float(0.95), ctypes.c_float(1e-8), ctypes.c_float(0.0), ctypes.c_int(1),
                                  ctypes.c_int(1), _lib.stream_ptr())
        t = _time(fn, a.iters)
        byt = n * (4 * 4 + 3 * 4 + 4 + 2)
        print(f"adamw n{n}: {t * 1e6:.1f} us, {byt / t / 1e9:.0f} GB/s ({byt / t / 1e9 / hbm:.2f} {tag} HBM)")
    _lib.check_status()


if __name__ == "__main__":
    main()
