"""Multi-GPU micro-benchmarks of the fused compute + collective kernels (one process per GPU under torchrun):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/collectives.py [--only zero_reduce,...] [--model qwen2.5-1.5b]

Every number is device-timed with CUDA events on the launching stream (3 warm-up launches, 10 timed ones separated by
a group barrier) and reported as the MAX over ranks. For each kernel the line gives the bytes that have to cross
NVLink per GPU and direction, the achieved GB/s and its fraction of the measured peer-copy rate (770 GB/s per
direction on this pool; 900 nominal), and for the GEMM-shaped ones the FLOP/s next to the measured cuBLAS rate.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 770.0


def peaks():
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), "of measured"
    except OSError:
        return 1590.0, "of fallback"


def timed(fn, group, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier(group)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t) * 1e-3


def report(rank, name, secs, link_bytes=None, flops=None, note=""):
    if rank != 0:
        return
    tf, how = peaks()
    out = {"kernel": name, "ms": round(secs * 1e3, 4), "world": dist.get_world_size()}
    if link_bytes is not None:
        out["nvlink_bytes_per_gpu_per_direction"] = int(link_bytes)
        out["nvlink_gbs"] = round(link_bytes / secs / 1e9, 1)
        out["frac_of_770_gbs"] = round(link_bytes / secs / 1e9 / LINK_GBS, 3)
    if flops is not None:
        out["tflops"] = round(flops / secs / 1e12, 1)
        out[f"frac_bf16_peak_{how.replace(' ', '_')}"] = round(flops / secs / 1e12 / tf, 3)
    if link_bytes is not None and flops is not None:
        bound = max(link_bytes / (LINK_GBS * 1e9), flops / (tf * 1e12))
        out["roofline_ms"] = round(bound * 1e3, 4)
        out["frac_of_roofline"] = round(bound / secs, 3)
    if note:
        out["note"] = note
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--model", default="qwen2.5-1.5b")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    G = dist.group.WORLD
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.parallel.zero import ZeroEngine
    from openrlhf_b200.parallel.zero3 import Zero3Engine

    want = set(x for x in args.only.split(",") if x)
    on = lambda n: not want or n in want
    L = _lib.lib()
    cfg = PRESETS[args.model]
    dev = torch.device("cuda")

    # ---------------------------------------------------------------- ZeRO-1/2 optimizer step kernels
    if on("zero_reduce") or on("zero_adam_gather"):
        model = TransformerLM(cfg, device=dev, seed=0, shard_world=world)
        eng = ZeroEngine(model, lr=1e-6, zero_stage=2, group=G, use_symm=True)
        sy = eng.symm
        n, lo = eng.shard_size, eng.lo
        red = torch.empty(n, dtype=torch.float32, device=dev)
        sy.grad.normal_()

        def reduce():
            rc = L.b200_zero_reduce(sy.grad_ptrs, ctypes.c_void_p(0), ctypes.c_int(world), ctypes.c_longlong(lo),
                                    ctypes.c_longlong(n), ctypes.c_float(1.0 / world), _lib.ptr(red),
                                    _lib.ptr(eng.scalars), ctypes.c_int(0), _lib.stream_ptr())
            _lib.check_rc(rc, "zero_reduce")

        if on("zero_reduce"):
            t = timed(reduce, G)
            report(rank, "zero_reduce (fp32 gradient pull-reduce, shard of " + args.model + ")", t,
                   link_bytes=(world - 1) * n * 4,
                   note=f"shard {n} elements; also reads the local copy and writes the reduced shard to HBM")
        eng.scalars.zero_()
        eng.scalars[2] = 1.0

        def adam():
            rc = L.b200_zero_adam_gather(_lib.ptr(eng.master), _lib.ptr(eng.exp_avg), _lib.ptr(eng.exp_avg_sq),
                                         _lib.ptr(red), sy.param_ptrs, ctypes.c_void_p(0), ctypes.c_int(world),
                                         ctypes.c_longlong(lo), ctypes.c_longlong(n), _lib.ptr(eng.scalars),
                                         ctypes.c_float(1e-6), ctypes.c_float(0.9), ctypes.c_float(0.95),
                                         ctypes.c_float(1e-8), ctypes.c_float(0.0), ctypes.c_int(1), None,
                                         ctypes.c_int(0), _lib.stream_ptr())
            _lib.check_rc(rc, "zero_adam_gather")

        if on("zero_adam_gather"):
            t = timed(adam, G)
            report(rank, "zero_adam_gather (AdamW on the shard + bf16 store into every peer)", t,
                   link_bytes=(world - 1) * n * 2,
                   note="HBM traffic of the AdamW itself: 28 B per element (fp32 master / moments read + write, gradient)")
        del eng, model, sy, red
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- ZeRO-3 gathers (reshard_copy over peer slices)
    if on("zero3_gather"):
        model = TransformerLM(cfg, device=dev, seed=0, shard_world=world)
        z3 = Zero3Engine(model, group=G, train=False)
        full = torch.empty(z3.padded, dtype=torch.bfloat16, device=dev)
        t = timed(lambda: z3.gather_full(full), G)
        report(rank, "reshard_copy: ZeRO-3 slices -> full parameter copy (weight sync)", t,
               link_bytes=(world - 1) * z3.per * 2, note=f"{z3.padded * 2 / 1e9:.2f} GB written locally")

        def layer():
            z3.slot_layer = [-1, -1]
            z3.gather_layer(0)

        t = timed(layer, G)
        a, b = z3.layer_rng[0]
        report(rank, "reshard_copy: one decoder layer into its slot (ZeRO-3 forward / backward gather)", t,
               link_bytes=(b - a) * 2 * (world - 1) / world)
        del z3, model, full
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- tensor-parallel GEMMs (Llama-3-8B shapes)
    if on("tp_gemm"):
        from openrlhf_b200.parallel.tp import TPContext

        H, I, M = 4096, 14336, 256 * 8
        ctx = TPContext(G, M, H, I // world, dev)
        x = torch.randn(M, I // world, device=dev, dtype=torch.bfloat16)
        w = torch.randn(H, I // world, device=dev, dtype=torch.bfloat16) * 0.02
        t = timed(lambda: ctx.row_parallel(x, w), G)
        report(rank, f"gemm_bf16_tp row-parallel down_proj M={M} N={H} K={I}/{world} (GEMM + all-reduce push)", t,
               link_bytes=(world - 1) * M * H * 4, flops=2.0 * M * H * (I // world),
               note="includes the buffer clear and two flag barriers of the call")
        t = timed(lambda: ctx.row_parallel_scatter(x, w), G)
        report(rank, f"gemm_bf16_tp reduce-scatter down_proj M={M} N={H} K={I}/{world} (tile -> owner of its rows)", t,
               link_bytes=(world - 1) / world * M * H * 4, flops=2.0 * M * H * (I // world),
               note="includes the buffer clear and two flag barriers of the call")
        ref = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

        def lib():
            torch.matmul(x, w.t(), out=ref)
            dist.all_reduce(ref, group=G)

        t2 = timed(lib, G)
        report(rank, "same shape: library matmul + NCCL all-reduce (bf16)", t2, link_bytes=2 * (world - 1) / world * M * H * 2,
               flops=2.0 * M * H * (I // world))
        xs = torch.randn(M // world, H, device=dev, dtype=torch.bfloat16)
        wq = torch.randn(2 * I // world, H, device=dev, dtype=torch.bfloat16) * 0.02
        t = timed(lambda: ctx.column_parallel_gathered(xs, wq), G)
        report(rank, f"gemm_bf16_tp gather-A gate_up M={M} N={2 * I}/{world} K={H} (all-gather fused into the A loads)", t,
               link_bytes=(world - 1) / world * M * H * 2, flops=2.0 * M * (2 * I // world) * H)
        del ctx

    # ---------------------------------------------------------------- context-parallel attention
    if on("cp_attention"):
        from openrlhf_b200.ops.functional import rope_table
        from openrlhf_b200.parallel.cp import CPContext

        Hq, Hkv, T = 8, 2, 32768                     # one 32768-token pack; heads of one GPU's share
        T_loc = T // world
        cp = CPContext(G, T_loc, Hq, Hkv, dev)
        qkv = torch.randn(T_loc, cp.W, device=dev, dtype=torch.bfloat16)
        pos = (torch.arange(T_loc, device=dev, dtype=torch.int32) + rank * T_loc)
        tab = rope_table(128, 1e6, T, dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        with torch.no_grad():
            t = timed(lambda: cp.attention(qkv.clone(), pos, tab, cu), G)
        flops_max = 4.0 * Hq * 128 * (T_loc * (T - T_loc / 2))       # the last rank attends to the most keys
        report(rank, f"attn_fwd_cp T={T} over {world} ranks, Hq={Hq} Hkv={Hkv} (K/V gather fused into attention)", t,
               link_bytes=(world - 1) * T_loc * cp.kv_cols * 2, flops=flops_max,
               note="contiguous slices: time and FLOPs are those of the last rank; includes rope, staging copy and barrier")
        del cp

    # ---------------------------------------------------------------- expert-parallel dispatch / combine
    if on("ep"):
        from openrlhf_b200.parallel.ep import EPContext, _gather, _scatter

        Hm, E, k, T = 2048, 128, 8, 8192
        ep = EPContext(G, T, k, Hm, E, dev)
        x = torch.randn(T, Hm, device=dev, dtype=torch.bfloat16)
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)])
        dr, drow, tg, offs = ep.plan(idx)
        t = timed(lambda: _scatter(ep, x, dr, drow, None, ep.recv_ptrs), G)
        remote = (world - 1) / world
        report(rank, f"ep_scatter T={T} k={k} H={Hm} E={E} (dispatch: peer stores to final expert-sorted rows)", t,
               link_bytes=remote * T * k * Hm * 2)
        y = torch.empty_like(x)
        rows = torch.empty(T * k, Hm, dtype=x.dtype, device=dev)
        wflat = torch.rand(T * k, device=dev)
        t = timed(lambda: _gather(ep, ep.out_ptrs, dr, drow, wflat, y, rows, None, None, T), G)
        report(rank, "ep_gather (combine: weighted pull of the k expert outputs)", t, link_bytes=remote * T * k * Hm * 2)
    torch.cuda.synchronize()
    _lib.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
