"""Headline benchmark: RL-step samples/s (and generated tokens/s) of a hybrid-engine REINFORCE++-baseline step on the
Qwen2.5-1.5B architecture, the second config of BASELINE.json, weak-scaled: every GPU runs 16 prompts x 512 tokens,
n = 8 responses x 2048 tokens (EOS ignored), rule reward, ZeRO-2, micro-batch 4 packed sequences, i.e. 128 prompts
per step on 8 GPUs as the config names. Random-init weights, synthetic prompts (no network on the box).

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Prints one JSON line on rank 0. `value` is device-timed (CUDA events around the K steps, max over ranks) with the
prompts already staged on the device; `e2e` times K further steps through the public API
(`HybridRLWorker.rl_step`) from pinned host prompts to the host-side loss, with a wall clock around a synchronize.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--n-samples", type=int, default=8)
    ap.add_argument("--max-new", type=int, default=2048)
    ap.add_argument("--micro", type=int, default=4)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--zero-stage", type=int, default=2, choices=[1, 2, 3])
    ap.add_argument("--rollout-tp", type=int, default=1, help="tensor-parallel size of the rollout engines (N > 1)")
    return ap.parse_args()


def reference_arm(args):
    # The reference's stock path (python -m openrlhf.cli.train_ppo_ray) imports ray and deepspeed at module load;
    # neither is installed in this image nor present in the offline wheelhouse, so it cannot start.
    why = None
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
    try:
        import importlib

        for mod in ("ray", "deepspeed"):
            importlib.import_module(mod)
        why = "reference installed but its launcher needs a Ray cluster runtime that this harness does not start"
    except Exception as e:  # noqa: BLE001
        why = f"reference's stock code path cannot import its engines: {type(e).__name__}: {e}"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    def __init__(self, index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200",
                                       "-i", str(index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import datetime

        # a rank that fails must not leave the others waiting for NCCL's default 10 minutes
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"),
                                timeout=datetime.timedelta(seconds=int(os.environ.get("BENCH_NCCL_TIMEOUT_S", "240"))))
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.trainer.hybrid_engine import HybridRLWorker, default_rl_args

    P, L, n, new = args.prompts_per_gpu, args.prompt_len, args.n_samples, args.max_new
    rl_args = default_rl_args(**{
        "rollout.n_samples_per_prompt": n, "rollout.max_new_tokens": new, "rollout.micro_batch_size": 8,
        "train.micro_batch_size": args.micro, "train.batch_size": 16 * world, "data.max_len": L + new,
        "algo.advantage.estimator": "reinforce_baseline", "algo.kl.init_coef": 0.0, "ds.zero_stage": args.zero_stage,
    })
    rl_args.rollout.ignore_eos = True
    if args.rollout_tp > 1:
        from types import SimpleNamespace

        rl_args.vllm = SimpleNamespace(tensor_parallel_size=args.rollout_tp)

    def rule_reward(exps):
        # (sum of response token ids) mod 7 == 0
        return [float(int(e.sequences[L:].sum()) % 7 == 0) for e in exps]

    worker = HybridRLWorker(args.model, rl_args, device=f"cuda:{local}", reward_fn=rule_reward, seed=0, group=group,
                            max_num_seqs=P * n, num_pages=P * n * ((L + new) // 128 + 1) + P * (L // 128) + 8,
                            use_cuda_graph=not args.no_graph,
                            use_symm=world > 1 and args.zero_stage != 3 and os.environ.get("OPENRLHF_B200_SYMM", "1") == "1")
    vocab = worker.cfg.vocab_size
    g = torch.Generator().manual_seed(1234 + rank)
    total_steps = args.warmup + 2 * args.steps
    host_prompts = [torch.randint(0, vocab, (P, L), generator=g, dtype=torch.int64).pin_memory()
                    for _ in range(total_steps)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def note(msg):
        if os.environ.get("BENCH_VERBOSE", "0") == "1":
            print(f"[bench rank {rank}] {time.strftime('%H:%M:%S')} {msg}", file=sys.stderr, flush=True)

    note("worker built")
    it = iter(host_prompts)
    for i in range(args.warmup):
        worker.rl_step(next(it))
        note(f"warm-up step {i} done")
    # ---- device-timed region: prompts pre-staged on the device
    staged = [next(it).to(f"cuda:{local}") for _ in range(args.steps)]
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = _lib.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    gen_tokens = 0.0
    phases = {}
    for x in staged:
        st = worker.rl_step(x)
        gen_tokens += st["gen_tokens"]
        for k, v in st.items():
            if k.startswith("timing/"):
                phases[k] = phases.get(k, 0.0) + v
    e1.record()
    barrier()
    launches = _lib.LAUNCHES - launches0
    dev_s = e0.elapsed_time(e1) / 1e3
    # ---- end-to-end region: pinned host prompts in, host-side loss out, wall clock
    barrier()
    t0 = time.perf_counter()
    d2h = 0
    for _ in range(args.steps):
        st = worker.rl_step(next(it))
        loss = float(st["policy_loss"])  # host-side result of the step
        d2h += 8 * P * n * new + 4 * P * n * new + 4
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([dev_s, e2e_s], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_s, e2e_s = float(t[0]), float(t[1])
    samples = P * n * world * args.steps
    if rank == 0:
        value = samples / dev_s
        out = {
            "metric": "RL-step samples/s (REINFORCE++-baseline hybrid engine, generation + experience + train + weight sync)",
            "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic prompts (uniform token ids), random-init weights",
            "gen_tokens_per_s": gen_tokens * world / dev_s,
            "phase_s_per_step": {k: v / args.steps for k, v in phases.items()},
            "config": {"model": args.model, "global_batch": P * n * world, "seq_len": L + new,
                       "prompts_per_gpu": P, "prompt_len": L, "n_samples_per_prompt": n, "max_new_tokens": new,
                       "estimator": "reinforce_baseline", "zero_stage": args.zero_stage, "micro_batch": args.micro,
                       "parallelism": f"dp{world}" + (f", rollout tp{args.rollout_tp}" if args.rollout_tp > 1 else ""), "optimizer_step": ("zero-3 peer-memory gathers and per-layer reductions" if getattr(worker, "zero3", False) else "peer-memory kernels" if worker.symm is not None else ("nccl" if world > 1 else "local")), "l2": "working set (3 GB weights + KV cache) is larger than L2"},
            "clocks": clocks,
            "e2e": {"value": samples / e2e_s, "unit": "samples/s", "h2d_bytes_per_step": P * L * 8,
                    "d2h_bytes_per_step": d2h // args.steps},
            "gpu_launches": launches,
            "impl": "b200",
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
