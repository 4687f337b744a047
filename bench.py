"""Headline benchmark: RL-step samples/s (and generated tokens/s, weight-sync ms) of hybrid-engine RL steps, driven
through the same worker class the launcher ``python -m openrlhf.cli.train_ppo_ray`` starts on every GPU
(``runtime.workers.RLWorker``; its SPMD subclass ``HybridRLWorker`` adds the ``rl_step`` loop that a torchrun rank
calls itself). Random-init weights, synthetic prompts (no network on the box).

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

``--config`` selects the workload (weak scaling: the per-GPU share is fixed):

* ``qwen2.5-7b-grpo`` (default): GRPO (group-normalised advantages, k3 KL loss against a reference model) on the
  Qwen2.5-7B architecture with ZeRO-3 for the policy and the reference model; 8 prompts x 512 tokens per GPU, n = 8
  responses x 1024 tokens (EOS ignored), rule reward; 512 samples per step on 8 GPUs. Every step gathers the ZeRO-3
  parameter slices into the rollout engine's copy (the weight sync) and, on more than one GPU, runs the per-layer
  gathers and gradient reductions over NVLink. Micro-batch 2 packed sequences on one GPU (which holds the whole
  optimizer state), 8 once the state is sharded.
* ``qwen2.5-1.5b-reinforce``: REINFORCE++-baseline on the Qwen2.5-1.5B architecture; every GPU runs 16 prompts x 512
  tokens, n = 8 responses x 2048 tokens, rule reward, ZeRO-2, micro-batch 4 packed sequences: 128 prompts per step on 8
  GPUs.
* ``llama3-8b-ppo``: full PPO on the Llama-3-8B architecture: actor, critic, reference and reward model, GAE
  (gamma 1, lambda 0.95), ZeRO-3 for all four, rollout engines with tensor parallelism 2, weight sync from the ZeRO-3
  slices into the tensor-parallel shards every step; 32 prompts x 1024 tokens per GPU, one response x 1024 tokens
  (256 prompts per step on 8 GPUs). Needs 8 GPUs for the memory of four 8B models.

Prints one JSON line on rank 0. `value` is device-timed (CUDA events around the K steps, max over ranks) with the
prompts already staged on the device; `e2e` times K further steps through the public API (`rl_step`) from pinned host
prompts to the host-side loss, with a wall clock around a synchronize (fewer than K steps, at least two, when K
more would overrun ``BENCH_TIME_BUDGET_S``; ``e2e.steps`` says how many). After the default config, when time allows
(``BENCH_TIME_BUDGET_S``), the other configs that fit the GPU count run for one short measurement each in child
processes and are attached under ``extra_configs``.
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

T_START = time.time()

CONFIGS = {
    "qwen2.5-1.5b-reinforce": dict(model="qwen2.5-1.5b", prompts_per_gpu=16, prompt_len=512, n_samples=8, max_new=2048,
                                   micro=4, estimator="reinforce_baseline", kl=0.0, zero_stage=2, rollout_tp=1,
                                   critic=False, reward_model=False, min_gpus=1,
                                   metric="RL-step samples/s (REINFORCE++-baseline hybrid engine, generation + "
                                          "experience + train + weight sync)"),
    "qwen2.5-7b-grpo": dict(model="qwen2.5-7b", prompts_per_gpu=8, prompt_len=512, n_samples=8, max_new=1024, micro=2,
                            micro_sharded=8,     # micro-batch once the ZeRO-3 state is sharded (N >= 2): fewer gathers
                            estimator="group_norm", kl=0.001, kl_loss=True, zero_stage=3, rollout_tp=1, critic=False,
                            reward_model=False, min_gpus=1,
                            metric="RL-step samples/s (GRPO hybrid engine, ZeRO-3 policy + reference, generation + "
                                   "experience + train + weight sync)"),
    "llama3-8b-ppo": dict(model="llama3-8b", prompts_per_gpu=32, prompt_len=1024, n_samples=1, max_new=1024, micro=4,
                          estimator="gae", kl=0.01, zero_stage=3, rollout_tp=2, critic=True, reward_model=True,
                          min_gpus=8,
                          metric="RL-step samples/s (PPO with critic, reward and reference models, ZeRO-3, rollout "
                                 "TP2, generation + experience + train + weight sync)"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="qwen2.5-7b-grpo", choices=sorted(CONFIGS))
    ap.add_argument("--model", default=None, help="override the architecture preset of the config")
    ap.add_argument("--layers", type=int, default=None, help="cut the layer count (functional tests on few GPUs)")
    ap.add_argument("--prompts-per-gpu", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--n-samples", type=int, default=None)
    ap.add_argument("--max-new", type=int, default=None)
    ap.add_argument("--micro", type=int, default=None)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--zero-stage", type=int, default=None, choices=[1, 2, 3])
    ap.add_argument("--rollout-tp", type=int, default=None, help="tensor-parallel size of the rollout engines")
    ap.add_argument("--extras", default="auto", choices=["auto", "none"],
                    help="auto: after the default config, measure the other configs in child processes if time allows")
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


def resolve(args) -> dict:
    c = dict(CONFIGS[args.config])
    for k, flag in (("model", args.model), ("prompts_per_gpu", args.prompts_per_gpu), ("prompt_len", args.prompt_len),
                    ("n_samples", args.n_samples), ("max_new", args.max_new), ("micro", args.micro),
                    ("zero_stage", args.zero_stage), ("rollout_tp", args.rollout_tp)):
        if flag is not None:
            c[k] = flag
    return c


def run_extras(args, world: int, rank: int) -> dict:
    """The configs other than the one just measured, one short run each in a child process per rank (a fresh CUDA
    context; a failure or an overrun there cannot take the headline number with it). Skipped when the time budget of
    the whole bench (BENCH_TIME_BUDGET_S, default 830 s) does not leave room."""
    budget = float(os.environ.get("BENCH_TIME_BUDGET_S", "830"))
    est = {"qwen2.5-7b-grpo": 150.0, "llama3-8b-ppo": 110.0, "qwen2.5-1.5b-reinforce": 100.0}
    out = {}
    port0 = int(os.environ.get("MASTER_PORT", "29500"))
    for k, name in enumerate(n for n in ("llama3-8b-ppo", "qwen2.5-1.5b-reinforce", "qwen2.5-7b-grpo")
                             if n != args.config):
        if world < CONFIGS[name]["min_gpus"]:
            out[name] = {"skipped": f"needs {CONFIGS[name]['min_gpus']} GPUs"}
            continue
        left = budget - (time.time() - T_START)
        if left < est[name] + 25:
            out[name] = {"skipped": f"time budget: {left:.0f} s left, about {est[name]:.0f} s needed"}
            continue
        env = dict(os.environ, MASTER_PORT=str(port0 + 17 + k), NCCL_NVLS_ENABLE="0")
        cmd = [sys.executable, os.path.abspath(__file__), "--config", name, "--gpus", str(world), "--steps", "1",
               "--warmup", "1", "--extras", "none"]
        try:
            r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=left - 15)
            line = next((ln for ln in reversed(r.stdout.splitlines()) if ln.startswith("{")), None)
            if rank == 0:
                if r.returncode == 0 and line:
                    d = json.loads(line)
                    out[name] = {k2: d[k2] for k2 in ("metric", "value", "unit", "ms_per_step", "gen_tokens_per_s",
                                                     "weight_sync_ms", "phase_s_per_step", "config", "e2e",
                                                     "steps", "warmup") if k2 in d}
                else:
                    out[name] = {"error": (r.stderr or r.stdout)[-400:]}
        except subprocess.TimeoutExpired:
            out[name] = {"error": "did not finish inside the time budget"}
    return out


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
    if world > 1:
        import datetime

        # a rank that fails must not leave the others waiting for NCCL's default 10 minutes
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"),
                                timeout=datetime.timedelta(seconds=int(os.environ.get("BENCH_NCCL_TIMEOUT_S", "240"))))
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.trainer.hybrid_engine import HybridRLWorker, default_rl_args

    c = resolve(args)
    if world < c["min_gpus"] and args.layers is None and args.model is None:
        if rank == 0:
            print(json.dumps({"impl": "b200", "config": args.config,
                              "unavailable": f"this config needs {c['min_gpus']} GPUs (four 8B models under ZeRO-3)"}))
        return 0
    P, L, n, new = c["prompts_per_gpu"], c["prompt_len"], c["n_samples"], c["max_new"]
    if world > 1 and args.micro is None and "micro_sharded" in c:
        # one GPU holds the whole optimizer state and has room for small micro-batches only; the work per GPU and per
        # optimizer step is the same, only the number of forward / backward passes it is cut into differs
        c["micro"] = c["micro_sharded"]
    model = c["model"]
    if args.layers is not None:
        import dataclasses

        model = dataclasses.replace(PRESETS[model], num_hidden_layers=args.layers)
    tp = c["rollout_tp"] if world >= c["rollout_tp"] else 1
    rl_args = default_rl_args(**{
        "rollout.n_samples_per_prompt": n, "rollout.max_new_tokens": new, "rollout.micro_batch_size": 8,
        "train.micro_batch_size": c["micro"], "train.batch_size": 16 * world,
        "data.max_len": L + new, "algo.advantage.estimator": c["estimator"], "algo.kl.init_coef": c["kl"],
        "algo.kl.use_loss": bool(c.get("kl_loss", False)), "algo.kl.estimator": "k3" if c.get("kl_loss") else "k1",
        "algo.advantage.lambd": 0.95, "algo.advantage.gamma": 1.0, "ds.zero_stage": c["zero_stage"],
        "vllm.tensor_parallel_size": tp, "rollout.ignore_eos": True,
    })

    def rule_reward(exps):
        # (sum of response token ids) mod 7 == 0
        return [float(int(e.sequences[L:].sum()) % 7 == 0) for e in exps]

    seqs = P * n
    worker = HybridRLWorker(model, rl_args, device=f"cuda:{local}", reward_fn=None if c["reward_model"] else rule_reward,
                            seed=0, max_num_seqs=seqs * tp, with_critic=c["critic"],
                            num_pages=(seqs * ((L + new) // 128 + 1) + P * (L // 128) + 8) * tp,
                            use_cuda_graph=not args.no_graph,
                            reward_model_path=(model if isinstance(model, str) else worker_name(model)) if c["reward_model"] else None)
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
    # as many steps as the device-timed region, unless the time budget of the whole run would be exceeded (slow
    # configs under a long --steps): then fewer, at least two, the same number on every rank
    budget = float(os.environ.get("BENCH_TIME_BUDGET_S", "830"))
    fit = int((budget - (time.time() - T_START) - 15.0) / max(dev_s / args.steps, 1e-3))
    e2e_steps = torch.tensor([max(min(2, args.steps), min(args.steps, fit))], device=f"cuda:{local}")
    if world > 1:
        dist.broadcast(e2e_steps, 0)
    e2e_steps = int(e2e_steps)
    barrier()
    t0 = time.perf_counter()
    d2h = 0
    for _ in range(e2e_steps):
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
    out = None
    if rank == 0:
        value = samples / dev_s
        opt = ("zero-3: peer-memory layer gathers and per-layer gradient reductions" if worker.zero3 else
               "peer-memory reduce + AdamW + parameter-store kernels" if worker.symm is not None else
               ("nccl" if world > 1 else "local"))
        gen_s = phases.get("timing/generation", 0.0)
        out = {
            "metric": c["metric"], "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic prompts (uniform token ids), random-init weights",
            # generated tokens over the whole step time (the headline's companion), and over the generation phase alone
            "gen_tokens_per_s": gen_tokens * world / dev_s,
            "gen_phase_tokens_per_s": gen_tokens * world / gen_s if gen_s > 0 else None,
            "weight_sync_ms": phases.get("timing/broadcast", 0.0) / args.steps * 1e3,
            "phase_s_per_step": {k: v / args.steps for k, v in phases.items()},
            "config": {"name": args.config, "model": c["model"] if args.layers is None else f"{c['model']} cut to {args.layers} layers",
                       "global_batch": P * n * world, "seq_len": L + new, "prompts_per_gpu": P, "prompt_len": L,
                       "n_samples_per_prompt": n, "max_new_tokens": new, "estimator": c["estimator"],
                       "kl_coef": c["kl"], "critic": c["critic"], "reward": "model" if c["reward_model"] else "rule",
                       "zero_stage": c["zero_stage"], "micro_batch": c["micro"],
                       "parallelism": f"dp{world}" + (f", rollout tp{tp} x {world // tp}" if tp > 1 else ""),
                       "optimizer_step": opt, "worker": "runtime.workers.RLWorker (SPMD subclass HybridRLWorker)",
                       "l2": "working set (weights + KV cache) is larger than L2"},
            "clocks": clocks,
            "e2e": {"value": P * n * world * e2e_steps / e2e_s, "unit": "samples/s", "steps": e2e_steps,
                    "h2d_bytes_per_step": P * L * 8, "d2h_bytes_per_step": d2h // e2e_steps},
            "gpu_launches": launches,
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(local) / 2 ** 30, 1),     # rank 0's allocator peak
            "impl": "b200",
        }
    # ---- release the GPU before the optional child runs
    if args.extras == "auto" and args.config == "qwen2.5-7b-grpo" and args.layers is None and args.model is None:
        try:
            worker.rollout.sleep()
        except Exception:  # noqa: BLE001
            pass
        del worker, staged
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        extras = run_extras(args, world, rank)
        if out is not None:
            out["extra_configs"] = extras
    elif world > 1:
        dist.destroy_process_group()
    if out is not None:
        print(json.dumps(out))
    return 0


def worker_name(cfg) -> str:
    """Preset name under which a modified ModelConfig is registered (reward model of a cut-down config)."""
    from openrlhf_b200.models.config import PRESETS

    name = f"_config_{id(cfg)}"
    PRESETS[name] = cfg
    return name


if __name__ == "__main__":
    sys.exit(main())
