"""RL steps of the hybrid worker on N GPUs in its non-default modes: ZeRO-3 actor (sharded parameters, rollout copy
refreshed by the gather kernel), tensor-parallel rollout engines (weights re-sliced by the copy plan), and both at once
with a critic, a reference model and a reward model (every model sharded; the tensor-parallel shards are filled
straight from the ZeRO-3 slices of their owners)."""
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.trainer.hybrid_engine import HybridRLWorker, default_rl_args

    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], num_attention_heads=4, num_key_value_heads=2, hidden_size=512,
                              intermediate_size=1024, num_hidden_layers=3, head_dim=128)
    from openrlhf_b200.models.config import PRESETS as _P

    _P["_hybrid_modes_cfg"] = cfg
    for mode in ("zero3", "rollout_tp", "ppo_zero3_tp"):
        full = mode == "ppo_zero3_tp"
        args = default_rl_args(**{"rollout.n_samples_per_prompt": 2, "rollout.max_new_tokens": 8,
                                  "train.micro_batch_size": 2, "train.batch_size": 4 * world, "data.max_len": 64,
                                  "algo.advantage.estimator": "gae" if full else "reinforce_baseline",
                                  "algo.kl.init_coef": 0.01 if full else 0.0,
                                  "ds.zero_stage": 2 if mode == "rollout_tp" else 3,
                                  "vllm.tensor_parallel_size": 1 if mode == "zero3" else world})
        args.rollout.ignore_eos = True
        w = HybridRLWorker(cfg, args, device="cuda", seed=0, max_num_seqs=8, num_pages=32,
                           reward_model_path="_hybrid_modes_cfg" if full else None,
                           reward_fn=None if full else (lambda exps: [float(int(e.sequences.sum()) % 2) for e in exps]))
        if full:
            assert w.critic is not None and w.ref is not None and w.reward is not None
            assert all(getattr(m.model, "z3", None) is not None for m in (w.actor, w.critic, w.ref, w.reward))
        g = torch.Generator().manual_seed(10 + rank)
        z3 = mode != "rollout_tp"
        before = w.engine.gather_full().float().clone() if z3 else w.model.flat.float().clone()
        for _ in range(2):
            prompts = [torch.randint(3, cfg.vocab_size, (12,), generator=g).tolist() for _ in range(2)]
            st = w.rl_step(prompts)
        torch.cuda.synchronize()
        _lib.check_status()
        after = w.engine.gather_full().float() if z3 else w.model.flat.float()
        moved = (after[: before.numel()] - before).abs().max().item()
        assert st["num_samples"] == 4 and all(torch.isfinite(torch.tensor(float(st[k]))) for k in ("policy_loss", "actor_grad_norm"))
        assert moved > 0, "parameters did not change"
        if mode == "zero3":   # the rollout copy follows the trainer's slices
            diff = (w.rollout_model.flat[: before.numel()].float() - after[: before.numel()]).abs().max().item()
            assert diff == 0.0, diff
        if full:              # the tensor-parallel shard equals the slice of the gathered parameters it stands for
            from openrlhf_b200.parallel.reshard import build_plan, run_plan_reference
            entries, size = build_plan(cfg, dist.get_rank(w.tp_group), world)
            want = torch.zeros(size, dtype=after.dtype, device="cpu")
            run_plan_reference(entries, [after.cpu()], want)
            got = w.rollout_model.flat[:size].float().cpu()
            assert torch.equal(got, want), (got - want).abs().max()
            assert "critic_loss" in st
        print(f"rank {rank} {mode}: policy_loss {st['policy_loss']:.4f} grad_norm {st['actor_grad_norm']:.4f} moved {moved:.2e}",
              flush=True)
        dist.barrier()
    if rank == 0:
        print("HYBRID_MODES_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
