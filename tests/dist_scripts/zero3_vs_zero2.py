"""ZeRO-3 engine (peer-memory parameter gathers and per-layer gradient reductions) against the ZeRO-2 engine (NCCL) on
N GPUs: same data, two optimizer steps with accumulation, parameters compared after gathering."""
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
    from openrlhf_b200.models.packing import pack_lists
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.parallel.zero import ZeroEngine
    from openrlhf_b200.parallel.zero3 import Zero3Engine

    cfg = PRESETS["tiny-qwen2"]
    g = torch.Generator().manual_seed(100 + rank)
    data = [[torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (300, 140)] for _ in range(4)]

    def loss_of(model, seqs):
        pb = pack_lists(seqs, device="cuda")
        h, _ = model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        lp, _ = model.logprobs(h, pb.labels)
        return -lp.float().mean()

    res = {}
    for kind, ckpt in (("z2", False), ("z3", False), ("z3", True)):
        model = TransformerLM(cfg, device="cuda", seed=0, shard_world=world)
        model.train()
        model.gradient_checkpointing = ckpt
        eng = (ZeroEngine(model, lr=1e-3, zero_stage=2) if kind == "z2" else Zero3Engine(model, lr=1e-3))
        losses = []
        for step in range(2):
            for j in range(2):
                l = loss_of(model, data[2 * step + j]) / 2
                losses.append(float(l))
                eng.backward(l)
            eng.step()
        torch.cuda.synchronize()
        _lib.check_status()
        full = model.flat[: model.total_numel].float().clone() if kind == "z2" else eng.gather_full().float()
        res[(kind, ckpt)] = (full, losses, eng.grad_norm())
    ref, ref_losses, ref_norm = res[("z2", False)]
    for key in (("z3", False), ("z3", True)):
        full, losses, norm = res[key]
        full = full[: ref.numel()]
        rel = ((full - ref).norm() / ref.norm()).item()
        # updates are lr-sized (1e-3 per step) on weights of size ~2e-2: compare the update, not the weight
        base = TransformerLM(cfg, device="cuda", seed=0).flat[: ref.numel()].float()
        upd_rel = ((full - ref).norm() / (ref - base).norm().clamp_min(1e-9)).item()
        print(f"rank {rank} {key}: weight rel {rel:.2e}, update rel {upd_rel:.2e}, losses {losses[:2]} vs {ref_losses[:2]}, "
              f"grad norm {norm:.4f} vs {ref_norm:.4f}", flush=True)
        assert abs(losses[0] - ref_losses[0]) < 1e-3 and upd_rel < 0.2 and abs(norm - ref_norm) < 0.05 * ref_norm, key
    # ---- mixture-of-experts model: ZeRO-3 sharding combined with expert-parallel compute against plain ZeRO-2
    from openrlhf_b200.parallel.ep import EPContext
    mcfg = PRESETS["tiny-qwen3-moe"]
    mdata = [[torch.randint(0, mcfg.vocab_size, (n,), generator=g) for n in (200, 90)] for _ in range(2)]
    outs = {}
    for kind in ("z2", "z3ep"):
        model = TransformerLM(mcfg, device="cuda", seed=0, shard_world=world, init_std=0.05)
        model.train()
        E_loc = mcfg.num_experts // world
        eng = (ZeroEngine(model, lr=1e-3, zero_stage=2) if kind == "z2"
               else Zero3Engine(model, lr=1e-3, expert_range=(rank * E_loc, (rank + 1) * E_loc)))
        if kind == "z3ep":
            model.ep = EPContext(None, 512, mcfg.num_experts_per_tok, mcfg.hidden_size, mcfg.num_experts, "cuda")
        for j in range(2):
            eng.backward(loss_of(model, mdata[j]) / 2)
        eng.step()
        torch.cuda.synchronize()
        _lib.check_status()
        outs[kind] = (model.flat[: model.total_numel].float().clone() if kind == "z2" else eng.gather_full().float(),
                      eng.grad_norm())
    ref, full = outs["z2"][0], outs["z3ep"][0][: outs["z2"][0].numel()]
    base = TransformerLM(mcfg, device="cuda", seed=0, init_std=0.05).flat[: ref.numel()].float()
    upd_rel = ((full - ref).norm() / (ref - base).norm().clamp_min(1e-9)).item()
    print(f"rank {rank} moe z3+ep: update rel {upd_rel:.2e}, grad norm {outs['z3ep'][1]:.4f} vs {outs['z2'][1]:.4f}", flush=True)
    assert upd_rel < 0.25 and abs(outs["z3ep"][1] - outs["z2"][1]) < 0.05 * outs["z2"][1]
    dist.barrier()
    if rank == 0:
        print("ZERO3_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
