"""A tiny Llama through Actor.forward with ring_attn_group set (context parallel over all ranks) against the same
model on one GPU: per-token log-probs and the parameter gradients after summing over the group."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from openrlhf_b200.models.actor import Actor
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.ops import _lib

    cfg = PRESETS["tiny-qwen2"]
    assert cfg.head_dim == 128
    actor = Actor("tiny-qwen2", device="cuda", seed=0)
    torch.manual_seed(1)
    B, L = 3, 400
    seqs = torch.randint(0, cfg.vocab_size, (B, L), device="cuda")
    mask = torch.ones(B, L, dtype=torch.long, device="cuda")
    mask[1, 250:] = 0
    mask[2, 130:] = 0

    def run(group):
        for p in actor.model.parameters():
            p.grad = None
        lp = actor(seqs, attention_mask=mask, ring_attn_group=group)
        w = torch.linspace(0.5, 1.5, lp.numel(), device="cuda").view_as(lp) * mask[:, 1:]
        (lp.float() * w).sum().backward()
        flat = torch.cat([p.grad.float().flatten() for p in actor.model.parameters() if p.grad is not None])
        return lp.detach().float(), flat

    lp_ref, g_ref = run(None)
    lp_cp, g_cp = run(dist.group.WORLD)
    torch.cuda.synchronize()
    _lib.check_status()
    m = mask[:, 1:].bool()
    err = (lp_cp[m] - lp_ref[m]).abs().max().item()
    print(f"rank {rank}: max |dlogp| {err:.3e}", flush=True)
    assert err < 5e-2, err
    if g_ref is not None:
        dist.all_reduce(g_cp)
        g_cp /= world          # _GatherTokens scales the local slice gradient by the group size
        rel = ((g_cp - g_ref).norm() / g_ref.norm()).item()
        print(f"rank {rank}: grad rel err {rel:.3e}", flush=True)
        assert rel < 3e-2, rel
    # reward model: value at the last token, with and without context parallelism
    from openrlhf_b200.models.model import get_llm_for_sequence_regression
    rm = get_llm_for_sequence_regression("tiny-qwen2", "reward", device="cuda", seed=0, init_value_head=True)
    with torch.no_grad():
        r_ref = rm(seqs, attention_mask=mask)
        r_cp = rm(seqs, attention_mask=mask, ring_attn_group=dist.group.WORLD)
    torch.cuda.synchronize()
    _lib.check_status()
    rerr = (r_ref.float() - r_cp.float()).abs().max().item()
    print(f"rank {rank}: reward max |diff| {rerr:.3e}", flush=True)
    assert rerr < 5e-2, rerr
    dist.barrier()
    if rank == 0:
        print("CP_MODEL_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
