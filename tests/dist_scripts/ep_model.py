"""tiny Qwen3-MoE with expert-parallel MoE layers on N GPUs against the same model without expert parallelism
(each rank runs its own tokens; log-probs and the gradient summed over ranks are compared)."""
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
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.parallel.ep import EPContext

    actor = Actor("tiny-qwen3-moe", device="cuda", seed=0)
    cfg = actor.cfg
    torch.manual_seed(100 + rank)
    B, L = 2, 200
    seqs = torch.randint(0, cfg.vocab_size, (B, L), device="cuda")
    mask = torch.ones(B, L, dtype=torch.long, device="cuda")

    def run(ep):
        for p in actor.model.parameters():
            p.grad = None
        actor.model.ep = ep
        lp = actor(seqs, attention_mask=mask)
        lp.float().sum().backward()
        actor.model.ep = None
        g = torch.cat([p.grad.float().flatten() if p.grad is not None else torch.zeros(p.numel(), device="cuda")
                       for p in actor.model.parameters()])
        return lp.detach().float(), g

    lp_ref, g_ref = run(None)
    ep = EPContext(None, B * L, cfg.num_experts_per_tok, cfg.hidden_size, cfg.num_experts, "cuda")
    lp_ep, g_ep = run(ep)
    torch.cuda.synchronize()
    _lib.check_status()
    err = (lp_ep - lp_ref).abs().max().item()
    dist.all_reduce(g_ref)
    dist.all_reduce(g_ep)
    rel = ((g_ep - g_ref).norm() / g_ref.norm()).item()
    print(f"rank {rank}: max |dlogp| {err:.3e}, summed-grad rel err {rel:.3e}", flush=True)
    assert err < 5e-2 and rel < 3e-2, (err, rel)
    dist.barrier()
    if rank == 0:
        print("EP_MODEL_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
