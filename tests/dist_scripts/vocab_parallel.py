"""Vocabulary-parallel fused log-prob on N GPUs against the single-GPU fused op (values, entropy, gradients)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from openrlhf_b200.ops import _lib, functional as F

    torch.manual_seed(0)
    T, H, V = 1000, 256, 4096
    h0 = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16)
    w0 = (torch.randn(V, H, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.randint(0, V, (T,), device="cuda")
    g = torch.randn(T, device="cuda")
    Vl = V // world
    for temp in (1.0, 0.8):
        h, w = h0.clone().requires_grad_(), w0.clone().requires_grad_()
        lp, ent = F.fused_logprob(h, w, y, temp, True, chunk=256)
        (lp * g).sum().backward()
        hl = h0.clone().requires_grad_()
        wl = w0[rank * Vl:(rank + 1) * Vl].clone().requires_grad_()
        lp2, ent2 = F.vocab_parallel_logprob(hl, wl, y, rank * Vl, dist.group.WORLD, temp, True, chunk=256)
        (lp2 * g).sum().backward()
        torch.cuda.synchronize()
        _lib.check_status()
        rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()
        e = (rel(lp2, lp), rel(ent2, ent), rel(hl.grad, h.grad), rel(wl.grad, w.grad[rank * Vl:(rank + 1) * Vl]))
        print(f"rank {rank} temp {temp}: logp {e[0]:.2e} ent {e[1]:.2e} dh {e[2]:.2e} dw {e[3]:.2e}", flush=True)
        assert e[0] < 1e-3 and e[1] < 1e-3 and e[2] < 2e-2 and e[3] < 2e-2, e
    dist.barrier()
    if rank == 0:
        print("VOCAB_PARALLEL_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
