"""Expert-parallel MoE block on N GPUs against the single-GPU grouped block with all experts (same tokens per rank
differ; every rank checks its own tokens, and expert weight gradients are compared after summing over ranks)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from openrlhf_b200.models import moe
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.parallel.ep import EPContext

    T, H, I, E, k = 700, 256, 128, 8, 2
    E_loc = E // world
    torch.manual_seed(0)                                   # same weights everywhere
    rw = (torch.randn(E, H, device="cuda") * 0.1).to(torch.bfloat16)
    gu = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16)
    xs = [(torch.randn(T - 50 * r, H, device="cuda") * 0.5).to(torch.bfloat16) for r in range(world)]  # per-rank tokens
    gs = [torch.randn(T - 50 * r, H, device="cuda").to(torch.bfloat16) for r in range(world)]
    ep = EPContext(None, T, k, H, E, "cuda")
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()

    for it in range(2):                                    # twice: buffers and barriers are reused
        # reference on this GPU: every rank's tokens through all experts
        ref_y, ref_dx, ref_dw = [], [], []
        gu_r, dn_r = gu.clone().requires_grad_(), dn.clone().requires_grad_()
        for r in range(world):
            x = xs[r].clone().requires_grad_()
            rwr = rw.clone().requires_grad_()
            y, _ = moe.moe_forward_grouped(x, rwr, gu_r, dn_r, k, True)
            (y.float() * gs[r].float()).sum().backward()
            ref_y.append(y.detach()); ref_dx.append(x.grad); ref_dw.append(rwr.grad)
        # expert parallel
        x = xs[rank].clone().requires_grad_()
        rwl = rw.clone().requires_grad_()
        gul = gu[rank * E_loc:(rank + 1) * E_loc].clone().requires_grad_()
        dnl = dn[rank * E_loc:(rank + 1) * E_loc].clone().requires_grad_()
        w, idx, _ = moe.router_topk(x, rwl, k, True)
        y = ep.moe(x, w, idx, gul, dnl)
        (y.float() * gs[rank].float()).sum().backward()
        torch.cuda.synchronize()
        _lib.check_status()
        e = (rel(y, ref_y[rank]), rel(x.grad, ref_dx[rank]), rel(rwl.grad, ref_dw[rank]),
             rel(gul.grad, gu_r.grad[rank * E_loc:(rank + 1) * E_loc]),
             rel(dnl.grad, dn_r.grad[rank * E_loc:(rank + 1) * E_loc]))
        print(f"rank {rank} it {it}: y {e[0]:.2e} dx {e[1]:.2e} drouter {e[2]:.2e} dgate_up {e[3]:.2e} ddown {e[4]:.2e}",
              flush=True)
        assert max(e) < 3e-2, e
        dist.barrier()
    if rank == 0:
        print("EP_MOE_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
