"""Context-parallel attention on N GPUs against single-GPU attention over the whole packed stream.

Launched by tests/test_multigpu.py through torch.distributed.run. Every rank computes the full-stream reference
locally (own kernels, already checked against PyTorch fp32 elsewhere) and compares its slice of output and dqkv.
"""
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from openrlhf_b200.models.packing import cp_slice, pack_lists_cp
    from openrlhf_b200.ops import _lib, functional as F
    from openrlhf_b200.ops.attention import rope_attention
    from openrlhf_b200.parallel.cp import CPContext

    for Hq, Hkv, lens in ((4, 2, [300, 77, 500, 130]), (5, 1, [700, 129, 5, 256, 900])):
        torch.manual_seed(0)
        D = 128
        W = (Hq + 2 * Hkv) * D
        seqs = [torch.randint(0, 1000, (n,)) for n in lens]
        pb, valid = pack_lists_cp(seqs, world, device="cuda")
        T = pb.input_ids.numel()
        T_loc = T // world
        x = torch.randn(T, W, device="cuda", dtype=torch.bfloat16)
        g = torch.randn(T, Hq * D, device="cuda", dtype=torch.bfloat16)
        table = F.rope_table(D, 10000.0, 2048, "cuda")
        scale = 1 / math.sqrt(D)
        # reference: whole stream on this GPU
        xr = x.clone().requires_grad_()
        ref = rope_attention(xr * 1.0, pb.position_ids, table, pb.cu_seqlens, Hq, Hkv, scale)
        ref.backward(g)
        # context parallel: this rank's rows
        cp = CPContext(None, T_loc, Hq, Hkv, "cuda")
        lo, hi = rank * T_loc, (rank + 1) * T_loc
        _, _, pos_loc = cp_slice(pb, rank, world)
        xl = x[lo:hi].clone().requires_grad_()
        out = cp.attention(xl * 1.0, pos_loc, table, pb.cu_seqlens, scale)
        out.backward(g[lo:hi])
        torch.cuda.synchronize()
        _lib.check_status()

        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()

        e_out = rel(out, ref[lo:hi])
        e_dq = rel(xl.grad[:, : Hq * D], xr.grad[lo:hi, : Hq * D])
        e_dkv = rel(xl.grad[:, Hq * D:], xr.grad[lo:hi, Hq * D:])
        print(f"rank {rank} Hq{Hq} Hkv{Hkv} T{T}: out {e_out:.2e} dq {e_dq:.2e} dkv {e_dkv:.2e}", flush=True)
        assert e_out < 1e-2 and e_dq < 2e-2 and e_dkv < 2e-2, (e_out, e_dq, e_dkv)
        dist.barrier()
    if rank == 0:
        print("CP_ATTENTION_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
