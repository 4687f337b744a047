"""Run under torchrun on >= 2 GPUs: fused tensor-parallel GEMMs against a dense fp32 computation."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from openrlhf_b200.ops import _lib  # noqa: E402
from openrlhf_b200.parallel.tp import TPContext  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    rank, tp = dist.get_rank(), dist.get_world_size()
    dev = torch.device(f"cuda:{local}")
    M, K, N = 256 * tp, 1024, 768
    ctx = TPContext(None, max_rows=M, max_cols=1024, hidden=K, device=dev)
    g = torch.Generator(device=dev).manual_seed(5)          # same data on every rank
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, generator=g, device=dev)).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    ks = K // tp
    for it in range(3):                                     # several calls: exercises the double buffering
        out = ctx.row_parallel(x[:, rank * ks:(rank + 1) * ks].contiguous(), w[:, rank * ks:(rank + 1) * ks].contiguous())
        torch.cuda.synchronize()
        _lib.check_status(dev)
        err = (out - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), f"row-parallel iter {it}: err {err}"
    rows = M // tp
    for it in range(3):                                     # reduce-scatter form: this rank's rows of the same sum
        out = ctx.row_parallel_scatter(x[:, rank * ks:(rank + 1) * ks].contiguous(),
                                       w[:, rank * ks:(rank + 1) * ks].contiguous())
        torch.cuda.synchronize()
        _lib.check_status(dev)
        want = ref[rank * rows:(rank + 1) * rows]
        err = (out - want).abs().max().item()
        assert out.shape == want.shape and err <= 2e-2 * ref.abs().max().item(), f"reduce-scatter iter {it}: err {err}"
    ns = N // tp
    bias = torch.randn(ns, generator=g, device=dev).to(torch.bfloat16)
    for it in range(2):
        out = ctx.column_parallel_gathered(x[rank * rows:(rank + 1) * rows].contiguous(),
                                           w[rank * ns:(rank + 1) * ns].contiguous(), bias)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        want = ref[:, rank * ns:(rank + 1) * ns] + bias.float()
        err = (out.float() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item(), f"column-parallel iter {it}: err {err}"
    dist.barrier()
    if rank == 0:
        print(f"tp_gemm ok (tp {tp})")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
