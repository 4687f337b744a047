"""Run under torchrun on >= 2 GPUs: the peer-memory optimizer step must match the NCCL reduce-scatter + AdamW +
all-gather path, and a barrier whose peer never arrives must end with an error status instead of hanging."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from openrlhf_b200.models.config import PRESETS  # noqa: E402
from openrlhf_b200.models.transformer import ALIGN, TransformerLM, build_param_specs  # noqa: E402
from openrlhf_b200.ops import _lib  # noqa: E402
from openrlhf_b200.parallel.symm import SymmBuffers  # noqa: E402
from openrlhf_b200.parallel.zero import ZeroEngine  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device(f"cuda:{local}")
    cfg = PRESETS["tiny-qwen2"]
    specs = build_param_specs(cfg)
    total = specs[-1].offset + (specs[-1].numel + ALIGN - 1) // ALIGN * ALIGN
    use_nvls = os.environ.get("OPENRLHF_B200_NVLS", "0") == "1"
    symm = SymmBuffers(None, ZeroEngine.padded_numel(total, world), dev, use_nvls=use_nvls)
    m_s = TransformerLM(cfg, device=dev, seed=7, shard_world=world, flat=symm.param)
    m_n = TransformerLM(cfg, device=dev, seed=7, shard_world=world)
    assert torch.equal(m_s.flat[:total], m_n.flat[:total])
    e_s = ZeroEngine(m_s, lr=1e-2, weight_decay=0.1, max_norm=1.0, symm=symm)
    e_n = ZeroEngine(m_n, lr=1e-2, weight_decay=0.1, max_norm=1.0)
    for step in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        grad = torch.randn(total, generator=g, device=dev) * 0.01
        e_s.grad_flat[:total].copy_(grad)
        e_n.grad_flat[:total].copy_(grad)
        e_s.step()
        e_n.step()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        a, b = m_s.flat[:total].float(), m_n.flat[:total].float()
        diff = (a - b).abs().max().item()
        gn = abs(e_s.grad_norm() - e_n.grad_norm())
        # the two paths sum the ranks in different orders: allow one bf16 ulp of the largest parameter
        assert diff <= b.abs().max().item() * 2 ** -7, f"step {step}: param diff {diff}"
        assert (a - b).abs().mean().item() <= 1e-6, "parameters drift apart on average"
        assert gn < 1e-3 * max(e_n.grad_norm(), 1e-6), f"grad norm differs by {gn}"
        assert float(e_s.grad_flat.abs().max()) == 0.0
    # every rank ends with the same full parameter buffer
    ref = m_s.flat[:total].clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, m_s.flat[:total])
    # bounded wait: rank 0 alone enters a barrier on a spare channel with a 0.5 s limit; the status word reports it
    dist.barrier()
    if rank == 0:
        symm.wait_limit_s = 0.5
        symm.epoch += 1000
        symm.barrier(channel=5)
        torch.cuda.synchronize()
        try:
            _lib.check_status(dev)
            raise AssertionError("expected a timeout status")
        except _lib.KernelError as e:
            assert "flag" in str(e)
    dist.barrier()
    if rank == 0:
        print(f"zero_symm_vs_nccl ok (world {world}, nvls {bool(symm.mc_param)})")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
