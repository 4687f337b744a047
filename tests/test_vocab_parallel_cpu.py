"""Vocabulary-parallel fused log-prob on two gloo ranks against the single-rank op (values and gradients)."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from openrlhf_b200.ops import functional as F
    torch.manual_seed(0)
    T, H, V = 37, 16, 50
    h0 = torch.randn(T, H)
    w0 = torch.randn(V, H) * 0.3
    y = torch.randint(0, V, (T,))
    g = torch.randn(T)
    ok = True
    for temp in (1.0, 0.7):
        h, w = h0.clone().requires_grad_(), w0.clone().requires_grad_()
        lp, ent = F.fused_logprob(h, w, y, temp, True)
        (lp * g).sum().backward()
        Vl = V // world
        hl = h0.clone().requires_grad_()
        wl = w0[rank * Vl:(rank + 1) * Vl].clone().requires_grad_()
        lp2, ent2 = F.vocab_parallel_logprob(hl, wl, y, rank * Vl, dist.group.WORLD, temp, True)
        (lp2 * g).sum().backward()
        ok &= torch.allclose(lp, lp2, atol=1e-5) and torch.allclose(ent, ent2, atol=1e-5)
        ok &= torch.allclose(h.grad, hl.grad, atol=1e-5)
        ok &= torch.allclose(w.grad[rank * Vl:(rank + 1) * Vl], wl.grad, atol=1e-5)
    q.put(bool(ok))
    dist.destroy_process_group()


def test_vocab_parallel_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_main, args=(r, 2, 29743, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) and q.get(timeout=5)
