"""Muon engine: Newton-Schulz against the SVD polar factor, one step against a direct restatement, and two gloo ranks
ending with identical parameters."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from openrlhf_b200.models.config import PRESETS
from openrlhf_b200.models.transformer import TransformerLM
from openrlhf_b200.parallel.muon import MuonEngine, is_muon_param, newton_schulz5


def test_newton_schulz_close_to_polar_factor():
    torch.manual_seed(0)
    for shape in ((64, 96), (128, 64)):
        g = torch.randn(*shape)
        o = newton_schulz5(g)
        s = torch.linalg.svdvals(o)
        assert s.max() < 1.3 and s.min() > 0.3          # singular values pushed towards 1 (the quintic does not converge to exactly 1)
        u, _, vh = torch.linalg.svd(g, full_matrices=False)
        cos = (o * (u @ vh)).sum() / (o.norm() * (u @ vh).norm())
        assert cos > 0.95


def _loss(model, ids):
    pos = torch.arange(ids.numel(), dtype=torch.int32)
    cu = torch.tensor([0, ids.numel()], dtype=torch.int32)
    h, _ = model(ids, pos, cu, ids.numel())
    lp, _ = model.logprobs(h, torch.roll(ids, -1))
    return -lp.float().mean()


def test_one_step_matches_restatement():
    cfg = PRESETS["tiny-llama"]
    model = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=0)
    before = {s.name: p.detach().clone() for s, p in model.named_specs()}
    eng = MuonEngine(model, muon_lr=0.02, momentum=0.9, adam_lr=1e-3, weight_decay=0.1)
    ids = torch.randint(0, cfg.vocab_size, (48,))
    eng.backward(_loss(model, ids))
    grads = {s.name: p.main_grad.clone() for s, p in model.named_specs()}
    eng.step()
    n_muon = 0
    for s, p in model.named_specs():
        g, w0 = grads[s.name], before[s.name]
        if is_muon_param(s.name, s.shape):
            n_muon += 1
            u = g + 0.9 * g                      # first step: buf = g, nesterov
            want = w0 * (1 - 0.02 * 0.1) - 0.02 * max(1.0, s.shape[0] / s.shape[1]) ** 0.5 * newton_schulz5(u)
        else:
            m, v = 0.1 * g, 0.05 * g * g
            want = (w0 * (1 - 1e-3 * 0.1) if s.decay else w0) - 1e-3 * (m / 0.1) / ((v / 0.05).sqrt() + 1e-8)
        # the Newton-Schulz iteration runs in bf16: rounding differences of its input show up at the 1e-2 level of its
        # output, i.e. lr * 1e-2 in the weights
        tol = 1e-3 if is_muon_param(s.name, s.shape) else 1e-5
        assert torch.allclose(p.detach(), want, rtol=1e-4, atol=tol), s.name
    assert n_muon == 4 * cfg.num_hidden_layers


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = PRESETS["tiny-llama"]
    model = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=0)
    eng = MuonEngine(model, muon_lr=0.02, adam_lr=1e-3)
    torch.manual_seed(rank)
    for _ in range(2):
        eng.backward(_loss(model, torch.randint(0, cfg.vocab_size, (40,))))
        eng.step()
    flat = torch.cat([p.detach().flatten() for _, p in model.named_specs()])
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    if rank == 0:
        out.put(all(torch.equal(gathered[0], t) for t in gathered[1:]) and bool(torch.isfinite(flat).all()))
    dist.destroy_process_group()


def test_two_ranks_stay_in_sync():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, 29741, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) is True
