"""ZeRO-3 engine (sharded parameters, rotating or persistent layer slots, per-layer gradient reduction) against the
ZeRO-2 engine on the same data: identical parameters after two optimizer steps with gradient accumulation. Two gloo
ranks, and one rank."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from openrlhf_b200.models.config import PRESETS
from openrlhf_b200.models.transformer import TransformerLM


def _loss(model, ids):
    pos = torch.arange(ids.numel(), dtype=torch.int32)
    cu = torch.tensor([0, ids.numel()], dtype=torch.int32)
    h, _ = model(ids, pos, cu, ids.numel())
    lp, _ = model.logprobs(h, torch.roll(ids, -1))
    return -lp.float().mean()


def _run(rank, world, ckpt):
    from openrlhf_b200.parallel.zero import ZeroEngine
    from openrlhf_b200.parallel.zero3 import Zero3Engine
    cfg = PRESETS["tiny-llama"]
    data = [torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(10 * rank + j))
            for j in range(4)]
    outs = []
    for kind in ("z2", "z3"):
        model = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=0, shard_world=world)
        model.gradient_checkpointing = ckpt
        model.train()
        eng = (ZeroEngine(model, lr=1e-2, weight_decay=0.1, zero_stage=2) if kind == "z2"
               else Zero3Engine(model, lr=1e-2, weight_decay=0.1))
        for step in range(2):
            for j in range(2):
                eng.backward(_loss(model, data[2 * step + j]) / 2)
            eng.step()
        n = model.total_numel if kind == "z2" else None
        flat = model.flat[: model.total_numel].clone() if kind == "z2" else None
        if kind == "z3":
            flat = eng.gather_full()
        outs.append((flat, eng.grad_norm()))
    total = outs[0][0].numel()
    return outs[0][0], outs[1][0][:total], outs[0][1], outs[1][1]


def _rank_main(rank, world, port, q, ckpt):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a, b, na, nb = _run(rank, world, ckpt)
    q.put((bool(torch.allclose(a, b, rtol=1e-4, atol=5e-5)), float((a - b).abs().max()), na, nb))
    dist.destroy_process_group()


@pytest.mark.parametrize("ckpt,persist", [(False, "0"), (True, "0"), (False, "1"), (True, "1")])
def test_zero3_matches_zero2_two_ranks(ckpt, persist, monkeypatch):
    """persist = "1": every layer keeps its gathered parameters in a slot of its own between optimizer steps (gathered
    once per step instead of twice per micro-batch); "0": two rotating slots. Same result either way."""
    monkeypatch.setenv("OPENRLHF_B200_ZERO3_PERSIST", persist)       # inherited by the spawned ranks
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29745 + int(ckpt) + 2 * int(persist)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, ckpt)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    for _ in range(2):
        ok, err, na, nb = q.get(timeout=5)
        assert ok, err
        assert abs(na - nb) < 1e-4 * max(1.0, abs(na))


def test_zero3_single_rank():
    a, b, na, nb = _run(0, 1, False)
    assert torch.allclose(a, b, rtol=1e-4, atol=5e-5), float((a - b).abs().max())
