"""Tensor-parallel training (column / row parallel shards, vocabulary-parallel head, differentiable collectives,
replicated-gradient averaging, TP-aware clipping norm) against the same model trained unsharded: same losses, same gradient norm, same weights after
two optimizer steps with gradient clipping. Runs on CPU ranks (gloo, fp32) and on GPUs (nccl, bf16); world = dp x tp
with tp = 2."""
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = torch.cuda.is_available() and os.environ.get("TP_TEST_CPU") != "1"
    if gpu:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl" if gpu else "gloo")
    dev = "cuda" if gpu else "cpu"
    from openrlhf_b200.models.config import ModelConfig
    from openrlhf_b200.models.packing import pack_lists
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.parallel.tp_train import shard_for_training
    from openrlhf_b200.parallel.zero import ZeroEngine
    from openrlhf_b200.utils.strategy import RankMesh

    tp = 2
    mesh = RankMesh(world, 1, tp, rank)
    for dim in ("dp", "sp", "tp"):
        mesh.group(dim)
    cfg = ModelConfig("qwen2", 1024, 256, 512, 2, 4, 2, head_dim=128, rope_theta=1e6, attention_bias=True)
    dtype = torch.bfloat16 if gpu else torch.float32
    # every dp replica sees its own data; the two tp ranks of a replica see the same
    g = torch.Generator().manual_seed(100 + mesh.dp_rank)
    data = [[torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (150, 70)] for _ in range(4)]

    def loss_of(model, seqs):
        pb = pack_lists(seqs, device=dev)
        h, _ = model(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        lp, _ = model.logprobs(h, pb.labels)
        return -lp.float().mean()

    def train(model, eng):
        losses = []
        for step in range(2):
            for j in range(2):
                l = loss_of(model, data[2 * step + j]) / 2
                losses.append(float(l))
                eng.backward(l)
            eng.step()
        return losses, eng.grad_norm()

    # reference: unsharded model, data-parallel over the dp group only
    ref = TransformerLM(cfg, device=dev, dtype=dtype, seed=0, shard_world=mesh.dp)
    ref.train()
    ref_losses, ref_norm = train(ref, ZeroEngine(ref, lr=1e-3, max_norm=0.5, weight_decay=0.01, group=mesh.group("dp"),
                                                 use_symm=False))
    full0 = TransformerLM(cfg, device=dev, dtype=dtype, seed=0)
    shard = shard_for_training(full0, mesh.group("tp"), shard_world=mesh.dp)
    shard.train()
    eng = ZeroEngine(shard, lr=1e-3, max_norm=0.5, weight_decay=0.01, group=mesh.group("dp"), use_symm=False)
    losses, norm = train(shard, eng)
    got = shard.tp_train.gather_full(shard).float()
    want = ref.flat[: got.numel()].float()
    base = full0.flat[: got.numel()].float()
    upd_rel = ((got - want).norm() / (want - base).norm().clamp_min(1e-12)).item()
    print(f"rank {rank} (dp {mesh.dp_rank}, tp {mesh.tp_rank}): losses {losses} vs {ref_losses}, grad norm {norm:.5f} vs "
          f"{ref_norm:.5f}, update rel err {upd_rel:.2e}", flush=True)
    tol_l, tol_u = (2e-2, 0.25) if gpu else (1e-4, 1e-3)
    assert all(abs(a - b) < tol_l for a, b in zip(losses, ref_losses))
    assert abs(norm - ref_norm) < (0.05 if gpu else 1e-4) * ref_norm
    assert upd_rel < tol_u
    # the replicas of replicated parameters stay bit-identical across the tp group
    emb = shard.p("embed.weight").detach().float().contiguous()
    other = [torch.empty_like(emb) for _ in range(tp)]
    dist.all_gather(other, emb, group=mesh.group("tp"))
    assert torch.equal(other[0], other[1])
    # HF export names the full layout
    from openrlhf_b200.models.hf_io import hf_state_dict

    sd = hf_state_dict(shard)
    # the head is vocabulary-parallel: half of the rows per rank, the full matrix in the export, and full logits
    # (evaluation only) equal to the unsharded model's
    assert shard.tp_train.vocab_parallel and shard.p("lm_head.weight").shape == (cfg.vocab_size // tp, cfg.hidden_size)
    assert sd["lm_head.weight"].shape == (cfg.vocab_size, cfg.hidden_size)
    with torch.no_grad():
        pb = pack_lists(data[0], device=dev)
        hs, _ = shard(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        hr, _ = ref(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        ls, lr = shard.logits(hs).float(), ref.logits(hr).float()
    assert ls.shape == lr.shape and (ls - lr).abs().max().item() < (0.25 if gpu else 1e-3) * lr.abs().max().item()
    assert sd["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size)
    assert sd["model.layers.1.mlp.down_proj.weight"].shape == (cfg.hidden_size, cfg.intermediate_size)
    dist.barrier()
    if gpu:
        from openrlhf_b200.ops import _lib

        torch.cuda.synchronize()
        _lib.check_status()
        # the row-parallel projections went through the fused GEMM + all-reduce kernel
        assert shard.tp_train._fctx is not None and shard.tp_train._fctx.epoch > 0
    if rank == 0:
        print("TP_TRAIN_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
