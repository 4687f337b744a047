"""Weight-sync copy plans: TP slicing of the fused layouts and sharded (ZeRO-3) sources, executed on CPU."""
import pytest
import torch

from openrlhf_b200.models.config import PRESETS
from openrlhf_b200.models.transformer import build_param_specs
from openrlhf_b200.parallel.reshard import build_plan, run_plan_reference, tp_param_specs


def _flat(cfg):
    specs = build_param_specs(cfg)
    size = specs[-1].offset + (specs[-1].numel + 127) // 128 * 128
    return specs, torch.arange(size, dtype=torch.float32)


def _expected(cfg, specs, flat, name, tp_rank, tp):
    s = next(x for x in specs if x.name == name)
    w = flat[s.offset:s.offset + s.numel].view(s.shape)
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    leaf = ".".join(name.split(".")[-2:])
    if tp == 1:
        return w
    if leaf in ("qkv.weight", "qkv.bias"):
        q, k, v = w[: Hq * D], w[Hq * D:(Hq + Hkv) * D], w[(Hq + Hkv) * D:]
        return torch.cat([t.chunk(tp, 0)[tp_rank] for t in (q, k, v)], 0)
    if leaf == "gate_up.weight":
        g, u = w.chunk(2, 0)
        return torch.cat([g.chunk(tp, 0)[tp_rank], u.chunk(tp, 0)[tp_rank]], 0)
    if leaf in ("o.weight", "down.weight"):
        return w.chunk(tp, 1)[tp_rank]
    return w


@pytest.mark.parametrize("preset,tp,src_world", [("tiny-llama", 1, 1), ("tiny-llama", 2, 1), ("tiny-qwen2", 1, 3),
                                                 ("tiny-llama", 2, 4)])
def test_plan_matches_slicing(preset, tp, src_world):
    cfg = PRESETS[preset]
    specs, flat = _flat(cfg)
    shard = None
    srcs = [flat]
    if src_world > 1:
        shard = (flat.numel() + src_world * 256 - 1) // (src_world * 256) * 256
        padded = torch.cat([flat, torch.zeros(shard * src_world - flat.numel())])
        srcs = [padded[r * shard:(r + 1) * shard].clone() for r in range(src_world)]
    for tp_rank in range(tp):
        entries, size = build_plan(cfg, tp_rank, tp, src_world, shard)
        dst = torch.full((size,), -1.0)
        run_plan_reference(entries, srcs, dst)
        for d in tp_param_specs(cfg, tp_rank, tp):
            got = dst[d.offset:d.offset + d.numel].view(d.shape)
            want = _expected(cfg, specs, flat, d.name, tp_rank, tp)
            assert torch.equal(got, want.reshape(d.shape)), d.name


def test_long_contiguous_entries_are_split_below_the_int32_limit():
    from openrlhf_b200.parallel.reshard import CopyEntry, ReshardPlan

    big = 3 * (1 << 30) + 4096            # elements: more than an int32 can hold
    parts = ReshardPlan.split_large([CopyEntry(128, 256, 1, big, big, big, 1), CopyEntry(0, 0, 4, 64, 128, 64, 0)])
    assert [p.row_elems for p in parts[:-1]] == [1 << 30, 1 << 30, 1 << 30, 4096]
    assert [p.src_off for p in parts[:-1]] == [128 + i * (1 << 30) for i in range(4)]
    assert [p.dst_off for p in parts[:-1]] == [256 + i * (1 << 30) for i in range(4)]
    assert all(p.src_rank == 1 and p.rows == 1 for p in parts[:-1]) and parts[-1].rows == 4
    with pytest.raises(ValueError):
        ReshardPlan([CopyEntry(0, 0, 2, 1 << 31, 1 << 31, 1 << 31, 0)], "cpu")
