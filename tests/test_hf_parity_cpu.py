"""HF round trip: a checkpoint written by this framework loads in transformers and produces the same logits as this
framework's own model definition (CPU, fp32), for the Llama, Qwen2 and Qwen3-MoE architectures."""
import dataclasses

import pytest
import torch

from openrlhf_b200.models import hf_io
from openrlhf_b200.models.config import PRESETS
from openrlhf_b200.models.packing import pack_lists
from openrlhf_b200.models.transformer import TransformerLM


@pytest.mark.parametrize("preset", ["tiny-llama", "tiny-qwen2", "tiny-qwen3-moe"])
def test_logits_match_transformers(preset, tmp_path):
    transformers = pytest.importorskip("transformers")
    cfg = dataclasses.replace(PRESETS[preset])
    if preset == "tiny-qwen2":
        cfg = dataclasses.replace(cfg, head_dim=64, num_attention_heads=4, num_key_value_heads=2, hidden_size=256)
    m = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=5)
    with torch.no_grad():
        for s, p in m.named_specs():
            if s.init in ("ones", "zeros"):
                p.add_(0.1 * torch.randn_like(p))
    hf_io.save_pretrained(m, str(tmp_path))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32)
    hf.eval()
    torch.manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab_size, (n,)) for n in (9, 17)]
    pb = pack_lists(seqs, "cpu")
    with torch.no_grad():
        h, _ = m(pb.input_ids, pb.position_ids, pb.cu_seqlens, pb.max_seqlen)
        mine = m.logits(h)
        cu = pb.cu_seqlens.tolist()
        for i, s in enumerate(seqs):
            ref = hf(input_ids=s[None]).logits[0]
            got = mine[cu[i]:cu[i + 1]]
            assert (got - ref).abs().max().item() < 2e-2 * max(ref.abs().max().item(), 1.0), preset


def test_reward_model_roundtrip(tmp_path):
    from openrlhf_b200.models.model import get_llm_for_sequence_regression
    cfg = PRESETS["tiny-llama"]
    base = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=2, with_lm_head=False, with_value_head=True)
    hf_io.save_pretrained(base, str(tmp_path), extra_config={"mean": 0.5, "std": 2.0, "normalize_reward": True})
    rm = get_llm_for_sequence_regression(str(tmp_path), "reward", device="cpu")
    rm.eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 7))
    mask = torch.tensor([[0, 0, 1, 1, 1, 1, 1], [1, 1, 1, 1, 1, 1, 1]])
    r = rm(ids, mask)
    assert r.shape == (2,) and float(rm.mean) == 0.5 and float(rm.std) == 2.0 and rm.normalize_reward
    cr = get_llm_for_sequence_regression(str(tmp_path), "critic", device="cpu")
    am = torch.ones(2, 3)
    v = cr(ids, am, torch.ones_like(ids))
    assert v.shape == (2, 3)
