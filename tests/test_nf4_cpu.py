"""NF4 block quantisation: level table, idempotence, error bound, model round trip and the QLoRA option of Actor."""
import torch

from openrlhf_b200.ops import nf4


def test_quantize_dequantize_properties():
    torch.manual_seed(0)
    w = torch.randn(64 * 50) * 0.02
    codes, absmax = nf4.quantize(w)
    assert codes.dtype == torch.uint8 and codes.numel() == w.numel() // 2 and absmax.numel() == w.numel() // 64
    d = nf4.dequantize(codes, absmax, torch.float32)
    # the largest value of every block is represented exactly, every value within half the widest level gap
    blocks, db = w.view(-1, 64), d.view(-1, 64)
    top = blocks.abs().argmax(dim=1)
    assert torch.allclose(db.gather(1, top[:, None]), blocks.gather(1, top[:, None]))
    gap = (nf4.LEVELS[1:] - nf4.LEVELS[:-1]).max() / 2
    assert ((db - blocks).abs() <= gap * absmax[:, None] + 1e-7).all()
    # quantising representable values changes nothing
    c2, a2 = nf4.quantize(d)
    assert torch.equal(c2, codes) and torch.allclose(a2, absmax)
    # a block of zeros stays zero
    z, za = nf4.quantize(torch.zeros(64))
    assert nf4.dequantize(z, za, torch.float32).abs().max() == 0


def test_levels_are_the_qlora_table():
    assert nf4.LEVELS.numel() == 16 and nf4.LEVELS[0] == -1 and nf4.LEVELS[7] == 0 and nf4.LEVELS[15] == 1
    assert (nf4.LEVELS[1:] > nf4.LEVELS[:-1]).all()


def test_actor_load_in_4bit_freezes_nf4_base_and_trains_adapters():
    from openrlhf_b200.models.actor import Actor
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.models.config import PRESETS

    lm = TransformerLM(PRESETS["tiny-llama"], device="cpu", dtype=torch.float32, seed=1)
    before = lm.p("layers.0.qkv.weight").detach().clone()
    emb = lm.p("embed.weight").detach().clone()
    actor = Actor(lm, device="cpu", lora_rank=4, load_in_4bit=True)
    w = lm.p("layers.0.qkv.weight").detach()
    assert not torch.equal(w, before) and torch.equal(lm.p("embed.weight").detach(), emb)
    packed = nf4.pack_model(lm)
    c, a = packed["layers.0.qkv.weight"]
    assert torch.allclose(nf4.dequantize(c, a, torch.float32).view_as(w), w)        # already on the NF4 grid
    seq = torch.randint(3, 1000, (2, 12))
    logp = actor(seq, None, torch.ones_like(seq))
    (-logp.mean()).backward()
    assert all(p.grad is None for _, p in lm.named_specs())
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in actor.lora.parameters())
    # compact form round trip
    lm2 = TransformerLM(PRESETS["tiny-llama"], device="cpu", dtype=torch.float32, seed=9)
    nf4.unpack_model(lm2, packed)
    assert torch.equal(lm2.p("layers.1.down.weight"), lm.p("layers.1.down.weight"))
