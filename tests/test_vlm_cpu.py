"""Vision-language path (Qwen2-VL architecture) against transformers on CPU in fp32: vision tower, placeholder
scatter, 3-component rotary positions, checkpoint names in both directions."""
import pytest
import torch

from openrlhf_b200.models import hf_io
from openrlhf_b200.models.config import ModelConfig
from openrlhf_b200.models.transformer import TransformerLM
from openrlhf_b200.models.vision import mrope_positions

IMG, VSTART, VEND = 500, 502, 503


def _hf_model(transformers):
    cfg = transformers.Qwen2VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=1024,
                         rope_theta=10000.0, rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]},
                         tie_word_embeddings=False),
        vision_config=dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3),
        image_token_id=IMG, video_token_id=501, vision_start_token_id=VSTART, vision_end_token_id=VEND)
    torch.manual_seed(0)
    m = transformers.Qwen2VLForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for p in m.parameters():
            if p.ndim == 1:
                p.add_(0.1 * torch.randn_like(p))
    return m


def _sample(grids, texts):
    """ids: text0 <vs> img*k <ve> text1 ...; pixel_values random."""
    ids = []
    for i, t in enumerate(texts):
        ids += t
        if i < len(grids):
            tt, h, w = grids[i]
            ids += [VSTART] + [IMG] * (tt * h * w // 4) + [VEND]
    n_patch = sum(t * h * w for t, h, w in grids)
    return ids, torch.randn(n_patch, 3 * 2 * 14 * 14), torch.tensor(grids)


def test_mrope_positions_layout():
    ids = [7, 8, IMG, IMG, IMG, IMG, IMG, IMG, 9, 10]
    pos, delta = mrope_positions(ids, [(1, 4, 6)], IMG, 2)       # 2 x 3 merged grid
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3]
    assert pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8:].tolist() == [[5, 6]] * 3                   # continues after the largest component (2 + 3)
    assert delta == 7 - 10


def test_logits_match_transformers_qwen2_vl(tmp_path):
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "Qwen2VLForConditionalGeneration"):
        pytest.skip("transformers without Qwen2-VL")
    hf = _hf_model(transformers)
    hf.save_pretrained(str(tmp_path / "hf"))
    m = hf_io.load_pretrained(str(tmp_path / "hf"), device="cpu")
    assert m.cfg.is_vlm and m.cfg.mrope_section == (4, 6, 6) and m.cfg.image_token_id == IMG
    m = TransformerLM(m.cfg, device="cpu", dtype=torch.float32, seed=None)
    hf_io.load_weights(m, str(tmp_path / "hf"))
    m.eval()

    torch.manual_seed(1)
    docs = [_sample([(1, 4, 6)], [[3, 4, 5], [6, 7]]),
            _sample([(1, 2, 2), (1, 4, 4)], [[11], [12, 13, 14], [15, 16, 17, 18]]),
            ([21, 22, 23, 24], None, None)]                        # text only
    ids_all = [t for d in docs for t in d[0]]
    cu = [0]
    for d in docs:
        cu.append(cu[-1] + len(d[0]))
    pv = torch.cat([d[1] for d in docs if d[1] is not None])
    thw = torch.cat([d[2] for d in docs if d[2] is not None])
    input_ids = torch.tensor(ids_all)
    with torch.no_grad():
        emb, pos = m.multimodal_inputs(input_ids, cu, pv, thw)
        h, _ = m(input_ids, pos, torch.tensor(cu, dtype=torch.int32), max(len(d[0]) for d in docs), inputs_embeds=emb)
        mine = m.logits(h)
        for i, (ids, p, g) in enumerate(docs):
            kw = {} if p is None else {"pixel_values": p, "image_grid_thw": g}
            t = torch.tensor(ids)[None]
            if p is not None:
                kw["mm_token_type_ids"] = (t == IMG).int()
            try:
                ref = hf(input_ids=t, **kw).logits[0]
            except TypeError:
                kw.pop("mm_token_type_ids", None)
                ref = hf(input_ids=t, **kw).logits[0]
            got = mine[cu[i]:cu[i + 1]]
            err = (got - ref).abs().max().item()
            assert err < 2e-3 * max(ref.abs().max().item(), 1.0), (i, err)

    # and back: a checkpoint written here loads in transformers with identical weights
    hf_io.save_pretrained(m, str(tmp_path / "mine"))
    back = transformers.Qwen2VLForConditionalGeneration.from_pretrained(str(tmp_path / "mine"), torch_dtype=torch.float32)
    sd, sd0 = back.state_dict(), hf.state_dict()
    assert set(sd) == set(sd0)
    for k in sd0:
        assert torch.allclose(sd[k].float(), sd0[k].float(), atol=1e-6), k


def test_vision_tower_gets_gradients():
    from openrlhf_b200.models.config import PRESETS
    import dataclasses

    cfg = dataclasses.replace(PRESETS["tiny-qwen2-vl"])
    m = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=3)
    ids = [5, 6, cfg.vision_start_token_id] + [cfg.image_token_id] * 4 + [cfg.vision_end_token_id, 7, 8, 9]
    pv, thw = torch.randn(16, 1176), torch.tensor([[1, 4, 4]])
    input_ids = torch.tensor(ids)
    emb, pos = m.multimodal_inputs(input_ids, [0, len(ids)], pv, thw)
    h, _ = m(input_ids, pos, torch.tensor([0, len(ids)], dtype=torch.int32), len(ids), inputs_embeds=emb)
    labels = torch.roll(input_ids, -1)
    logp, _ = m.logprobs(h, labels)
    (-logp[:-1].mean()).backward()
    g = m.p("visual.blocks.0.attn.qkv.weight").grad
    assert g is not None and g.abs().sum() > 0
    assert m.p("visual.merger.mlp.2.weight").grad.abs().sum() > 0


def test_stray_placeholder_token_is_text():
    """A placeholder id the policy sampled itself (not part of a complete image run) keeps its ordinary embedding and a
    text position; the real run still receives the tower's rows."""
    import dataclasses

    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.vision import image_runs

    cfg = dataclasses.replace(PRESETS["tiny-qwen2-vl"])
    IMGT = cfg.image_token_id
    ids = [5, cfg.vision_start_token_id] + [IMGT] * 4 + [cfg.vision_end_token_id, 7, IMGT, 9]
    assert image_runs(ids, [(1, 4, 4)], IMGT, 2) == [(2, 4, (1, 4, 4))]
    pos, delta = mrope_positions(ids, [(1, 4, 4)], IMGT, 2)
    assert pos[:, -3:].tolist() == [[5, 6, 7]] * 3 and delta == 8 - len(ids)
    m = TransformerLM(cfg, device="cpu", dtype=torch.float32, seed=3)
    t = torch.tensor(ids)
    emb, _ = m.multimodal_inputs(t, [0, len(ids)], torch.randn(16, 1176), torch.tensor([[1, 4, 4]]))
    plain = m.p("embed.weight")[t]
    assert torch.equal(emb[8], plain[8]) and not torch.equal(emb[2], plain[2])
