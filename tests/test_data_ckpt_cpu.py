"""Datasets on synthetic sources, checkpoint rotation, world-size-agnostic sharded checkpoints and host-side fault
injection (a corrupted shard, a missing manifest)."""
import json
import os

import pytest
import torch

from openrlhf_b200.datasets import PromptDataset, RewardDataset, SFTDataset
from openrlhf_b200.datasets.utils import blending_datasets
from openrlhf_b200.models.config import PRESETS
from openrlhf_b200.models.transformer import TransformerLM
from openrlhf_b200.parallel.zero import ZeroEngine
from openrlhf_b200.utils import checkpoint as ckpt
from openrlhf_b200.utils.utils import SyntheticTokenizer


class _Strategy:
    def print(self, *a, **k):
        pass

    def is_rank_0(self):
        return True


def _args(**kw):
    from types import SimpleNamespace as NS
    data = dict(input_key="input", output_key="output", label_key="label", prompt_key="prompt", chosen_key="chosen",
                rejected_key="rejected", apply_chat_template=False, tokenizer_chat_template=None, image_key=None)
    data.update(kw)
    return NS(data=NS(**data))


def test_sft_dataset_masks_and_collate():
    s = _Strategy()
    s.args = _args()
    tok = SyntheticTokenizer(1000)
    data = blending_datasets("synthetic://sft?n=6&len=10&vocab=1000&out_len=5", None, s)
    ds = SFTDataset(data, tok, 64, s)
    assert len(ds) == 6
    batch = ds.collate_fn([ds[i] for i in range(3)])
    ids, att, loss_mask = batch[0], batch[1], batch[2]
    assert ids.shape == att.shape == loss_mask.shape and ids.shape[0] == 3
    for i in range(3):
        n = int(att[i].sum())
        assert int(ids[i, n - 1]) == tok.eos_token_id              # forced EOS at the end of the response
        # the loss covers exactly the response tokens, shifted by one: positions prompt_len-1 .. n-2
        assert int(loss_mask[i].sum()) == 5 and loss_mask[i, :9].sum() == 0 and loss_mask[i, n - 1] == 0


def test_reward_dataset_padding_sides():
    s = _Strategy()
    s.args = _args()
    tok = SyntheticTokenizer(1000)
    data = blending_datasets("synthetic://pairs?n=4&len=8&vocab=1000&out_len=6", None, s)
    rm = RewardDataset(data, tok, 64, s)
    c_ids, c_mask, r_ids, r_mask, _ = rm.collate_fn([rm[i] for i in range(2)] + [(rm[2][0][:, 2:], rm[2][1][:, 2:], *rm[2][2:])])
    assert c_mask[2, 0] == 0 and c_mask[2, -1] == 1                # RM batches are left-padded
    dpo = RewardDataset(data, tok, 64, s, is_dpo=True)
    item = dpo[0]
    assert item[-1] == 8                                           # DPO items carry the prompt length


def test_prompt_dataset_items():
    s = _Strategy()
    s.args = _args()
    tok = SyntheticTokenizer(1000)
    data = blending_datasets("synthetic://prompts?n=5&len=7&vocab=1000", None, s)
    ds = PromptDataset(data, tok, s)
    src, prompt, label = ds[3][:3]
    assert src == "synthetic" and len(prompt.split()) == 7 and label == "3"


def _engine(world=1, rank=0, seed=0):
    m = TransformerLM(PRESETS["tiny-llama"], device="cpu", dtype=torch.float32, seed=seed, shard_world=world)
    e = ZeroEngine(m, lr=1e-3)
    e.world, e.rank = world, rank          # single process standing in for one rank of a larger job
    per = e.padded_numel(m.total_numel, world) // world
    return m, e, per


def test_rotation_keeps_newest(tmp_path):
    d = str(tmp_path)
    for i in range(5):
        os.makedirs(os.path.join(d, f"global_step{i}"))
        open(os.path.join(d, f"global_step{i}", "x.bin"), "wb").write(b"0" * 10)
        os.utime(os.path.join(d, f"global_step{i}"), (i, i))
    ckpt.rotate(d, "global_step5", max_num=3, max_mem=1000, log=lambda *a: None)
    left = sorted(os.listdir(d))
    assert left == ["global_step3", "global_step4"], left          # room for the one about to be written


def test_sharded_checkpoint_round_trip_and_fault_injection(tmp_path):
    d = str(tmp_path)
    m, e, _ = _engine()
    e.master.add_(0.25)
    e.exp_avg.fill_(0.5)
    e.opt_step = 7
    ckpt.save_sharded(e, d, "global_step7", {"consumed_samples": 123}, rank=0, world=1)
    m2, e2, _ = _engine(seed=1)
    path, state = ckpt.load_sharded(e2, d)
    assert path.endswith("global_step7") and state["consumed_samples"] == 123 and e2.opt_step == 7
    assert torch.equal(e2.master, e.master) and torch.equal(e2.exp_avg, e.exp_avg)
    assert torch.allclose(m2.flat[: m2.total_numel], e.master[: m2.total_numel].to(m2.flat.dtype))
    # fault injection on the host: truncated shard, then missing manifest
    shard = os.path.join(d, "global_step7", "shard_00000.safetensors")
    blob = open(shard, "rb").read()
    open(shard, "wb").write(blob[: len(blob) // 2])
    with pytest.raises(Exception):
        ckpt.load_sharded(_engine(seed=2)[1], d)
    open(shard, "wb").write(blob)
    os.remove(os.path.join(d, "global_step7", "manifest.json"))
    with pytest.raises(Exception):
        ckpt.load_sharded(_engine(seed=2)[1], d)
    assert ckpt.load_sharded(_engine(seed=2)[1], str(tmp_path / "nothing"))[0] is None


class _ListDataset:
    """Minimal stand-in for a datasets.Dataset (map / filter / column access) over a list of dict rows."""

    def __init__(self, rows):
        self.rows = rows
        self.column_names = sorted({k for r in rows for k in r})

    def map(self, fn, remove_columns=None, num_proc=None):
        return _ListDataset([fn(dict(r)) for r in self.rows])

    def filter(self, fn):
        return _ListDataset([r for r in self.rows if fn(r)])

    def __getitem__(self, key):
        return [r[key] for r in self.rows]

    def __len__(self):
        return len(self.rows)


def test_sft_dataset_multiturn_pretrain_and_truncation():
    """Conversations: the loss covers every assistant turn and nothing else (shifted by one position). Pre-training
    rows: the loss covers everything. A sample longer than max_length is cut and still ends with a real EOS id; a row
    whose prompt nearly fills the window is dropped."""
    tok = SyntheticTokenizer(1000)
    s = _Strategy()
    s.args = _args(apply_chat_template=True, output_key=None)
    conv = [{"role": "user", "content": "11 12 13"}, {"role": "assistant", "content": "21 22"},
            {"role": "user", "content": "31"}, {"role": "assistant", "content": "41 42 43"}]
    ds = SFTDataset(_ListDataset([{"input": conv}]), tok, 64, s, multiturn=True)
    ids, att, mask = ds[0]
    assert ids[0].tolist() == [11, 12, 13, 21, 22, 31, 41, 42, 43, tok.eos_token_id]
    toks = ids[0].tolist()
    # position t is trained iff token t + 1 belongs to an assistant turn
    want = [1.0 if toks[t + 1] in (21, 22, 41, 42, 43) else 0.0 for t in range(len(toks) - 1)] + [0.0]
    assert mask[0].tolist() == want and att.all()

    s2 = _Strategy()
    s2.args = _args(output_key=None)
    pre = SFTDataset(_ListDataset([{"input": " ".join(str(i) for i in range(100, 140))}]), tok, 16, s2,
                     pretrain_mode=True)
    ids, att, mask = pre[0]
    assert ids.shape == (1, 16) and mask.sum() == 16 and ids[0, -1] == 115      # cut, no EOS forced, loss everywhere

    s3 = _Strategy()
    s3.args = _args()
    rows = [{"input": " ".join(str(i) for i in range(200, 210)), "output": " ".join(str(i) for i in range(300, 330))},
            {"input": " ".join(str(i) for i in range(400, 415)), "output": "5"},          # prompt of 15 >= 16 - 2
            {"input": "7 8", "output": ""}]                                                # nothing to learn
    cut = SFTDataset(_ListDataset(rows), tok, 16, s3)
    assert len(cut) == 1
    ids, att, mask = cut[0]
    assert ids.shape == (1, 16) and int(ids[0, -1]) == tok.eos_token_id
    assert mask[0].tolist() == [0.0] * 9 + [1.0] * 6 + [0.0]           # positions prompt_len - 1 .. L - 2
