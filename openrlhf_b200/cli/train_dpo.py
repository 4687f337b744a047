"""``python -m openrlhf.cli.train_dpo``: DPO / IPO / cDPO training (flag-compatible with openrlhf/cli/train_dpo.py:174-370)."""
from __future__ import annotations

import argparse
import math
import os

from ..datasets import RewardDataset
from ..datasets.utils import blending_datasets
from ..models.actor import Actor
from ..trainer.dpo_trainer import DPOTrainer
from ..utils.strategy import get_strategy
from ..utils.utils import get_tokenizer
from . import flags as F


def train(args):
    strategy = get_strategy(args)
    strategy.setup_distributed()
    model = Actor(args.model.model_name_or_path, device=strategy.device(), packing_samples=args.ds.packing_samples,
                  shard_world=strategy.zero_world, seed=args.train.seed, lora_rank=args.ds.lora.rank,
                  lora_alpha=args.ds.lora.alpha, target_modules=args.ds.lora.target_modules,
                  lora_dropout=args.ds.lora.dropout, load_in_4bit=args.ds.load_in_4bit)
    tokenizer = get_tokenizer(args.model.model_name_or_path, model.model, "right", strategy,
                              use_fast=not args.data.disable_fast_tokenizer)
    ref_device = "cpu" if args.ref.offload else strategy.device()
    ref_model = Actor(args.ref.model_name_or_path or args.model.model_name_or_path, device=ref_device,
                      packing_samples=args.ds.packing_samples, seed=args.train.seed)
    ref_model.requires_grad_(False)
    if args.model.gradient_checkpointing_enable:
        model.gradient_checkpointing_enable()

    def make_loader(spec, probs, split, shuffle):
        data = blending_datasets(spec, probs, strategy, args.train.seed, max_count=args.data.max_samples,
                                 dataset_split=split)
        data = data.select(range(min(args.data.max_samples, len(data))))
        ds = RewardDataset(data, tokenizer, args.data.max_len, strategy, input_template=args.data.input_template,
                           is_dpo=True)
        return ds, strategy.setup_dataloader(ds, args.train.micro_batch_size, True, shuffle, ds.collate_fn,
                                             num_workers=args.data.dataloader_num_workers)

    train_ds, train_dl = make_loader(args.data.dataset, args.data.dataset_probs, args.data.dataset_split, True)
    eval_dl = None
    if getattr(args.eval, "dataset", None):
        _, eval_dl = make_loader(args.eval.dataset, None, args.eval.split, False)
    steps_per_epoch = len(train_ds) // args.train.batch_size
    max_steps = math.ceil(args.train.max_epochs * steps_per_epoch)
    model, ref_model = strategy.prepare((model, F.optimizer_cfg(args, max_steps)), ref_model)
    consumed = 0
    if args.ckpt.load_enable and os.path.exists(args.ckpt.path):
        path, states = strategy.load_ckpt(model, args.ckpt.path)
        if path is not None:
            consumed = states["consumed_samples"]
            strategy.print(f"Loaded the checkpoint: {args.ckpt.path}, consumed_samples: {consumed}")
    os.makedirs(args.ckpt.output_dir, exist_ok=True)
    trainer = DPOTrainer(model=model, ref_model=ref_model, tokenizer=tokenizer, strategy=strategy, optim=None,
                         train_dataloader=train_dl, eval_dataloader=eval_dl, scheduler=None, max_norm=args.max_norm,
                         beta=args.model.beta, max_epochs=args.train.max_epochs, save_hf_ckpt=args.ckpt.save_hf,
                         disable_ds_ckpt=args.ckpt.disable_ds)
    trainer.fit(args, consumed, steps_per_epoch)
    strategy.save_model(model, tokenizer, args.ckpt.output_dir)


def build_parser():
    p = argparse.ArgumentParser()
    F.add_flags(p, F.checkpoint_flags("./ckpt/checkpoints_dpo"), F.logger_flags("openrlhf_train_dpo", "exp"),
                [("--train.micro_batch_size", int, 8), ("--train.max_epochs", int, 1), ("--eval.split", str, "test"),
                 ("--ref.offload", F.BOOL, False), ("--ref.model_name_or_path", str, None),
                 ("--model.beta", float, 0.1), ("--model.ipo_enable", F.BOOL, False),
                 ("--model.label_smoothing", float, 0.0), ("--model.nll_loss_coef", float, 0),
                 ("--data.prompt_key", str, None), ("--data.chosen_key", str, "chosen"),
                 ("--data.rejected_key", str, "rejected"), ("--data.input_template", str, None),
                 ("--data.max_len", int, 512)],
                F.SPMD_TRAIN, F.ENGINE, F.optimizer_flags("", 1e-5))
    return p


def validate(args):
    if args.ref.model_name_or_path is None or args.ref.model_name_or_path == "":
        args.ref.model_name_or_path = args.model.model_name_or_path
    if args.data.input_template and "{}" not in args.data.input_template:
        print("[Warning] '{}' not in --data.input_template; set to None")
        args.data.input_template = None
    if args.ds.ring_attn_size > 1 and not args.ds.packing_samples:
        print("[Warning] --ds.ring_attn_size > 1 requires --ds.packing_samples; enabling it.")
        args.ds.packing_samples = True
    return args


if __name__ == "__main__":
    train(validate(F.finalize(build_parser())))
