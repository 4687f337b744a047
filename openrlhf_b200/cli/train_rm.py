"""``python -m openrlhf.cli.train_rm``: reward-model training (flag-compatible with openrlhf/cli/train_rm.py:161-347)."""
from __future__ import annotations

import argparse
import math
import os

from ..datasets import RewardDataset
from ..datasets.utils import blending_datasets
from ..models.model import get_llm_for_sequence_regression
from ..trainer.rm_trainer import RewardModelTrainer
from ..utils.strategy import get_strategy
from ..utils.utils import get_tokenizer
from . import flags as F


def train(args):
    strategy = get_strategy(args)
    strategy.setup_distributed()
    model = get_llm_for_sequence_regression(args.model.model_name_or_path, "reward", init_value_head=True,
                                            value_head_prefix=args.ds.value_head_prefix, device=strategy.device(),
                                            packing_samples=args.ds.packing_samples, shard_world=strategy.zero_world,
                                            seed=args.train.seed, load_in_4bit=args.ds.load_in_4bit)
    tokenizer = get_tokenizer(args.model.model_name_or_path, model, "left", strategy,
                              use_fast=not args.data.disable_fast_tokenizer)
    if args.model.gradient_checkpointing_enable:
        model.gradient_checkpointing_enable()
    data = blending_datasets(args.data.dataset, args.data.dataset_probs, strategy, args.train.seed,
                             max_count=args.data.max_samples, dataset_split=args.data.dataset_split)
    data = data.select(range(min(args.data.max_samples, len(data))))
    train_ds = RewardDataset(data, tokenizer, args.data.max_len, strategy, input_template=args.data.input_template)
    train_dl = strategy.setup_dataloader(train_ds, args.train.micro_batch_size, True, True, train_ds.collate_fn,
                                         num_workers=args.data.dataloader_num_workers)
    if getattr(args.eval, "dataset", None):
        ev = blending_datasets(args.eval.dataset, None, strategy, dataset_split=args.eval.split)
    else:  # reward mean / std need an eval pass: default to about 1 % of the training pairs
        ev = data.select(range(min(max(1, int(len(data) * 0.01)), len(data))))
    eval_ds = RewardDataset(ev, tokenizer, args.data.max_len, strategy, input_template=args.data.input_template)
    eval_dl = strategy.setup_dataloader(eval_ds, args.train.micro_batch_size, True, False, eval_ds.collate_fn,
                                        drop_last=False, num_workers=args.data.dataloader_num_workers)
    steps_per_epoch = len(train_ds) // args.train.batch_size
    max_steps = math.ceil(args.train.max_epochs * steps_per_epoch)
    model = strategy.prepare((model, F.optimizer_cfg(args, max_steps)))
    consumed = 0
    if args.ckpt.load_enable and os.path.exists(args.ckpt.path):
        path, states = strategy.load_ckpt(model, args.ckpt.path)
        if path is not None:
            consumed = states["consumed_samples"]
            strategy.print(f"Loaded the checkpoint: {args.ckpt.path}, consumed_samples: {consumed}")
    os.makedirs(args.ckpt.output_dir, exist_ok=True)
    trainer = RewardModelTrainer(model=model, strategy=strategy, optim=None, tokenizer=tokenizer, train_dataloader=train_dl,
                                 eval_dataloader=eval_dl, scheduler=None, max_norm=args.max_norm,
                                 max_epochs=args.train.max_epochs, loss=args.model.loss_type,
                                 save_hf_ckpt=args.ckpt.save_hf, disable_ds_ckpt=args.ckpt.disable_ds)
    trainer.fit(args, consumed, steps_per_epoch)
    strategy.save_model(model, tokenizer, args.ckpt.output_dir)   # writes value_head_prefix / mean / std to config.json


def build_parser():
    p = argparse.ArgumentParser()
    F.add_flags(p, F.checkpoint_flags("./ckpt/checkpoints_rm"), F.logger_flags("openrlhf_train_rm", "rm"),
                [("--train.micro_batch_size", int, 1), ("--train.max_epochs", int, 1), ("--eval.split", str, "train"),
                 ("--model.compute_fp32_loss_enable", F.BOOL, False), ("--model.margin_loss_enable", F.BOOL, False),
                 ("--model.loss_type", str, "sigmoid"), ("--data.prompt_key", str, None),
                 ("--data.chosen_key", str, "chosen"), ("--data.rejected_key", str, "rejected"),
                 ("--data.input_template", str, None), ("--data.max_len", int, 512)],
                F.SPMD_TRAIN, F.ENGINE, F.optimizer_flags("", 9e-6))
    return p


def validate(args):
    if args.data.input_template and "{}" not in args.data.input_template:
        print("[Warning] '{}' not in --data.input_template; set to None")
        args.data.input_template = None
    if args.ds.ring_attn_size > 1 and not args.ds.packing_samples:
        print("[Warning] --ds.ring_attn_size > 1 requires --ds.packing_samples; enabling it.")
        args.ds.packing_samples = True
    return args


if __name__ == "__main__":
    train(validate(F.finalize(build_parser())))
