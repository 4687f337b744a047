"""``python -m openrlhf.cli.train_sft``: supervised fine-tuning, one process per GPU (torchrun).
Flag-compatible with openrlhf/cli/train_sft.py:150-336."""
from __future__ import annotations

import argparse
import math
import os

from ..datasets import SFTDataset
from ..datasets.utils import blending_datasets
from ..models.actor import Actor
from ..trainer.sft_trainer import SFTTrainer
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
    if args.model.gradient_checkpointing_enable:
        model.gradient_checkpointing_enable()

    def make_loader(spec, probs, split, shuffle, max_samples):
        data = blending_datasets(spec, probs, strategy, args.train.seed, max_count=max_samples, dataset_split=split)
        data = data.select(range(min(max_samples, len(data))))
        ds = SFTDataset(data, tokenizer, args.data.max_len, strategy, pretrain_mode=args.model.pretrain_mode_enable,
                        input_template=args.data.input_template, multiturn=args.data.multiturn)
        return ds, strategy.setup_dataloader(ds, args.train.micro_batch_size, True, shuffle, ds.collate_fn,
                                             num_workers=args.data.dataloader_num_workers)

    train_ds, train_dl = make_loader(args.data.dataset, args.data.dataset_probs, args.data.dataset_split, True,
                                     args.data.max_samples)
    eval_dl = None
    if getattr(args.eval, "dataset", None):
        _, eval_dl = make_loader(args.eval.dataset, None, args.eval.split, False, args.data.max_samples)
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
    trainer = SFTTrainer(model=model, strategy=strategy, optim=None, train_dataloader=train_dl, eval_dataloader=eval_dl,
                         scheduler=None, max_norm=args.max_norm, pretrain_mode=args.model.pretrain_mode_enable,
                         batch_size=args.train.batch_size, max_epochs=args.train.max_epochs, tokenizer=tokenizer,
                         save_hf_ckpt=args.ckpt.save_hf, disable_ds_ckpt=args.ckpt.disable_ds)
    trainer.fit(args, consumed, steps_per_epoch)
    strategy.save_model(model, tokenizer, args.ckpt.output_dir)


def build_parser():
    p = argparse.ArgumentParser()
    F.add_flags(p, F.checkpoint_flags("./ckpt/checkpoints_sft"), F.logger_flags("openrlhf_train_sft", "sft"),
                [("--train.micro_batch_size", int, 8), ("--train.max_epochs", int, 2),
                 ("--model.pretrain_mode_enable", F.BOOL, False), ("--eval.split", str, "train"),
                 ("--data.multiturn", F.BOOL, False), ("--data.input_key", str, "input"),
                 ("--data.output_key", str, None), ("--data.input_template", str, "User: {}\nAssistant: "),
                 ("--data.max_len", int, 2048)],
                F.SPMD_TRAIN, F.ENGINE, F.optimizer_flags("", 5e-6))
    return p


def validate(args):
    if args.data.multiturn and not args.data.apply_chat_template:
        raise AssertionError("apply_chat_template must be enabled when multiturn is enabled")
    if args.data.input_template and "{}" not in args.data.input_template:
        print("[Warning] '{}' not in --data.input_template; set to None")
        args.data.input_template = None
    if args.data.input_template and "\\n" in args.data.input_template:
        print("[Warning] input_template contains \\n characters instead of newline.")
    if args.ds.ring_attn_size > 1 and not args.ds.packing_samples:
        print("[Warning] --ds.ring_attn_size > 1 requires --ds.packing_samples; enabling it.")
        args.ds.packing_samples = True
    return args


if __name__ == "__main__":
    train(validate(F.finalize(build_parser())))
