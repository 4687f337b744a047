"""Scaffolding shared by the SPMD trainers (SFT / reward model / DPO): resume arithmetic from ``consumed_samples``,
sampler epochs, the log / eval / checkpoint cadence and logger fan-out. The three reference trainers repeat this code
inline (openrlhf/trainer/{sft,rm,dpo}_trainer.py); behaviour is kept, structure is shared."""
from __future__ import annotations

import os
from abc import ABC, abstractmethod

import torch

from ..utils.distributed_sampler import DistributedSampler
from ..utils.logging_utils import build_loggers


class SPMDTrainer(ABC):
    def __init__(self, model, strategy, optim, train_dataloader, eval_dataloader, scheduler, max_norm: float = 0.5,
                 max_epochs: int = 2, tokenizer=None, save_hf_ckpt: bool = False, disable_ds_ckpt: bool = False) -> None:
        self.model, self.strategy, self.optimizer, self.scheduler = model, strategy, optim, scheduler
        self.train_dataloader, self.eval_dataloader = train_dataloader, eval_dataloader
        self.max_norm, self.epochs, self.tokenizer = max_norm, max_epochs, tokenizer
        self.save_hf_ckpt, self.disable_ds_ckpt = save_hf_ckpt, disable_ds_ckpt
        self.args = strategy.args
        self.aux_loss = getattr(getattr(self.args, "model", None), "aux_loss_coef", 0) > 1e-8
        self.loggers = build_loggers(self.args, strategy.is_rank_0())

    # subclasses -------------------------------------------------------------
    @abstractmethod
    def train_micro_batch(self, batch, loss_info, device) -> tuple[torch.Tensor, dict]:
        """Returns (loss to back-propagate, dict of python floats to log)."""

    @abstractmethod
    def evaluate(self, eval_dataloader, steps: int = 0) -> dict: ...

    def micro_batches(self):
        """Iterator of (batch, loss_info); overridden where global loss normalisers are needed."""
        for b in self.train_dataloader:
            yield b, {}

    # loop -------------------------------------------------------------------
    def device(self):
        return next(self.model.parameters()).device

    def current_lr(self):
        eng = getattr(self.model, "engine", None)
        return eng.current_lr() if eng is not None else 0.0

    def fit(self, args, consumed_samples: int = 0, num_update_steps_per_epoch=None):
        if num_update_steps_per_epoch is None:
            num_update_steps_per_epoch = len(self.train_dataloader)
        if num_update_steps_per_epoch <= 0:
            raise ValueError(f"num_update_steps_per_epoch must be positive, got {num_update_steps_per_epoch}. "
                             "Check that your dataset is not smaller than train_batch_size.")
        if args.eval.steps == -1:
            args.eval.steps = num_update_steps_per_epoch
        if args.ckpt.save_steps == -1:
            args.ckpt.save_steps = float("inf")
        self.num_update_steps_per_epoch = num_update_steps_per_epoch
        gas = self.strategy.accumulated_gradient
        bs = args.train.batch_size
        step = consumed_samples // bs * gas + 1                       # 1-indexed micro-step counter
        start_epoch = consumed_samples // bs // num_update_steps_per_epoch
        consumed_samples %= num_update_steps_per_epoch * bs
        sums: dict[str, float] = {}
        for epoch in range(start_epoch, self.epochs):
            sampler = getattr(self.train_dataloader, "sampler", None)
            if isinstance(sampler, DistributedSampler):
                sampler.set_epoch(epoch, consumed_samples=consumed_samples if epoch == start_epoch else 0)
            self.model.train()
            dev = self.device()
            for batch, info in self.micro_batches():
                loss, logs = self.train_micro_batch(batch, info, dev)
                self.strategy.backward(loss, self.model, self.optimizer)
                self.strategy.optimizer_step(self.optimizer, self.model, self.scheduler)
                logs["lr"] = self.current_lr()
                logs["grad_norm"] = self.strategy.get_grad_norm(self.model)
                for k in self.MEAN_KEYS:
                    sums[k] = sums.get(k, 0.0) + logs[k]
                logs = self.strategy.all_reduce(logs)
                if step % gas == 0:
                    for k in self.MEAN_KEYS:
                        logs[f"{k}_mean"] = sums[k] / gas
                    sums = {}
                    global_step = step // gas
                    self.save_logs_and_checkpoints(args, global_step, None, logs,
                                                   {"consumed_samples": global_step * bs})
                step += 1
        for lg in self.loggers:
            lg.close()

    MEAN_KEYS: tuple = ("loss",)

    def save_logs_and_checkpoints(self, args, global_step, step_bar=None, logs_dict=None, client_states=None):
        logs_dict, client_states = logs_dict or {}, client_states or {}
        if global_step % args.logger.logging_steps == 0:
            for lg in self.loggers:
                lg.log_train(global_step, logs_dict)
            self.strategy.print(f"step {global_step}: " + ", ".join(f"{k}={v:.5g}" for k, v in logs_dict.items()))
        if global_step % args.eval.steps == 0 and self.eval_dataloader is not None and len(self.eval_dataloader) > 0:
            ev = self.evaluate(self.eval_dataloader, global_step)
            for lg in self.loggers:
                lg.log_eval(global_step, ev)
        if global_step % args.ckpt.save_steps == 0:
            tag = f"global_step{global_step}"
            if not self.disable_ds_ckpt:
                self.strategy.save_ckpt(self.model, args.ckpt.path, tag, args.ckpt.max_num, args.ckpt.max_mem, client_states)
            if self.save_hf_ckpt:
                self.strategy.save_model(self.model, self.tokenizer, os.path.join(args.ckpt.path, f"{tag}_hf"))


def left_pad_cat(a: torch.Tensor, b: torch.Tensor, pad_value) -> torch.Tensor:
    """Stack two (B, L) batches along dim 0, left-padding the shorter one."""
    L = max(a.shape[1], b.shape[1])
    f = lambda t: torch.nn.functional.pad(t, (L - t.shape[1], 0), value=pad_value)
    return torch.cat([f(a), f(b)], 0)


def right_pad_cat(a: torch.Tensor, b: torch.Tensor, pad_value) -> torch.Tensor:
    L = max(a.shape[1], b.shape[1])
    f = lambda t: torch.nn.functional.pad(t, (0, L - t.shape[1]), value=pad_value)
    return torch.cat([f(a), f(b)], 0)
