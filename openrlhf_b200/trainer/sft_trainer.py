"""Supervised fine-tuning trainer (openrlhf/trainer/sft_trainer.py:104-285): per optimizer step one global token-mean
of -log p over response tokens, accumulated over micro-batches and data-parallel ranks."""
from __future__ import annotations

import torch

from ..models.loss import SFTLoss
from ..utils.loss_utils import iter_grad_accum_global_norm
from .base import SPMDTrainer


class SFTTrainer(SPMDTrainer):
    MEAN_KEYS = ("gpt_loss",)

    def __init__(self, model, strategy, optim, train_dataloader, eval_dataloader, scheduler, max_norm: float = 1,
                 pretrain_mode: bool = False, batch_size: int = 1, max_epochs: int = 2, tokenizer=None,
                 save_hf_ckpt: bool = False, disable_ds_ckpt: bool = False) -> None:
        super().__init__(model, strategy, optim, train_dataloader, eval_dataloader, scheduler, max_norm, max_epochs,
                         tokenizer, save_hf_ckpt, disable_ds_ckpt)
        self.pretrain_mode, self.batch_size = pretrain_mode, batch_size
        self.loss_fn = SFTLoss()

    def micro_batches(self):
        shifted_mask = lambda b: b[2].squeeze(1)[:, :-1]
        yield from iter_grad_accum_global_norm(self.train_dataloader, self.strategy, self.strategy.accumulated_gradient,
                                               shifted_mask)

    def _logps(self, batch, dev):
        ids, att, lm = (t.to(dev).squeeze(1) for t in batch)
        logps, out = self.model(ids, attention_mask=att, return_output=True, return_logprobs=True,
                                ring_attn_group=self.strategy.ring_attn_group)
        return logps, lm[:, :-1], out

    def train_micro_batch(self, batch, info, dev):
        logps, mask, out = self._logps(batch, dev)
        gpt_loss = self.loss_fn(logps, mask, **info)
        loss = gpt_loss
        logs = {"gpt_loss": gpt_loss.item()}
        if self.aux_loss:
            loss = loss + out.aux_loss * self.args.model.aux_loss_coef
            logs["aux_loss"] = float(out.aux_loss)
        return loss, logs

    @torch.no_grad()
    def evaluate(self, eval_dataloader, steps: int = 0) -> dict:
        self.model.eval()
        dev = self.device()
        tot, n = 0.0, 0
        for batch in eval_dataloader:
            logps, mask, _ = self._logps(batch, dev)
            tot += self.loss_fn(logps, mask).item()
            n += 1
        logs = self.strategy.all_reduce({"eval gpt_loss": tot / max(n, 1)})
        self.strategy.print(f"eval at step {steps}: {logs}")
        self.model.train()
        return logs
