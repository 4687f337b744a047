"""Reward-model trainer (openrlhf/trainer/rm_trainer.py:105-363): chosen and rejected sequences go through the model
in one concatenated, left-padded batch; pairwise sigmoid or log-exp loss with optional margin; evaluation computes the
reward mean / std over the eval set and stores them in the model config (they end up in config.json)."""
from __future__ import annotations

import torch

from ..models.loss import LogExpLoss, PairWiseLoss
from .base import SPMDTrainer, left_pad_cat


class RewardModelTrainer(SPMDTrainer):
    MEAN_KEYS = ("loss", "acc")

    def __init__(self, model, strategy, optim, train_dataloader, eval_dataloader, scheduler, tokenizer,
                 max_norm: float = 0.5, max_epochs: int = 2, loss: str = "sigmoid", disable_ds_ckpt: bool = False,
                 save_hf_ckpt: bool = False) -> None:
        super().__init__(model, strategy, optim, train_dataloader, eval_dataloader, scheduler, max_norm, max_epochs,
                         tokenizer, save_hf_ckpt, disable_ds_ckpt)
        self.loss_fn = PairWiseLoss() if loss == "sigmoid" else LogExpLoss()
        self.strategy.print("LogSigmoid Loss" if loss == "sigmoid" else "LogExp Loss")
        self.margin_loss = getattr(self.args.model, "margin_loss_enable", False)
        self.compute_fp32_loss = getattr(self.args.model, "compute_fp32_loss_enable", False)

    def concatenated_inputs(self, chosen_ids, c_mask, reject_ids, r_mask):
        return (left_pad_cat(chosen_ids, reject_ids, self.tokenizer.pad_token_id), left_pad_cat(c_mask, r_mask, 0))

    def concatenated_forward(self, model, chosen_ids, c_mask, reject_ids, r_mask):
        ids, att = self.concatenated_inputs(chosen_ids, c_mask, reject_ids, r_mask)
        values, out = model(ids, attention_mask=att, return_output=True, ring_attn_group=self.strategy.ring_attn_group)
        n = chosen_ids.shape[0]
        return values[:n], values[n:], out.get("aux_loss", []) if isinstance(out, dict) else []

    def _pair(self, batch, dev):
        c_ids, c_m, r_ids, r_m, margin = batch
        c, r, aux = self.concatenated_forward(self.model, c_ids.squeeze(1).to(dev), c_m.squeeze(1).to(dev),
                                              r_ids.squeeze(1).to(dev), r_m.squeeze(1).to(dev))
        margin = torch.tensor(margin, device=dev, dtype=c.dtype) if self.margin_loss else None
        if self.compute_fp32_loss:
            c, r = c.float(), r.float()
        return c, r, margin, aux

    def train_micro_batch(self, batch, info, dev):
        c, r, margin, aux = self._pair(batch, dev)
        pref = self.loss_fn(c, r, margin)
        loss = pref + (aux * self.args.model.aux_loss_coef if self.aux_loss else 0)
        return loss, {"loss": pref.item(), "acc": (c > r).float().mean().item(), "chosen_reward": c.mean().item(),
                      "reject_reward": r.mean().item()}

    @torch.no_grad()
    def evaluate(self, eval_dataloader, steps: int = 0) -> dict:
        self.model.eval()
        dev = self.device()
        acc = loss_sum = 0.0
        rewards = []
        for batch in eval_dataloader:
            c, r, margin, _ = self._pair(batch, dev)
            loss_sum += self.loss_fn(c, r, margin).item()
            acc += (c > r).float().mean().item()
            rewards += [c.flatten(), r.flatten()]
        n = max(len(eval_dataloader), 1)
        allr = self.strategy.all_gather(torch.cat(rewards).float())
        mean, std = allr.mean(), allr.std().clamp(min=1e-8) if allr.numel() > 1 else torch.tensor(1.0)
        self.strategy.print("Set reward mean std")
        inner = getattr(self.model, "module", self.model)
        inner.cfg.mean, inner.cfg.std = mean.item(), float(std)
        inner.mean[0], inner.std[0] = mean.item(), float(std)
        logs = self.strategy.all_reduce({"eval_loss": loss_sum / n, "acc_mean": acc / n, "reward_mean": mean.item(),
                                         "reward_std": float(std)})
        hist = torch.histogram(allr.cpu(), bins=10, range=(-10, 10), density=True)[0] * 2
        self.strategy.print("histgram", hist)
        self.model.train()
        return logs
