"""DPO trainer (openrlhf/trainer/dpo_trainer.py:106-382): policy forward with gradients and frozen-reference forward on
one concatenated, right-padded chosen+rejected batch; summed response log-probs feed DPO / IPO / cDPO; optional NLL
regulariser on the chosen responses and MoE auxiliary loss."""
from __future__ import annotations

import torch

from ..models.loss import DPOLoss
from .base import SPMDTrainer, right_pad_cat


class DPOTrainer(SPMDTrainer):
    MEAN_KEYS = ("loss", "acc")

    def __init__(self, model, ref_model, strategy, tokenizer, optim, train_dataloader, eval_dataloader, scheduler,
                 max_norm: float = 0.5, beta: float = 0.01, max_epochs: int = 2, save_hf_ckpt: bool = False,
                 disable_ds_ckpt: bool = False) -> None:
        super().__init__(model, strategy, optim, train_dataloader, eval_dataloader, scheduler, max_norm, max_epochs,
                         tokenizer, save_hf_ckpt, disable_ds_ckpt)
        self.ref_model, self.beta = ref_model, beta
        m = self.args.model
        self.loss_fn = DPOLoss(beta, getattr(m, "label_smoothing", 0.0), getattr(m, "ipo_enable", False))
        self.nll_loss = getattr(m, "nll_loss_coef", 0) > 1e-8

    def concatenated_inputs(self, chosen_ids, c_mask, reject_ids, r_mask, prompt_id_lens):
        return (right_pad_cat(chosen_ids, reject_ids, self.tokenizer.pad_token_id), right_pad_cat(c_mask, r_mask, 0),
                list(prompt_id_lens) * 2)

    @staticmethod
    def _get_batch_logps(per_token_logps, attention_mask, prompt_id_lens):
        """Sum and mean of response-token log-probs per row (prompt positions and padding masked out)."""
        m = attention_mask.clone().bool()
        for row, n in zip(m, prompt_id_lens):
            row[:n] = False
        m = m[:, 1:].float()
        s = (per_token_logps * m).sum(-1)
        return s, s / m.sum(-1).clamp_min(1)

    def concatenated_forward(self, model, chosen_ids, c_mask, reject_ids, r_mask, prompt_id_lens):
        ids, att, plens = self.concatenated_inputs(chosen_ids, c_mask, reject_ids, r_mask, prompt_id_lens)
        logps, out = model(ids, attention_mask=att, return_output=True, return_logprobs=True,
                           ring_attn_group=self.strategy.ring_attn_group)
        sums, means = self._get_batch_logps(logps, att, plens)
        n = chosen_ids.shape[0]
        aux = out.aux_loss if getattr(out, "aux_loss", None) is not None else []
        return sums[:n], sums[n:], aux, -means[:n].mean()

    def _both(self, batch, dev, grad=True):
        c_ids, c_m, r_ids, r_m, plens = batch
        t = [x.squeeze(1).to(dev) for x in (c_ids, c_m, r_ids, r_m)]
        pc, pr, aux, nll = self.concatenated_forward(self.model, *t, plens)
        with torch.no_grad():
            rc, rr, _, _ = self.concatenated_forward(self.ref_model, *t, plens)
        pref, cw, rj = self.loss_fn(pc, pr, rc, rr)
        return pref, cw, rj, aux, nll

    def train_micro_batch(self, batch, info, dev):
        pref, cw, rj, aux, nll = self._both(batch, dev)
        loss = pref
        if self.aux_loss:
            loss = loss + aux * self.args.model.aux_loss_coef
        if self.nll_loss:
            loss = loss + nll * self.args.model.nll_loss_coef
        logs = {"loss": pref.item(), "acc": (cw > rj).float().mean().item(), "chosen_reward": cw.mean().item(),
                "reject_reward": rj.mean().item()}
        if self.nll_loss:
            logs["nll_loss"] = nll.item()
        return loss, logs

    @torch.no_grad()
    def evaluate(self, eval_dataloader, steps: int = 0) -> dict:
        self.model.eval()
        dev = self.device()
        acc = tot = 0.0
        n = 0
        for batch in eval_dataloader:
            pref, cw, rj, _, _ = self._both(batch, dev)
            acc += (cw > rj).float().mean().item()
            tot += pref.item()
            n += 1
        logs = self.strategy.all_reduce({"eval_loss": tot / max(n, 1), "acc_mean": acc / max(n, 1)})
        self.strategy.print(f"eval at step {steps}: {logs}")
        self.model.train()
        return logs
