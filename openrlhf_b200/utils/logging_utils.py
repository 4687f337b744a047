"""Console logger format and the wandb / TensorBoard writers (openrlhf/utils/logging_utils.py:10-138)."""
from __future__ import annotations

import logging
import os
import sys
from typing import Any, Dict

_FORMAT = "%(levelname)s %(asctime)s %(filename)s:%(lineno)d] %(message)s"
_DATE_FORMAT = "%m-%d %H:%M:%S"


class NewLineFormatter(logging.Formatter):
    """Repeats the prefix on every line of a multi-line message."""

    def format(self, record):
        msg = super().format(record)
        if record.message:
            prefix = msg.split(record.message)[0]
            msg = msg.replace("\n", "\r\n" + prefix)
        return msg


_root = logging.getLogger("openrlhf")
_configured = False


def _setup_logger():
    global _configured
    if _configured:
        return
    _root.setLevel(logging.DEBUG)
    h = logging.StreamHandler(sys.stdout)
    h.flush = sys.stdout.flush
    h.setLevel(logging.INFO)
    h.setFormatter(NewLineFormatter(_FORMAT, datefmt=_DATE_FORMAT))
    _root.addHandler(h)
    _root.propagate = False
    _configured = True


def init_logger(name: str):
    _setup_logger()
    lg = logging.getLogger(name)
    lg.setLevel(logging.DEBUG)
    if not any(isinstance(h, logging.StreamHandler) for h in lg.handlers):
        for h in _root.handlers:
            lg.addHandler(h)
    lg.propagate = False
    return lg


class WandbLogger:
    """train/* against train/global_step, eval/* against eval/epoch, plus a growing table of generated samples."""

    def __init__(self, args) -> None:
        import wandb

        w = args.logger.wandb
        if not wandb.api.api_key:
            wandb.login(key=w.key)
        wandb.init(entity=w.org, project=w.project, group=w.group, name=w.run_name, config=args.__dict__, reinit=True)
        wandb.define_metric("train/global_step")
        wandb.define_metric("train/*", step_metric="train/global_step", step_sync=True)
        wandb.define_metric("eval/epoch")
        wandb.define_metric("eval/*", step_metric="eval/epoch", step_sync=True)
        self.handle = wandb
        self.samples_table = wandb.Table(columns=["global_step", "text", "reward"])

    def log_train(self, global_step: int, logs_dict: Dict[str, Any]) -> None:
        logs = dict(logs_dict)
        sample = logs.pop("generated_samples", None)
        if sample:
            t = self.handle.Table(columns=self.samples_table.columns, data=self.samples_table.data)
            t.add_data(global_step, *sample)
            self.samples_table = t
            self.handle.log({"train/generated_samples": t})
        self.handle.log({f"train/{k}": v for k, v in {**logs, "global_step": global_step}.items() if v is not None})

    def log_eval(self, global_step: int, logs_dict: Dict[str, Any]) -> None:
        self.handle.log({f"eval/{k}": v for k, v in {**logs_dict, "global_step": global_step}.items() if v is not None})

    def close(self) -> None:
        self.handle.finish()


class TensorboardLogger:
    def __init__(self, args) -> None:
        from torch.utils.tensorboard import SummaryWriter

        os.makedirs(args.logger.tensorboard_dir, exist_ok=True)
        self.writer = SummaryWriter(log_dir=os.path.join(args.logger.tensorboard_dir, args.logger.wandb.run_name))

    def log_train(self, global_step: int, logs_dict: Dict[str, Any]) -> None:
        for k, v in logs_dict.items():
            if v is None:
                continue
            if k == "generated_samples":
                text, reward = v
                self.writer.add_text("train/generated_samples", f"Sample:\n{text}\n\nReward: {reward:.4f}", global_step)
            else:
                self.writer.add_scalar(f"train/{k}", v, global_step)

    def log_eval(self, global_step: int, logs_dict: Dict[str, Any]) -> None:
        for k, v in logs_dict.items():
            if v is not None:
                self.writer.add_scalar(f"eval/{k}", v, global_step)

    def close(self) -> None:
        self.writer.close()


class JsonlLogger:
    """Always-available sink: one JSON object per logged step (used when neither wandb nor TensorBoard is set)."""

    def __init__(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.f = open(path, "a")

    def _w(self, kind, step, logs):
        import json

        clean = {k: (v if isinstance(v, (int, float, str)) or v is None else str(v)) for k, v in logs.items()}
        self.f.write(json.dumps({"kind": kind, "step": step, **clean}) + "\n")
        self.f.flush()

    def log_train(self, global_step, logs_dict):
        self._w("train", global_step, logs_dict)

    def log_eval(self, global_step, logs_dict):
        self._w("eval", global_step, logs_dict)

    def close(self):
        self.f.close()


def build_loggers(args, is_rank_0: bool = True) -> list:
    """Loggers requested by the flag tree (--logger.wandb.key, --logger.tensorboard_dir), on rank 0 only."""
    out = []
    if not is_rank_0:
        return out
    lg = getattr(args, "logger", None)
    if lg is None:
        return out
    if getattr(getattr(lg, "wandb", None), "key", None):
        out.append(WandbLogger(args))
    if getattr(lg, "tensorboard_dir", None):
        out.append(TensorboardLogger(args))
    return out
