"""Declarative definition of the command-line surface shared by the entry points.

Flag names, defaults and meanings follow the reference CLIs (openrlhf/cli/train_{sft,rm,dpo,ppo_ray}.py) because they
are the public API; here they are data (tuples grouped by theme) instead of hundreds of ``add_argument`` lines.
Flags that configured machinery this framework replaces (``--ds.deepcompile``, ``--ds.zpg``, ``--vllm.sync_with_ray``,
``--use_ms`` ...) are still accepted so existing launch scripts keep working; they are reported once and ignored.
"""
from __future__ import annotations

import argparse
from datetime import datetime

BOOL = "bool"


def _add(parser: argparse.ArgumentParser, spec):
    name, typ, default, *rest = spec
    extra = rest[0] if rest else {}
    if typ == BOOL:
        parser.add_argument(name, action="store_true", default=bool(default), **extra)
    else:
        parser.add_argument(name, type=typ, default=default, **extra)


def add_flags(parser, *groups):
    seen = {a.option_strings[0] for a in parser._actions if a.option_strings}
    for g in groups:
        for spec in g:
            if spec[0] not in seen:
                _add(parser, spec)
                seen.add(spec[0])
    return parser


def optimizer_flags(prefix: str = "", adam_lr: float = 1e-6):
    """--{prefix}optim / adam.* / muon.* / scheduler / clipping (per entity in RL: prefix 'actor.' or 'critic.')."""
    p = prefix
    return [
        (f"--{p}optim", str, "adam", {"choices": ["adam", "muon"]}),
        (f"--{p}muon.lr", float, 0.02), (f"--{p}muon.momentum", float, 0.95), (f"--{p}muon.ns_steps", int, 5),
        (f"--{p}muon.nesterov", BOOL, True),
        (f"--{p}muon.no_nesterov", BOOL, False),
        (f"--{p}adam.lr", float, adam_lr), (f"--{p}adam.betas", float, (0.9, 0.95), {"nargs": 2}),
        (f"--{p}adam.eps", float, 1e-8), (f"--{p}adam.weight_decay", float, 0.0),
        (f"--{p}lr_scheduler", str, "cosine_with_min_lr"), (f"--{p}lr_warmup_ratio", float, 0.03),
        (f"--{p}min_lr_ratio", float, 0.1), (f"--{p}max_norm", float, 1.0),
    ]


ENGINE = [
    ("--local_rank", int, -1), ("--ds.zero_stage", int, 2), ("--ds.param_dtype", str, "bf16", {"choices": ["bf16", "fp16"]}),
    ("--ds.zpg", int, 1), ("--ds.adam_offload", BOOL, False), ("--ds.attn_implementation", str, "flash_attention_2"),
    ("--ds.experts_implementation", str, None), ("--ds.use_liger_kernel", BOOL, False),
    ("--ds.grad_accum_dtype", str, None), ("--ds.overlap_comm", BOOL, False), ("--ds.deepcompile", BOOL, False),
    ("--ds.tensor_parallel_size", int, 1), ("--ds.ring_attn_size", int, 1), ("--ds.ring_attn_head_stride", int, 1),
    # expert parallelism for mixture-of-experts models: this many consecutive data-parallel ranks split the experts of
    # every MoE layer between them (dispatch / combine over peer memory); the reference has no counterpart
    ("--ds.expert_parallel_size", int, 1),
    ("--ds.load_in_4bit", BOOL, False), ("--ds.lora.rank", int, 0), ("--ds.lora.alpha", int, 16),
    ("--ds.lora.target_modules", str, "all-linear", {"nargs": "*"}), ("--ds.lora.dropout", float, 0),
    ("--ds.packing_samples", BOOL, False), ("--ds.use_universal_ckpt", BOOL, False),
    ("--ds.value_head_prefix", str, "score"), ("--use_ms", BOOL, False),
]


def checkpoint_flags(path_default: str):
    return [
        ("--ckpt.output_dir", str, "./ckpt"), ("--ckpt.save_steps", int, -1), ("--ckpt.save_hf", BOOL, False),
        ("--ckpt.disable_ds", BOOL, False), ("--ckpt.path", str, path_default), ("--ckpt.max_num", int, 3),
        ("--ckpt.max_mem", int, int(1e8)), ("--ckpt.load_enable", BOOL, False),
    ]


def logger_flags(project: str, run_prefix: str):
    return [
        ("--logger.logging_steps", int, 1), ("--logger.wandb.key", str, None), ("--logger.wandb.org", str, None),
        ("--logger.wandb.group", str, None), ("--logger.wandb.project", str, project),
        ("--logger.wandb.run_name", str, f"{run_prefix}_{datetime.now().strftime('%m%dT%H:%M')}"),
        ("--logger.tensorboard_dir", str, None),
    ]


SPMD_TRAIN = [
    ("--train.seed", int, 42), ("--train.full_determinism_enable", BOOL, False),
    ("--train.batch_size", int, 128), ("--eval.steps", int, -1),
    ("--model.model_name_or_path", str, None), ("--model.gradient_checkpointing_enable", BOOL, False),
    ("--model.gradient_checkpointing_reentrant", BOOL, False), ("--model.aux_loss_coef", float, 0),
    ("--data.disable_fast_tokenizer", BOOL, False), ("--data.dataloader_num_workers", int, 0),
    ("--data.dataset", str, None), ("--data.dataset_probs", str, None), ("--eval.dataset", str, None),
    ("--data.dataset_split", str, "train"), ("--data.max_samples", int, 1000000),
    ("--data.apply_chat_template", BOOL, False), ("--data.tokenizer_chat_template", str, None),
]

IGNORED = ("ds.zpg", "ds.deepcompile", "ds.use_liger_kernel", "ds.overlap_comm", "ds.grad_accum_dtype",
           "ds.attn_implementation", "ds.experts_implementation", "use_ms", "vllm.sync_with_ray", "vllm.sync_backend",
           "ds.use_universal_ckpt", "local_rank")


def report_ignored(parser: argparse.ArgumentParser, ns) -> list[str]:
    """One line for every accepted-but-ignored flag that the user set to a non-default value."""
    flat = vars(ns)
    out = []
    for k in IGNORED:
        if k in flat and flat[k] != parser.get_default(k):
            out.append(k)
    if out:
        print("[Info] flags accepted for launch-script compatibility and ignored by this framework: "
              + ", ".join("--" + k for k in out))
    return out


def finalize(parser: argparse.ArgumentParser, argv=None):
    """Parse, fold --X.muon.no_nesterov into X.muon.nesterov, build the nested namespace."""
    from ..utils.config import hierarchize

    ns = parser.parse_args(argv)
    report_ignored(parser, ns)
    flat = vars(ns)
    for k in [k for k in flat if k.endswith("muon.no_nesterov")]:
        if flat[k]:
            flat[k.replace("no_nesterov", "nesterov")] = False
        del flat[k]
    for k in list(flat):
        if k.endswith("adam.betas") and flat[k] is not None:
            flat[k] = tuple(flat[k])
    return hierarchize(ns)


def optimizer_cfg(node, max_steps: int) -> dict:
    """Namespace holding optim/adam/muon/scheduler flags -> the cfg dict Strategy.prepare() expects."""
    adam = node.adam
    return {"optim": getattr(node, "optim", "adam"), "lr": adam.lr, "betas": tuple(adam.betas), "eps": adam.eps,
            "weight_decay": adam.weight_decay, "lr_scheduler": node.lr_scheduler,
            "lr_warmup_ratio": node.lr_warmup_ratio, "min_lr_ratio": node.min_lr_ratio, "max_steps": max_steps,
            "muon": vars(node.muon) if hasattr(node, "muon") else None}
