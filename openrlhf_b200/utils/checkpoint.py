"""Sharded training-state checkpoints and their rotation policy.

Format (world-size agnostic, replaces DeepSpeed's ``engine.save_checkpoint`` used at
openrlhf/utils/deepspeed/deepspeed.py:679-782):

    <save_dir>/<tag>/shard_{rank:05d}.safetensors   fp32 master / exp_avg / exp_avg_sq of the rank's flat slice
    <save_dir>/<tag>/manifest.json                  world size, shard size, parameter table (name -> offset, shape),
                                                    optimizer step, scheduler state, client_state
    <save_dir>/<tag>/metric.json                    {"metric_key", "metric_value"} written after a successful save
    <save_dir>/latest                               text file with the newest tag

Because every shard is a contiguous slice ``[lo, hi)`` of one flat index space, loading on a different number of
ranks only needs interval arithmetic (``load_sharded`` reads the overlapping pieces of the old shards).
Rotation: a new ``best*`` checkpoint replaces older best ones; regular checkpoints are evicted while there are
``max_num`` of them or the directory exceeds ``max_mem`` GiB, no-metric first, then worst metric, then oldest; best
checkpoints are never evicted and do not count.
"""
from __future__ import annotations

import json
import os
import shutil

import torch

METRIC_FILE = "metric.json"


def write_metric(ckpt_dir: str, value, key=None) -> None:
    os.makedirs(ckpt_dir, exist_ok=True)
    with open(os.path.join(ckpt_dir, METRIC_FILE), "w") as f:
        json.dump({"metric_key": key, "metric_value": value}, f, indent=2, sort_keys=True)


def read_metric(ckpt_dir: str):
    try:
        with open(os.path.join(ckpt_dir, METRIC_FILE)) as f:
            v = json.load(f).get("metric_value")
        return None if v is None else float(v)
    except (OSError, ValueError, TypeError, AttributeError):
        return None


def _dir_bytes(path: str) -> int:
    return sum(os.path.getsize(os.path.join(d, f)) for d, _, fs in os.walk(path) for f in fs)


def rotate(save_dir: str, tag: str | None, max_num: int = 3, max_mem: float = 1000, log=print) -> list[str]:
    """Apply the rotation policy *before* saving `tag`. Returns the deleted directories."""
    os.makedirs(save_dir, exist_ok=True)
    is_best = tag is not None and tag.startswith("best")
    deleted = []
    if is_best:
        for d in os.listdir(save_dir):
            p = os.path.join(save_dir, d)
            if d.startswith("best") and d != tag and os.path.isdir(p):
                shutil.rmtree(p)
                deleted.append(p)
                log(f"Removed old best checkpoint {p}")
    limit = max_mem * 1024 ** 3
    while True:
        subdirs = [os.path.join(save_dir, d) for d in os.listdir(save_dir) if os.path.isdir(os.path.join(save_dir, d))]
        regular = [p for p in subdirs if not os.path.basename(p).startswith("best")]
        too_many = (len(regular) - max_num + 1 > 0) and not is_best
        too_big = sum(_dir_bytes(p) for p in subdirs) > limit
        if not (too_many or too_big) or not regular:
            break
        def rank_key(p):
            m = read_metric(p)
            return (m is not None, m if m is not None else float("-inf"), os.path.getmtime(p))
        victim = min(regular, key=rank_key)
        shutil.rmtree(victim)
        deleted.append(victim)
        log(f"Deleted checkpoint {victim}")
    return deleted


def save_sharded(engine, save_dir: str, tag: str, client_state: dict | None = None, save_latest: bool = True,
                 rank: int = 0, world: int = 1) -> str:
    from .st_io import available as _native_st, save_file as _native_save

    if _native_st():
        save_file = _native_save          # parallel native writer, same file format
    else:
        from safetensors.torch import save_file

    d = os.path.join(save_dir, tag)
    os.makedirs(d, exist_ok=True)
    st = engine.shard_state()
    save_file({"master": st["master"].detach().cpu().contiguous(), "exp_avg": st["exp_avg"].detach().cpu().contiguous(),
               "exp_avg_sq": st["exp_avg_sq"].detach().cpu().contiguous()},
              os.path.join(d, f"shard_{rank:05d}.safetensors"), metadata={"lo": str(st["lo"]), "hi": str(st["hi"])})
    if rank == 0:
        manifest = {
            "format": "openrlhf_b200.sharded.v1", "world_size": world, "shard_size": st["shard_size"],
            "total_numel": st["total_numel"], "opt_step": st["opt_step"],
            "scheduler": engine.scheduler.state_dict() if engine.scheduler is not None else None,
            "params": {s.name: {"offset": s.offset, "numel": s.numel, "shape": list(s.shape)} for s in engine.model.specs},
            "client_state": _jsonable(client_state or {}),
        }
        with open(os.path.join(d, "manifest.json"), "w") as f:
            json.dump(manifest, f, indent=1)
        if save_latest:
            with open(os.path.join(save_dir, "latest"), "w") as f:
                f.write(tag)
    return d


def _jsonable(x):
    if isinstance(x, dict):
        return {str(k): _jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    if isinstance(x, torch.Tensor):
        # kept as a tensor through the round trip (a dataloader's generator state must come back as a ByteTensor)
        return {"__tensor__": x.detach().cpu().tolist(), "dtype": str(x.dtype).replace("torch.", "")}
    if isinstance(x, (int, float, str, bool)) or x is None:
        return x
    return repr(x)


def _from_jsonable(x):
    if isinstance(x, dict):
        if set(x) == {"__tensor__", "dtype"}:
            return torch.tensor(x["__tensor__"], dtype=getattr(torch, x["dtype"]))
        return {k: _from_jsonable(v) for k, v in x.items()}
    if isinstance(x, list):
        return [_from_jsonable(v) for v in x]
    return x


def resolve_tag(load_dir: str, tag: str | None) -> str | None:
    if tag is not None:
        return tag if os.path.isdir(os.path.join(load_dir, tag)) else None
    latest = os.path.join(load_dir, "latest")
    if os.path.exists(latest):
        t = open(latest).read().strip()
        if os.path.isdir(os.path.join(load_dir, t)):
            return t
    return None


def load_sharded(engine, load_dir: str, tag: str | None = None, load_optimizer_states: bool = True,
                 load_lr_scheduler_states: bool = True):
    """Restore this rank's slice from a checkpoint written by any number of ranks. Returns (path, client_state) or
    (None, {}) when nothing is found."""
    from safetensors import safe_open

    tag = resolve_tag(load_dir, tag)
    if tag is None:
        return None, {}
    d = os.path.join(load_dir, tag)
    with open(os.path.join(d, "manifest.json")) as f:
        man = json.load(f)
    names = {s.name: (s.offset, s.numel) for s in engine.model.specs}
    for k, v in man["params"].items():
        if k not in names or names[k] != (v["offset"], v["numel"]):
            raise ValueError(f"checkpoint parameter table does not match the model at {k}")
    old_per, old_world = man["shard_size"], man["world_size"]
    lo, hi = engine.lo, engine.hi
    bufs = {k: torch.zeros(hi - lo, dtype=torch.float32) for k in ("master", "exp_avg", "exp_avg_sq")}
    for r in range(old_world):
        a, b = r * old_per, (r + 1) * old_per
        x, y = max(a, lo), min(b, hi)
        if x >= y:
            continue
        with safe_open(os.path.join(d, f"shard_{r:05d}.safetensors"), framework="pt", device="cpu") as h:
            for k in bufs:
                if k != "master" and not load_optimizer_states:
                    continue
                bufs[k][x - lo:y - lo] = h.get_slice(k)[x - a:y - a]
    cur = engine.shard_state()               # tensors on the device, or on the host while the states are offloaded
    dev = engine.device
    engine.load_shard_state(bufs["master"].to(dev),
                            bufs["exp_avg"].to(dev) if load_optimizer_states else cur["exp_avg"].to(dev),
                            bufs["exp_avg_sq"].to(dev) if load_optimizer_states else cur["exp_avg_sq"].to(dev),
                            man["opt_step"] if load_optimizer_states else engine.opt_step)
    if load_lr_scheduler_states and engine.scheduler is not None and man.get("scheduler"):
        engine.scheduler.load_state_dict(man["scheduler"])
    return d, _from_jsonable(man.get("client_state", {}))
