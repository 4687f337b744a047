"""Dataset loading and blending (openrlhf/datasets/utils.py:10-99): comma-separated sources, optional ``path@data_dir``,
json/jsonl/csv/parquet/arrow files, ``load_from_disk`` directories, hub names, python loading scripts, concatenation or
probability interleaving. Adds ``synthetic://`` sources that need no files (benchmarks and tests run offline)."""
from __future__ import annotations

import os
import random
from urllib.parse import parse_qs, urlparse


def exist_and_not_none(d, key) -> bool:
    return key in d and d[key] is not None


class ListDataset(list):
    """Minimal stand-in for a ``datasets.Dataset``: a list of dict rows with select / map / filter / column access."""

    @property
    def column_names(self):
        return list(self[0].keys()) if len(self) else []

    def select(self, idx):
        return ListDataset(self[i] for i in idx)

    def map(self, fn, remove_columns=None, num_proc=None, **_kw):
        out = []
        for row in self:
            new = fn(dict(row))
            keep = {k: v for k, v in row.items() if not remove_columns or k not in remove_columns}
            keep.update(new)
            out.append(keep)
        return ListDataset(out)

    def filter(self, fn, **_kw):
        return ListDataset(r for r in self if fn(r))

    def column(self, name):
        return [r[name] for r in self]

    def __getitem__(self, key):
        if isinstance(key, str):
            return [r[key] for r in self]
        return super().__getitem__(key)


def synthetic_dataset(spec: str) -> ListDataset:
    """``synthetic://prompts?n=128&len=512&vocab=151936&seed=0``: rows {"input": "<ids>", "label": "<ids>"} whose text
    is a space-separated list of token ids (pairs with utils.SyntheticTokenizer). ``synthetic://pairs?...`` yields
    {"prompt","chosen","rejected"} rows and ``synthetic://sft`` {"input","output"} rows;
    ``synthetic://vlm_prompts?...&image=56`` prepends an ``<image>`` tag and attaches one random RGB image of that
    side length per row (pairs with utils.SyntheticProcessor)."""
    u = urlparse(spec)
    q = {k: v[0] for k, v in parse_qs(u.query).items()}
    n, ln, vocab, seed = int(q.get("n", 64)), int(q.get("len", 64)), int(q.get("vocab", 1024)), int(q.get("seed", 0))
    out_len = int(q.get("out_len", max(ln // 2, 1)))
    rng = random.Random(seed)
    ids = lambda k: " ".join(str(rng.randrange(3, vocab)) for _ in range(k))
    kind = u.netloc or u.path.strip("/")
    rows = []
    for i in range(n):
        if kind in ("pairs", "preference"):
            rows.append({"prompt": ids(ln), "chosen": ids(out_len), "rejected": ids(out_len)})
        elif kind == "sft":
            rows.append({"input": ids(ln), "output": ids(out_len)})
        elif kind == "vlm_prompts":
            from PIL import Image

            side = int(q.get("image", 56))
            img = Image.frombytes("RGB", (side, side), bytes(rng.randrange(256) for _ in range(3 * side * side)))
            rows.append({"input": "<image> " + ids(ln), "label": str(i % 7), "datasource": "synthetic", "images": [img]})
        else:
            rows.append({"input": ids(ln), "label": str(i % 7), "datasource": "synthetic"})
    return ListDataset(rows)


def _load_one(path: str, data_dir, strategy):
    if path.startswith("synthetic://"):
        return synthetic_dataset(path)
    from datasets import load_dataset, load_from_disk

    ext = os.path.splitext(path)[-1].lower()
    base = os.path.basename(path)
    if ext == ".py" or (os.path.isdir(path) and os.path.exists(os.path.join(path, f"{base}.py"))):
        return load_dataset(path, trust_remote_code=True)
    if ext in (".json", ".jsonl", ".csv", ".parquet", ".arrow"):
        kind = "json" if ext == ".jsonl" else ext.strip(".")
        return load_dataset(kind, data_files=path)
    if os.path.isdir(path):
        try:
            return load_from_disk(path)
        except Exception as e:  # noqa: BLE001
            strategy.print(f"load_from_disk({path}) failed ({e}); trying load_dataset")
            return load_dataset(path, data_dir=data_dir)
    if getattr(getattr(strategy, "args", None), "use_ms", False):
        from modelscope.msdatasets import MsDataset

        ns, name = path.split("/")
        return MsDataset.load(name, namespace=ns)
    return load_dataset(path, data_dir=data_dir)


def blending_datasets(datasets: str, probabilities: str | None = None, strategy=None, seed: int = 42,
                      max_count: int = int(1e8), stopping_strategy: str = "all_exhausted", dataset_split: str = "train"):
    names = [d.strip() for d in datasets.split(",")]
    probs = None
    if probabilities is not None:
        probs = [float(p) for p in str(probabilities).split(",")]
        if len(probs) != len(names):
            raise AssertionError("one probability per dataset is required")
    parts = []
    for name in names:
        strategy.print(f"dataset: {name}")
        path, _, data_dir = name.partition("@")
        data = _load_one(path.strip(), data_dir.strip() or None, strategy)
        if dataset_split and not isinstance(data, ListDataset) and dataset_split in data:
            data = data[dataset_split]
        data = data.select(range(min(int(max_count), len(data))))
        parts.append(data)
    if all(isinstance(p, ListDataset) for p in parts):
        if probs is None:
            return ListDataset(r for p in parts for r in p)
        rng = random.Random(seed)
        iters = [iter(p) for p in parts]
        alive = [True] * len(parts)
        done_once = [False] * len(parts)
        out = []
        while not all(done_once):
            i = rng.choices(range(len(parts)), probs)[0]
            try:
                out.append(next(iters[i]))
            except StopIteration:
                done_once[i] = True
                iters[i] = iter(parts[i])
        return ListDataset(out)
    from datasets import concatenate_datasets, interleave_datasets

    if probs is None:
        return concatenate_datasets(parts)
    return interleave_datasets(parts, probabilities=probs, seed=seed, stopping_strategy=stopping_strategy)
