"""Dotted command-line flags -> nested namespaces (``--actor.adam.lr`` becomes ``args.actor.adam.lr``), the flag
system of the reference (openrlhf/utils/config.py:12-26)."""
from __future__ import annotations

from types import SimpleNamespace


def hierarchize(args):
    """Turn a flat namespace whose attribute names contain dots into a tree of SimpleNamespace objects."""
    tree: dict = {}
    for dotted, value in vars(args).items():
        node = tree
        *parents, leaf = dotted.split(".")
        for p in parents:
            nxt = node.get(p)
            if not isinstance(nxt, dict):
                nxt = node[p] = {}
            node = nxt
        node[leaf] = value

    def to_ns(x):
        return SimpleNamespace(**{k: to_ns(v) for k, v in x.items()}) if isinstance(x, dict) else x

    return to_ns(tree)


def flatten(ns, prefix: str = "") -> dict:
    """Inverse of hierarchize: nested namespaces -> {dotted name: value}."""
    out = {}
    for k, v in vars(ns).items():
        name = f"{prefix}{k}"
        if isinstance(v, SimpleNamespace):
            out.update(flatten(v, name + "."))
        else:
            out[name] = v
    return out
