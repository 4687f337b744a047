"""Example rule reward: ``reward_func(queries, prompts, labels, **kwargs)`` returns rewards (used for advantages),
scores (used for dynamic filtering, in [0, 1]) and optional extra logs. This toy rule rewards responses whose token
ids (the synthetic tokenizer renders ids as text) are mostly even."""
import torch


def reward_func(queries, prompts, labels, **kwargs):
    rewards = []
    for q, p in zip(queries, prompts):
        resp = q[len(p):].split()
        vals = [int(t) for t in resp if t.lstrip("-").isdigit()]
        rewards.append(sum(v % 2 == 0 for v in vals) / max(len(vals), 1))
    r = torch.tensor(rewards, dtype=torch.float32)
    return {"rewards": r, "scores": r, "extra_logs": {"even_fraction": r}}
