"""Rule reward for math prompts: 1.0 when the last \\boxed{...} answer of the response is equivalent to the label
(string normalisation first, symbolic comparison second), else 0.0. Same calling convention as reward_func.py:
``reward_func(queries, prompts, labels, **kwargs) -> {"rewards", "scores", "extra_logs"}``
(the reference ships examples/python/math_reward_func.py with this interface)."""
import torch

from openrlhf_b200.utils.math_utils import extract_boxed_answer, grade_answer


def reward_func(queries, prompts, labels, **kwargs):
    rewards = []
    for q, p, label in zip(queries, prompts, labels):
        response = q[len(p):] if q.startswith(p) else q
        answer = extract_boxed_answer(response)
        rewards.append(1.0 if (answer is not None and grade_answer(answer, str(label))) else 0.0)
    r = torch.tensor(rewards, dtype=torch.float32)
    return {"rewards": r, "scores": r, "extra_logs": {"accuracy": r}}
