"""Multi-turn agent against a gym-style text environment (``reset() -> (obs, info)``,
``step(action) -> (obs, reward, terminated, truncated, info)``).

With the ``gem`` package installed the environment is ``gem.make(ENV_ID)`` (the reference example plays
"game:GuessTheNumber-v0", examples/python/agent_func_gem_multiturn.py:48-143); without it a built-in number-guessing
game with the same interface is used, so the example runs offline. The policy's answer is taken from the last
``\\boxed{...}`` of its turn; every environment message is wrapped in a chat turn before it is appended to the
conversation.
"""
from __future__ import annotations

import random
import re
import time

import torch

from openrlhf.utils.agent import AgentInstanceBase, MultiTurnAgentExecutor

ENV_ID = "game:GuessTheNumber-v0"
MAX_TURNS = 8


class GuessTheNumber:
    """Stand-in with the interface of a GEM environment."""

    def __init__(self, lo: int = 1, hi: int = 20, max_turns: int = MAX_TURNS, seed=None):
        self.lo, self.hi, self.max_turns = lo, hi, max_turns
        self.rng = random.Random(seed)
        self.target, self.turn = lo, 0

    def reset(self):
        self.target, self.turn = self.rng.randint(self.lo, self.hi), 0
        return (f"I picked a number between {self.lo} and {self.hi}. Guess it in at most {self.max_turns} turns. "
                "Give each guess as \\boxed{number}."), {}

    def step(self, action: str):
        self.turn += 1
        m = re.findall(r"\\boxed\{\s*(-?\d+)\s*\}", action)
        if not m:
            return "Your turn had no \\boxed{number}.", -0.1, False, self.turn >= self.max_turns, {"invalid": 1.0}
        guess = int(m[-1])
        if guess == self.target:
            return "Correct.", 1.0, True, False, {"invalid": 0.0}
        hint = "higher" if guess < self.target else "lower"
        return f"The number is {hint} than {guess}.", 0.0, False, self.turn >= self.max_turns, {"invalid": 0.0}


def make_env():
    try:
        import gem

        return gem.make(ENV_ID, seed=time.time_ns())
    except ImportError:
        return GuessTheNumber(seed=time.time_ns())


def user_turn(text: str) -> str:
    """A ChatML user turn followed by the opening of the assistant turn (Qwen-style templates)."""
    return f"<|im_start|>user\n{text}<|im_end|>\n<|im_start|>assistant\n"


class AgentInstance(AgentInstanceBase):
    def __init__(self, *args, **kwargs):
        self.env = make_env()
        self.turns = 0

    async def reset(self, states: dict, **kwargs):
        obs, _ = self.env.reset()
        self.turns = 0
        return {"observation": user_turn(obs)}

    async def step(self, states: dict, **kwargs):
        self.turns += 1
        obs, reward, terminated, truncated, info = self.env.step(states["action_text"])
        done = bool(terminated or truncated)
        r = torch.tensor(float(reward))
        return {
            "rewards": r,
            "scores": torch.tensor(1.0 if terminated and float(reward) > 0 else 0.0),
            "environment_feedback": "" if done else "<|im_end|>\n" + user_turn(obs),
            "done": done,
            "sampling_params": states.get("sampling_params"),
            "extra_logs": {"turns": torch.tensor(float(self.turns)),
                           "invalid": torch.tensor(float(info.get("invalid", 0.0)) if isinstance(info, dict) else 0.0)},
        }


class AgentExecutor(MultiTurnAgentExecutor):
    def __init__(self):
        super().__init__(AgentInstance)
