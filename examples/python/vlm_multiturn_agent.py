"""Multi-turn agent whose observations contain images, both in the dataset prompt and in the environment's replies
(the counterpart of the reference's examples/python/vlm_multiturn_agent.py: ``environment_images`` returned by
``step`` are tokenised by the processor, appended to the conversation, and their patches join the sample's
``mm_train_inputs`` so that the trainer sees exactly what the rollout engine saw).

The toy task is self-contained: every turn the environment shows a picture with one bright quadrant and asks for
its number (0 = top-left, 1 = top-right, 2 = bottom-left, 3 = bottom-right). The reward of a turn is 1 for the right
digit; the episode ends after ``TURNS`` pictures.

    python -m openrlhf.cli.train_ppo_ray --train.agent_func_path examples/python/vlm_multiturn_agent.py \\
        --actor.model_name_or_path qwen2-vl-2b --data.image_key images --data.max_images_per_prompt 4 ...
"""
import random
import re

import torch
from PIL import Image, ImageDraw

from openrlhf.utils.agent import AgentInstanceBase, MultiTurnAgentExecutor

TURNS = 3
SIDE = 56


def quadrant_picture(which: int, side: int = SIDE) -> Image.Image:
    img = Image.new("RGB", (side, side), (20, 20, 20))
    half = side // 2
    x0, y0 = (which % 2) * half, (which // 2) * half
    ImageDraw.Draw(img).rectangle([x0, y0, x0 + half - 1, y0 + half - 1], fill=(240, 240, 240))
    return img


def first_digit(text: str):
    m = re.search(r"[0-3]", text)
    return int(m.group()) if m else None


class AgentInstance(AgentInstanceBase):
    def __init__(self, *args, **kwargs):
        self.rng = random.Random()
        self.turn = 0
        self.answer = 0
        self.right = 0

    async def reset(self, states: dict, **kwargs):
        # the dataset prompt (with its own image, if any) opens the episode; the first quadrant task follows in the
        # first environment reply
        self.turn, self.right = 0, 0
        self.answer = None
        return {"observation": states["observation"]}

    async def step(self, states: dict, **kwargs):
        guess = first_digit(states["action_text"])
        reward = 0.0
        if self.answer is not None:
            reward = 1.0 if guess == self.answer else 0.0
            self.right += int(reward)
        self.turn += 1
        done = self.turn > TURNS
        out = {"rewards": torch.tensor(reward), "scores": torch.tensor(self.right / TURNS), "done": done,
               "environment_feedback": "", "sampling_params": states.get("sampling_params"),
               "extra_logs": {"right_answers": torch.tensor(float(self.right))}}
        if not done:
            self.answer = self.rng.randrange(4)
            out["environment_feedback"] = " <image> which quadrant is bright ? "
            out["environment_images"] = [quadrant_picture(self.answer)]
        return out


class AgentExecutor(MultiTurnAgentExecutor):
    def __init__(self):
        super().__init__(AgentInstance)
