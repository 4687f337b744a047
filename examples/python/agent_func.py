"""Example multi-turn agent: the environment asks for one more number until three turns have passed.
Defines ``AgentExecutor`` as required by ``--train.agent_func_path``."""
import torch

from openrlhf.utils.agent import AgentInstanceBase, MultiTurnAgentExecutor


class AgentInstance(AgentInstanceBase):
    def __init__(self, *args, **kwargs):
        self.turn = 0

    async def reset(self, states, **kwargs):
        self.turn = 0
        return {"observation": states["observation"]}

    async def step(self, states, **kwargs):
        self.turn += 1
        toks = [int(t) for t in states["action_text"].split() if t.isdigit()]
        reward = torch.tensor(sum(t % 2 == 0 for t in toks) / max(len(toks), 1))
        done = self.turn >= 3
        return {"rewards": reward, "scores": reward, "environment_feedback": "" if done else " 7 7 ", "done": done,
                "sampling_params": states.get("sampling_params"), "extra_logs": {"turns": torch.tensor(float(self.turn))}}


class AgentExecutor(MultiTurnAgentExecutor):
    def __init__(self):
        super().__init__(AgentInstance)
