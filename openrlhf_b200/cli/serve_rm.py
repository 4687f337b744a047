"""``python -m openrlhf.cli.serve_rm``: HTTP reward-model server. ``POST /get_reward {"query": [...], "prompts": [...],
"labels": [...]}`` -> ``{"rewards", "scores", "extra_logs"}`` (the contract of openrlhf/cli/serve_rm.py:16-137 and of the
remote-reward client in ``utils/agent.py``)."""
from __future__ import annotations

import argparse

import torch
from fastapi import FastAPI, Request          # module level: the route's `request: Request` annotation is resolved
from fastapi.responses import JSONResponse    # against the module globals

from ..models.model import get_llm_for_sequence_regression
from ..utils.utils import get_tokenizer
from . import flags as F


class RewardModelProxy:
    def __init__(self, args):
        device = "cuda" if torch.cuda.is_available() else "cpu"
        self.reward_model = get_llm_for_sequence_regression(
            args.reward.model_name_or_path, "reward", normalize_reward=args.reward.normalize_enable,
            value_head_prefix=args.ds.value_head_prefix, device=device, packing_samples=args.ds.packing_samples,
            load_in_4bit=args.ds.load_in_4bit)
        self.reward_model.eval()
        self.device = device
        self.tokenizer = get_tokenizer(args.reward.model_name_or_path, self.reward_model, "left", None,
                                       use_fast=not args.data.disable_fast_tokenizer)
        self.max_length, self.batch_size = args.data.max_len, args.batch_size

    def tokenize_fn(self, texts, device):
        batch = self.tokenizer(texts, return_tensors="pt", add_special_tokens=False, max_length=self.max_length,
                               padding=True, truncation=True)
        return {k: v.to(device) for k, v in batch.items()}

    @torch.no_grad()
    def get_reward(self, queries: list[str]) -> list[float]:
        bs = self.batch_size or len(queries)
        scores: list[float] = []
        for i in range(0, len(queries), bs):
            inp = self.tokenize_fn(queries[i:i + bs], self.device)
            scores += self.reward_model(inp["input_ids"], inp["attention_mask"]).float().tolist()
        return scores


def build_app(proxy: RewardModelProxy):
    app = FastAPI()

    @app.post("/get_reward")
    async def get_reward(request: Request):
        data = await request.json()
        rewards = proxy.get_reward(data.get("query"))
        return JSONResponse({"rewards": rewards, "scores": rewards, "extra_logs": {"dummy_scores": rewards}})

    return app


def build_parser():
    p = argparse.ArgumentParser()
    F.add_flags(p, [("--reward.model_name_or_path", str, None), ("--reward.normalize_enable", F.BOOL, False),
                    ("--ds.value_head_prefix", str, "score"), ("--data.max_len", int, 2048), ("--port", int, 5000),
                    ("--host", str, "0.0.0.0"), ("--ds.load_in_4bit", F.BOOL, False),
                    ("--ds.param_dtype", str, "bf16", {"choices": ["bf16", "fp16"]}),
                    ("--ds.attn_implementation", str, "flash_attention_2"), ("--ds.experts_implementation", str, None),
                    ("--data.disable_fast_tokenizer", F.BOOL, False), ("--ds.packing_samples", F.BOOL, False),
                    ("--batch_size", int, None), ("--use_ms", F.BOOL, False)])
    return p


if __name__ == "__main__":
    import uvicorn

    args = F.finalize(build_parser())
    uvicorn.run(build_app(RewardModelProxy(args)), host=args.host, port=args.port, log_level="info")
