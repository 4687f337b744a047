"""Asyncio front of the rollout engine: ``await engine.generate(token_ids, sampling_params)`` from many coroutines
at once; a single driver task turns the outstanding requests into continuous batches.

This is the handle the agent executors receive as ``llm_engine`` (the reference hands them a vLLM
``AsyncLLMEngine`` wrapper: openrlhf/trainer/ray/vllm_engine.py:155-179)."""
from __future__ import annotations

import asyncio
import itertools

from .engine import RolloutEngine, SamplingParams


class AsyncRolloutEngine:
    def __init__(self, engine: RolloutEngine, tokenizer=None):
        self.engine = engine
        self.tokenizer = tokenizer
        self._ids = itertools.count()
        self._futures: dict = {}
        self._driver: asyncio.Task | None = None
        self._lock = asyncio.Lock()

    async def generate(self, prompt_token_ids, sampling_params: SamplingParams, multi_modal_data=None):
        loop = asyncio.get_running_loop()
        rid = ("async", next(self._ids))
        fut = loop.create_future()
        self._futures[rid] = fut
        self.engine.add_request(rid, prompt_token_ids, sampling_params, multi_modal_data)
        if self._driver is None or self._driver.done():
            self._driver = loop.create_task(self._drive())
        out = await fut
        if self.tokenizer is not None:
            for c in out.outputs:
                c.text = self.tokenizer.decode(c.token_ids, skip_special_tokens=sampling_params.skip_special_tokens)
        return out

    async def _drive(self):
        while self.engine.has_unfinished():
            if self.engine.paused:
                await asyncio.sleep(0.01)
                continue
            await asyncio.sleep(0)              # let newly arrived requests join before the next burst
            try:
                done = self.engine.step()
            except Exception as e:  # noqa: BLE001
                for f in self._futures.values():
                    if not f.done():
                        f.set_exception(e)
                self._futures.clear()
                raise
            for ro in done:
                f = self._futures.pop(ro.request_id, None)
                if f is not None and not f.done():
                    f.set_result(ro)

    def get_num_unfinished_requests(self) -> int:
        return len(self._futures)
