"""Token-in / token-out agent API executed next to the rollout engine.

Keeps the user-facing contract of the reference (openrlhf/utils/agent.py:12-356): an executor's ``execute`` coroutine
receives a prompt, label, sampling parameters, a length budget, the tokenizer and an engine handle whose
``generate(token_ids, sampling_params)`` coroutine returns an object with ``.outputs[0].token_ids / .text /
.logprobs / .finish_reason``, and returns a dict with the keys listed in ``RESULT_KEYS``.
User files passed as ``--train.agent_func_path`` define ``class AgentExecutor(AgentExecutorBase)``; reward files
define ``reward_func(queries, prompts, labels, **kw)``.
"""
from __future__ import annotations

import asyncio
import copy
import importlib.util
import logging
from abc import ABC, abstractmethod

logger = logging.getLogger(__name__)

RESULT_KEYS = ("prompt", "label", "images", "mm_train_inputs", "observation_tokens", "action_ranges",
               "rollout_log_probs", "truncated", "reward", "scores", "extra_logs")


class AgentExecutorBase(ABC):
    @abstractmethod
    async def execute(self, prompt, label, sampling_params, max_length: int, hf_tokenizer, llm_engine, images=None):
        raise NotImplementedError


class AgentInstanceBase(ABC):
    """One environment instance per prompt: ``reset(states) -> {"observation": str}`` and
    ``step(states) -> {"rewards", "scores", "environment_feedback", "done", ["sampling_params", "extra_logs",
    "environment_images"]}``."""

    def __init__(self, *args, **kwargs):
        pass

    async def reset(self, states: dict, **kwargs):
        return {"observation": states["observation"]}

    @abstractmethod
    async def step(self, states: dict, **kwargs):
        raise NotImplementedError


def _encode(tokenizer, text: str) -> list[int]:
    ids = tokenizer(text=text, add_special_tokens=False)["input_ids"]
    if ids and isinstance(ids[0], (list, tuple)):
        ids = ids[0]
    return list(ids.tolist() if hasattr(ids, "tolist") else ids)


def _token_logprobs(token_ids, logprobs) -> list[float]:
    """Accepts either a list of floats or vLLM-style [{token_id: obj-with-.logprob}] entries."""
    out = []
    for tok, lp in zip(token_ids, logprobs):
        if isinstance(lp, dict):
            item = lp.get(tok)
            out.append(float(getattr(item, "logprob", item)) if item is not None else 0.0)
        else:
            out.append(float(lp))
    return out


def _to_float(x) -> float:
    return float(x.item()) if hasattr(x, "item") else float(x)


def load_python_object(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return getattr(mod, name)


class MultiTurnAgentExecutor(AgentExecutorBase):
    """Environment loop: observe -> generate within the remaining token budget -> env.step -> append feedback."""

    def __init__(self, agent_instance_cls):
        if not issubclass(agent_instance_cls, AgentInstanceBase):
            raise AssertionError("AgentInstance must inherit from AgentInstanceBase")
        self.agent_instance_cls = agent_instance_cls

    async def execute(self, prompt, label, sampling_params, max_length: int, hf_tokenizer, llm_engine, images=None):
        env = self.agent_instance_cls()
        obs_text = (await env.reset({"observation": prompt, "label": label}))["observation"]
        mm_train_inputs, pil_images = None, []
        if images and hasattr(hf_tokenizer, "image_processor"):
            from .vlm_utils import process_prompt_with_images

            tokens, mm_train_inputs, pil_images = process_prompt_with_images(hf_tokenizer, obs_text, images)
        else:
            tokens = _encode(hf_tokenizer, obs_text)
        room = max_length - (getattr(sampling_params, "max_tokens", None) or 1)
        if len(tokens) > room:
            if pil_images:
                raise ValueError(f"VLM prompt of {len(tokens)} tokens exceeds the budget of {room}; truncation would "
                                 "break the image-token alignment. Raise --data.max_len or lower --rollout.max_new_tokens.")
            logger.warning("initial observation of %d tokens truncated to %d", len(tokens), room)
            tokens = tokens[-room:]
            obs_text = hf_tokenizer.decode(tokens, skip_special_tokens=False)
        want_lp = sampling_params.logprobs is not None
        logps = [0.0] * len(tokens) if want_lp else None
        ranges, total_reward, scores, extra = [], 0.0, 0.0, {}
        sp = sampling_params
        while True:
            sp.max_tokens = max_length - len(tokens)
            if sp.max_tokens <= 0:
                break
            res = await llm_engine.generate(tokens, copy.deepcopy(sp),
                                            multi_modal_data={"image": pil_images} if pil_images else None)
            gen = res.outputs[0]
            action, action_text = list(gen.token_ids), gen.text
            ranges.append((len(tokens), len(tokens) + len(action)))
            step = await env.step({"observation_text": obs_text, "action_text": action_text, "label": label,
                                   "sampling_params": sp})
            total_reward += _to_float(step["rewards"])
            scores = step.get("scores", total_reward)
            extra = step.get("extra_logs", {})
            fb_text = step["environment_feedback"]
            env_images = step.get("environment_images")
            if env_images and hasattr(hf_tokenizer, "image_processor"):
                from .vlm_utils import accumulate_mm_inputs, process_prompt_with_images

                fb, new_mm, new_pil = process_prompt_with_images(hf_tokenizer, fb_text, env_images)
                if len(tokens) + len(action) + len(fb) <= max_length or new_mm is None:
                    pil_images.extend(new_pil)
                    mm_train_inputs = accumulate_mm_inputs(mm_train_inputs, new_mm)
                else:
                    drop = {getattr(hf_tokenizer, a, None) for a in ("image_token_id", "video_token_id")} - {None}
                    fb = [t for t in fb if t not in drop]
            else:
                fb = _encode(hf_tokenizer, fb_text)
            obs_text = obs_text + action_text + fb_text
            tokens = tokens + action + fb
            if want_lp:
                logps += _token_logprobs(action, gen.logprobs) + [0.0] * len(fb)
            if step.get("sampling_params"):
                sp = step["sampling_params"]
            if step["done"]:
                break
        return {"prompt": prompt, "label": label, "images": images, "mm_train_inputs": mm_train_inputs,
                "reward": total_reward, "scores": scores, "observation_tokens": tokens, "action_ranges": ranges,
                "rollout_log_probs": logps, "extra_logs": extra}


class SingleTurnAgentExecutor(AgentExecutorBase):
    """One generation per prompt, optionally scored by a ``reward_func.py`` file or HTTP reward servers."""

    HTTP_RETRIES = 5
    HTTP_TIMEOUT_S = 180

    def __init__(self, remote_rm_url=None):
        urls = [remote_rm_url] if isinstance(remote_rm_url, str) else (remote_rm_url or [])
        self.reward_endpoints = list(urls)
        self.reward_func = None
        if self.reward_endpoints and self.reward_endpoints[0].endswith(".py"):
            logger.info("loading reward_func(queries, prompts, labels) from %s", self.reward_endpoints[0])
            self.reward_func = load_python_object(self.reward_endpoints[0], "reward_func")

    async def execute(self, prompt, label, sampling_params, max_length: int, hf_tokenizer, llm_engine, images=None):
        mm_train_inputs, pil_images = None, []
        if images and hasattr(hf_tokenizer, "image_processor"):
            from .vlm_utils import process_prompt_with_images

            prompt_ids, mm_train_inputs, pil_images = process_prompt_with_images(hf_tokenizer, prompt, images)
        else:
            prompt_ids = _encode(hf_tokenizer, prompt)
        sp = sampling_params
        if sp.max_tokens is None:
            sp = copy.deepcopy(sp)
            sp.max_tokens = max(1, max_length - len(prompt_ids))
        room = max_length - sp.max_tokens
        if len(prompt_ids) > room:
            if pil_images:
                raise ValueError(f"VLM prompt of {len(prompt_ids)} tokens exceeds the budget of {room}; truncation "
                                 "would break the image-token alignment.")
            logger.warning("prompt of %d tokens truncated from the left to %d", len(prompt_ids), room)
            prompt_ids = prompt_ids[-room:] if room > 0 else []
        res = await llm_engine.generate(prompt_ids, copy.deepcopy(sp),
                                        multi_modal_data={"image": pil_images} if pil_images else None)
        gen = res.outputs[0]
        action = list(gen.token_ids)
        tokens = prompt_ids + action
        logps = None
        if sampling_params.logprobs is not None and gen.logprobs is not None:
            logps = [0.0] * len(prompt_ids) + _token_logprobs(action, gen.logprobs)
        out = {"prompt": prompt, "label": label, "images": images, "mm_train_inputs": mm_train_inputs,
               "observation_tokens": tokens, "action_ranges": [(len(prompt_ids), len(tokens))],
               "rollout_log_probs": logps, "truncated": gen.finish_reason == "length", "reward": None,
               "scores": None, "extra_logs": {}}
        if self.reward_endpoints:
            try:
                query = hf_tokenizer.decode(tokens, skip_special_tokens=False)
                fetch = self._fetch_rewards_via_func if self.reward_func else self._fetch_rewards_via_http
                infos = await fetch([query], [prompt], [label])
                info = infos[0] if infos else None
                if info:
                    sc = info.get("scores")
                    out.update(reward=info.get("rewards"), scores=sc if sc is not None else info.get("rewards"),
                               extra_logs=info.get("extra_logs") or {})
            except Exception as e:  # noqa: BLE001
                logger.error("reward fetch failed for one sample: %s", e)
                out["extra_logs"] = {"reward_error": 1.0}
        return out

    async def _fetch_rewards_via_func(self, queries, prompts, labels):
        jobs = [asyncio.to_thread(self.reward_func, queries[i:i + 1], prompts[i:i + 1], labels[i:i + 1])
                for i in range(len(queries))]
        return await asyncio.gather(*jobs)

    async def _fetch_rewards_via_http(self, queries, prompts, labels):
        import aiohttp

        n = len(self.reward_endpoints)
        per = (len(queries) + n - 1) // n
        timeout = aiohttp.ClientTimeout(total=self.HTTP_TIMEOUT_S)

        async def post(url, payload):
            for _ in range(self.HTTP_RETRIES):
                try:
                    async with aiohttp.ClientSession(timeout=timeout) as s:
                        async with s.post(url, json=payload) as r:
                            r.raise_for_status()
                            return await r.json()
                except Exception as e:  # noqa: BLE001
                    logger.info("reward request to %s failed: %s", url, e)
                await asyncio.sleep(1)
            raise RuntimeError(f"reward server {url} did not answer after {self.HTTP_RETRIES} attempts")

        jobs = []
        for i, url in enumerate(self.reward_endpoints):
            sl = slice(i * per, min((i + 1) * per, len(queries)))
            jobs.append(asyncio.create_task(post(url, {"query": queries[sl], "prompts": prompts[sl], "labels": labels[sl]})))
        return await asyncio.gather(*jobs)
