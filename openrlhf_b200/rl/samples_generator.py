"""Controller-side rollout driver: prompt batches -> per-prompt generate calls on the least-loaded rollout worker ->
Experiences, with oversampling buffer and DAPO-style dynamic filtering (replacement prompts for dropped groups).

Same behaviour as the reference's ``SamplesGenerator`` (openrlhf/trainer/ppo_utils/samples_generator.py:40-314), on
this framework's runtime futures instead of Ray object refs.
"""
from __future__ import annotations

import heapq
import logging

import torch

from ..rollout.engine import SamplingParams
from ..runtime.core import get, wait
from .experience import Experience

logger = logging.getLogger(__name__)


def collect_prompt_batch(dataloader_iter, num_prompts: int):
    """Pull prompts from the iterator until `num_prompts` are collected or it ends.
    Returns (prompts, labels, images, exhausted)."""
    prompts, labels, images = [], [], []
    exhausted = False
    while len(prompts) < num_prompts:
        try:
            _, p, l, im = next(dataloader_iter)
        except StopIteration:
            exhausted = True
            break
        prompts += list(p)
        labels += list(l)
        images += list(im)
    return prompts[:num_prompts], labels[:num_prompts], images[:num_prompts], exhausted


def response_to_experience(response: dict, max_len: int) -> Experience:
    """One executor result -> single-sample Experience (batch dim 1, CPU tensors); layout per the action-mask
    convention: T-1 columns, column i = predicting token i+1."""
    tokens = list(response["observation_tokens"])
    T = len(tokens)
    full_mask = torch.zeros(T, dtype=torch.long)
    for a, b in response["action_ranges"]:
        full_mask[a:b] = 1
    seq = torch.tensor(tokens[:max_len], dtype=torch.long)
    att = torch.ones(min(T, max_len), dtype=torch.long)
    am = full_mask[1:max_len]
    rlp = response.get("rollout_log_probs")
    rlp = torch.tensor(rlp[1:max_len], dtype=torch.float32).unsqueeze(0) if rlp is not None else None
    on = torch.where(am)[0]
    resp_len = int(on[-1] - on[0] + 1) if len(on) else 0
    total = float(att.sum())
    info = {"response_clip_ratio": torch.tensor([total >= max_len])}
    reward, score = response.get("reward"), response.get("scores")
    if reward is not None:
        info["reward"] = torch.tensor([reward])
    if score is not None:
        info["score"] = torch.tensor([score])
    for k, v in (response.get("extra_logs") or {}).items():
        info[k] = torch.tensor([v.flatten()[0].item() if isinstance(v, torch.Tensor) else v])
    return Experience(
        sequences=seq.unsqueeze(0), attention_mask=att.unsqueeze(0), action_mask=am.unsqueeze(0).bool(),
        rollout_log_probs=rlp, prompts=[response["prompt"]], labels=[response["label"]],
        images=[response.get("images")], mm_train_inputs=[response.get("mm_train_inputs")],
        rewards=torch.tensor([reward], dtype=torch.float32) if reward is not None else None,
        scores=torch.tensor([score], dtype=torch.float32) if score is not None else None,
        response_length=torch.tensor([resp_len]), truncated=torch.tensor([bool(response.get("truncated", False))]),
        total_length=torch.tensor([total]), info=info)


class SamplesGenerator:
    def __init__(self, engines: list, strategy, tokenizer, prompts_dataloader, eval_dataloader=None,
                 followers: list | None = None):
        self.engines = engines               # WorkerHandle objects that hold the rollout role (leaders under TP)
        # members of tensor-parallel rollout engines other than their leader: they mirror the leader for the length
        # of a generation phase (rollout/tp_engine.py::TPLockstepEngine)
        self.followers = list(followers or [])
        self.strategy, self.args = strategy, strategy.args
        self.tokenizer = tokenizer
        self.prompts_dataloader, self.eval_dataloader = prompts_dataloader, eval_dataloader
        self._dataloader_iter = None
        self._sample_buffer: list[Experience] = []

    # ------------------------------------------------------------------ engine helpers
    def _call_all(self, method: str, *a, **kw):
        if method in ("wake_up", "sleep"):       # memory management concerns every member of an engine
            return get([e.call(method, *a, **kw) for e in self.engines + self.followers])
        return get([e.call(method, *a, **kw) for e in self.engines])

    class _Phase:
        """Generation phase: followers enter their mirror loop, the leaders release them on exit."""

        def __init__(self, gen):
            self.gen = gen

        def __enter__(self):
            self.futs = [f.call("follow_generation") for f in self.gen.followers]
            return self

        def __exit__(self, *exc):
            if self.gen.followers:
                get([e.call("end_generation") for e in self.gen.engines])
                get(self.futs)
            return False

    def generation_phase(self):
        return SamplesGenerator._Phase(self)

    def _dispatch(self, prompts, labels, images=None, **gen):
        sp = SamplingParams(temperature=gen.get("temperature", 1.0), top_p=gen.get("top_p", 1.0),
                            top_k=gen.get("top_k", -1), max_tokens=gen.get("max_new_tokens"),
                            min_tokens=gen.get("min_new_tokens", 1),
                            skip_special_tokens=gen.get("skip_special_tokens", False),
                            logprobs=1 if self.args.algo.advantage.is_correction_enable else None,
                            ignore_eos=gen.get("ignore_eos", False))
        max_len = gen.get("max_len", 2048)
        n = gen.get("n_samples_per_prompt", self.args.rollout.n_samples_per_prompt)
        load = self._call_all("get_num_unfinished_requests")
        heap = [(c, i) for i, c in enumerate(load)]
        heapq.heapify(heap)
        images = images or [None] * len(prompts)
        futs = []
        for p, l, im in zip(prompts, labels, images):
            c, i = heapq.heappop(heap)
            heapq.heappush(heap, (c + n, i))
            futs.append(self.engines[i].call("generate_responses", prompt=p, label=l, sampling_params=sp,
                                             max_length=max_len, num_samples=n, images=im))
        return futs

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate_eval_samples(self, **gen) -> list[Experience]:
        if self.args.vllm.enable_sleep:
            self._call_all("wake_up")
        out = []
        with self.generation_phase():
            for _, prompts, labels, images in self.eval_dataloader:
                for res in get(self._dispatch(list(prompts), list(labels), list(images), **gen)):
                    out += [response_to_experience(r, gen.get("max_len", 2048)) for r in res]
        if self.args.vllm.enable_sleep:
            self._call_all("sleep")
        return out

    @torch.no_grad()
    def generate_samples(self, **gen):
        """One training-sized batch: (experiences, filter pass rate or None, prompts consumed, exhausted)."""
        a = self.args
        if self._dataloader_iter is None and not getattr(self, "_started", False):
            self._dataloader_iter = iter(self.prompts_dataloader)
            self._started = True
        chunk = a.rollout.batch_size * a.rollout.n_samples_per_prompt
        consumed, pass_rate = 0, None
        if len(self._sample_buffer) < chunk and self._dataloader_iter is not None:
            if a.vllm.enable_sleep:
                self._call_all("wake_up")
            n_prompts = getattr(a.rollout, "vllm_generate_batch_size", None) or a.rollout.batch_size
            with self.generation_phase():
                exps, consumed, done = self._generate(self._dataloader_iter, n_prompts,
                                                      a.algo.dynamic_filtering_enable, **gen)
            if a.vllm.enable_sleep:
                self._call_all("sleep")
            if a.algo.dynamic_filtering_enable and consumed:
                pass_rate = len(exps) / a.rollout.n_samples_per_prompt / consumed * 100
            self._sample_buffer += exps
            if done:
                self._dataloader_iter = None
                logger.info("Prompt dataloader is exhausted.")
        out, self._sample_buffer = self._sample_buffer[:chunk], self._sample_buffer[chunk:]
        return out, pass_rate, consumed, (self._dataloader_iter is None and not self._sample_buffer)

    def restart_epoch(self):
        self._dataloader_iter = iter(self.prompts_dataloader)
        self._started = True

    def _generate(self, it, num_prompts: int, dynamic_filtering: bool, **gen):
        prompts, labels, images, exhausted = collect_prompt_batch(it, num_prompts)
        if not prompts:
            return [], 0, True
        consumed = len(prompts)
        pending = self._dispatch(prompts, labels, images, **gen)
        accepted: list[Experience] = []
        max_len = gen.get("max_len", 2048)
        while pending:
            ready, pending = wait(pending, num_returns=1, timeout=10.0)
            for f in ready:
                group = [response_to_experience(r, max_len) for r in f.result()]
                if dynamic_filtering and all(e.scores is not None for e in group):
                    mean = sum(float(e.scores[0]) for e in group) / len(group)
                    lo, hi = self.args.algo.dynamic_filtering_range
                    if not (lo < mean < hi):
                        logger.info("filtered out a prompt group: mean score %.3f outside (%.2f, %.2f)", mean, lo, hi)
                        group = []
                if group:
                    accepted += group
                elif dynamic_filtering:
                    np_, nl, ni, exhausted = collect_prompt_batch(it, 1)
                    consumed += len(np_)
                    if exhausted and not np_:
                        for p in pending:
                            p.cancel()
                        return [], consumed, True
                    if np_:
                        pending += self._dispatch(np_, nl, ni, **gen)
        return accepted, consumed, exhausted
