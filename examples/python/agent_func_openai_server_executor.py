"""Agent executor that exposes the rollout engine as a local OpenAI-compatible chat endpoint.

An agent written against ``POST /v1/chat/completions`` (any HTTP client, any framework) can be trained without
changes: every call that carries the same ``session_id`` extends one token-level trace, and when ``run_agent``
returns the trace is folded into one RL sample (observation tokens, the ranges the policy generated, their rollout
log-probabilities). Same contract as the reference example
(examples/python/agent_func_openai_server_executor.py:52-298); the pieces are split differently here:

* ``SessionTraces`` is pure bookkeeping (delta tokenisation against the session's token buffer, prefix checks,
  stitching) and is testable without a server;
* ``build_app`` is the thin FastAPI layer around it;
* ``AgentExecutor.run_agent`` is the method to override for multi-turn workflows.

Delta tokenisation: turn k's prompt is rendered with the chat template and must start with the tokens the session has
already seen (prompt + completion of turn k-1); only the tail is new. The engine therefore sees exactly the tokens
the trainer will later see.

    python -m openrlhf.cli.train_ppo_ray --train.agent_func_path examples/python/agent_func_openai_server_executor.py ...
"""

import asyncio
import copy
import json
import socket
import threading
import time
import urllib.request
from uuid import uuid4

from openrlhf.utils.agent import AgentExecutorBase


def render_chat(tokenizer, messages) -> list[int]:
    """Token ids of the conversation with the generation prompt appended."""
    if getattr(tokenizer, "chat_template", None) or hasattr(tokenizer, "apply_chat_template"):
        try:
            text = tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)
        except Exception:  # noqa: BLE001  tokenizers without a template
            text = "".join(f"{m['role']}: {m['content']}\n" for m in messages) + "assistant: "
    else:
        text = "".join(f"{m['role']}: {m['content']}\n" for m in messages) + "assistant: "
    ids = tokenizer(text=text, add_special_tokens=False)["input_ids"]
    return list(ids[0] if ids and isinstance(ids[0], (list, tuple)) else ids)


class SessionTraces:
    """Per-session token buffers and call records."""

    def __init__(self):
        self.buffers: dict[str, list[int]] = {}
        self.calls: dict[str, list[dict]] = {}

    def prompt_for(self, session_id: str, full_prompt_ids: list[int]) -> list[int]:
        seen = self.buffers.get(session_id)
        if seen is None:
            ids = list(full_prompt_ids)
        else:
            if len(full_prompt_ids) < len(seen) or full_prompt_ids[:len(seen)] != seen:
                raise ValueError(f"session {session_id}: the new prompt does not extend the {len(seen)} tokens "
                                 "already in the session (chat template or tokenizer is not prefix-stable)")
            ids = seen + list(full_prompt_ids[len(seen):])
        self.buffers[session_id] = list(ids)
        return ids

    def record(self, session_id: str, prompt_ids, completion_ids, logprobs, finish_reason):
        self.calls.setdefault(session_id, []).append({
            "prompt": list(prompt_ids), "completion": list(completion_ids),
            "logprobs": None if logprobs is None else [float(x) for x in logprobs], "finish": finish_reason})
        self.buffers[session_id] = list(prompt_ids) + list(completion_ids)

    def drop(self, session_id: str):
        self.buffers.pop(session_id, None)
        self.calls.pop(session_id, None)

    def stitch(self, session_id: str, want_logprobs: bool) -> dict:
        calls = self.calls.get(session_id) or []
        if not calls:
            raise RuntimeError(f"session {session_id} made no completion call")
        for a, b in zip(calls, calls[1:]):
            whole = a["prompt"] + a["completion"]
            if b["prompt"][:len(whole)] != whole:
                raise ValueError(f"session {session_id}: a later call dropped tokens of an earlier one")
        tokens = calls[-1]["prompt"] + calls[-1]["completion"]
        ranges = [(len(c["prompt"]), len(c["prompt"]) + len(c["completion"])) for c in calls]
        logps = None
        if want_logprobs:
            logps = [0.0] * len(tokens)
            for c, (lo, hi) in zip(calls, ranges):
                if c["logprobs"] is not None:
                    logps[lo:hi] = c["logprobs"][:hi - lo] + [0.0] * max(0, hi - lo - len(c["logprobs"]))
        return {"observation_tokens": tokens, "action_ranges": ranges, "rollout_log_probs": logps,
                "truncated": calls[-1]["finish"] == "length"}


def _chosen_logprobs(token_ids, logprobs):
    if logprobs is None:
        return None
    out = []
    for tok, lp in zip(token_ids, logprobs):
        if isinstance(lp, dict):
            item = lp.get(tok)
            out.append(float(getattr(item, "logprob", item)) if item is not None else 0.0)
        else:
            out.append(float(lp))
    return out


async def complete(executor, body: dict) -> dict:
    """One chat-completions call against the engine; shared by the HTTP route and by in-process callers."""
    messages = body.get("messages") or []
    if not messages:
        raise ValueError("no messages")
    session_id = body.get("session_id") or uuid4().hex
    base = executor.sampling_params
    prompt_ids = executor.traces.prompt_for(session_id, render_chat(executor.tokenizer, messages))
    room = executor.max_length - len(prompt_ids)
    if room <= 0:
        raise ValueError(f"prompt of {len(prompt_ids)} tokens leaves no room under max_length {executor.max_length}")
    sp = copy.deepcopy(base)
    sp.max_tokens = min(int(body.get("max_tokens") or base.max_tokens or room), room)
    for key in ("temperature", "top_p"):
        if body.get(key) is not None:
            setattr(sp, key, body[key])
    res = await executor.engine.generate(prompt_ids, sp)
    out = res.outputs[0]
    lps = _chosen_logprobs(out.token_ids, getattr(out, "logprobs", None))
    executor.traces.record(session_id, prompt_ids, out.token_ids, lps, out.finish_reason)
    choice = {"index": 0, "finish_reason": out.finish_reason, "message": {"role": "assistant", "content": out.text}}
    if body.get("logprobs") and lps is not None:
        choice["logprobs"] = {"content": [{"token": str(t), "logprob": l} for t, l in zip(out.token_ids, lps)]}
    return {"id": "chatcmpl-" + uuid4().hex, "object": "chat.completion", "created": int(time.time()),
            "model": executor.model_name, "session_id": session_id, "choices": [choice],
            "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": len(out.token_ids),
                      "total_tokens": len(prompt_ids) + len(out.token_ids)}}


def build_app(executor):
    from fastapi import FastAPI, HTTPException, Request

    app = FastAPI()

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": executor.model_name, "object": "model"}]}

    @app.post("/tokenize")
    async def tokenize(request: Request):
        body = await request.json()
        ids = executor.tokenizer(text=body.get("prompt", ""), add_special_tokens=False)["input_ids"]
        return {"tokens": list(ids), "count": len(ids)}

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        try:
            return await complete(executor, await request.json())
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))

    return app


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class AgentExecutor(AgentExecutorBase):
    model_name = "policy"

    def __init__(self, serve_http: bool = True):
        self.serve_http = serve_http
        self.traces = SessionTraces()
        self.engine = self.tokenizer = self.sampling_params = None
        self.max_length = 0
        self.base_url = None
        self._loop = None

    # ---- server ----
    def _ensure_server(self):
        if self.base_url is not None or not self.serve_http:
            return
        import uvicorn

        port = _free_port()
        config = uvicorn.Config(build_app(self), host="127.0.0.1", port=port, log_level="warning")
        server = uvicorn.Server(config)
        threading.Thread(target=server.run, daemon=True).start()
        self.base_url = f"http://127.0.0.1:{port}"
        deadline = time.time() + 30
        while time.time() < deadline:
            try:
                with urllib.request.urlopen(self.base_url + "/health", timeout=1) as r:
                    if r.status == 200:
                        return
            except OSError:
                time.sleep(0.1)
        raise RuntimeError("the local chat endpoint did not come up")

    async def chat(self, messages, session_id: str, **kw) -> dict:
        """What an external agent would do over HTTP; in-process when ``serve_http`` is off."""
        body = {"messages": messages, "session_id": session_id, **kw}
        if not self.serve_http:
            return await complete(self, body)

        def post():
            req = urllib.request.Request(self.base_url + "/v1/chat/completions", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=3600) as r:
                return json.loads(r.read())

        return await asyncio.get_running_loop().run_in_executor(None, post)

    # ---- the method to override ----
    async def run_agent(self, prompt: str, label: str, session_id: str) -> dict:
        """Single-turn default. A multi-turn agent calls ``self.chat`` (or the HTTP endpoint) several times with the
        same session id and returns {"reward", "scores", "extra_logs"}."""
        await self.chat([{"role": "user", "content": prompt}], session_id, logprobs=True)
        return {}

    async def execute(self, prompt, label, sampling_params, max_length, hf_tokenizer, llm_engine, images=None):
        self.engine, self.tokenizer = llm_engine, hf_tokenizer
        self.sampling_params, self.max_length = sampling_params, max_length
        self._ensure_server()
        session_id = uuid4().hex
        try:
            verdict = await self.run_agent(prompt, label, session_id) or {}
            sample = self.traces.stitch(session_id, sampling_params.logprobs is not None)
        finally:
            self.traces.drop(session_id)
        sample.update({"prompt": prompt, "label": label, "reward": verdict.get("reward"),
                       "scores": verdict.get("scores"), "extra_logs": verdict.get("extra_logs", {})})
        return sample
