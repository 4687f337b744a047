"""Agent API: the multi-turn executor and the example agent files against a scripted engine."""
import asyncio
import os
import re
from types import SimpleNamespace

import pytest

from openrlhf_b200.utils.agent import load_python_object

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples", "python")


class CharTokenizer:
    """One token per character; no chat template."""

    def __call__(self, text=None, add_special_tokens=False, **kw):
        return {"input_ids": [ord(c) for c in text]}

    def decode(self, ids, skip_special_tokens=False):
        return "".join(chr(i) for i in ids)


class ScriptedEngine:
    """Replies with the next scripted text; records the prompts it was given."""

    def __init__(self, replies):
        self.replies = list(replies)
        self.prompts = []

    async def generate(self, token_ids, sampling_params, multi_modal_data=None):
        self.prompts.append(list(token_ids))
        text = self.replies.pop(0)[: sampling_params.max_tokens]
        ids = [ord(c) for c in text]
        out = SimpleNamespace(token_ids=ids, text=text, logprobs=[-0.5] * len(ids),
                              finish_reason="stop" if self.replies else "length")
        return SimpleNamespace(outputs=[out])


def _sp(max_tokens=64, logprobs=1):
    return SimpleNamespace(max_tokens=max_tokens, temperature=1.0, top_p=1.0, logprobs=logprobs)


def _check_sample(res, tok_prompt_len):
    toks, ranges = res["observation_tokens"], res["action_ranges"]
    assert ranges and ranges[0][0] == tok_prompt_len
    for (a, b), (c, d) in zip(ranges, ranges[1:]):
        assert a < b <= c < d
    assert ranges[-1][1] <= len(toks)
    if res["rollout_log_probs"] is not None:
        lp = res["rollout_log_probs"]
        assert len(lp) == len(toks)
        inside = set(i for a, b in ranges for i in range(a, b))
        assert all((lp[i] == -0.5) == (i in inside) for i in range(len(toks)))


def test_multiturn_example_agent():
    ex = load_python_object(os.path.join(EX, "agent_func.py"), "AgentExecutor")()
    eng = ScriptedEngine(["2 4 5 ", "6 ", "1 "])
    res = asyncio.run(ex.execute("count: ", None, _sp(), 256, CharTokenizer(), eng))
    assert len(res["action_ranges"]) == 3 and len(eng.prompts) == 3
    _check_sample(res, len("count: "))
    # each later prompt is the earlier prompt + action + feedback
    assert eng.prompts[1][:len(eng.prompts[0])] == eng.prompts[0]
    assert res["reward"] == pytest.approx(2 / 3 + 1.0 + 0.0)


def test_gem_style_example_agent_wins_and_stops():
    mod_cls = load_python_object(os.path.join(EX, "agent_func_gem_multiturn.py"), "AgentExecutor")
    ex = mod_cls()
    inst_cls = ex.agent_instance_cls

    class Fixed(inst_cls):
        def __init__(self):
            super().__init__()
            if hasattr(self.env, "rng"):
                self.env.rng.seed(3)

    ex.agent_instance_cls = Fixed
    probe = Fixed()
    probe.env.reset()
    target = getattr(probe.env, "target", None)
    if target is None:
        pytest.skip("external gem environment in use")
    wrong = target + 1 if target < 20 else target - 1
    eng = ScriptedEngine([f"maybe \\boxed{{{wrong}}}", "no box here", f"so \\boxed{{{target}}}", "unused"])
    res = asyncio.run(ex.execute("ignored", None, _sp(), 4096, CharTokenizer(), eng))
    assert len(res["action_ranges"]) == 3          # stopped at the correct guess
    assert res["reward"] == pytest.approx(0.0 - 0.1 + 1.0)
    text = CharTokenizer().decode(res["observation_tokens"])
    assert re.search(r"(higher|lower) than", text) and "no \\boxed" in text
    _check_sample(res, len(eng.prompts[0]))


def test_openai_shim_stitches_sessions_in_process():
    mod_cls = load_python_object(os.path.join(EX, "agent_func_openai_server_executor.py"), "AgentExecutor")

    class TwoTurns(mod_cls):
        async def run_agent(self, prompt, label, session_id):
            msgs = [{"role": "user", "content": prompt}]
            r1 = await self.chat(msgs, session_id, logprobs=True)
            a1 = r1["choices"][0]["message"]["content"]
            msgs += [{"role": "assistant", "content": a1}, {"role": "user", "content": "again"}]
            r2 = await self.chat(msgs, session_id, max_tokens=3)
            assert r2["usage"]["completion_tokens"] <= 3
            return {"reward": 1.0, "scores": 1.0, "extra_logs": {"calls": 2}}

    class Tok(CharTokenizer):
        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
            s = "".join(f"<{m['role'][0]}>{m['content']}\n" for m in messages)
            return s + ("<a>" if add_generation_prompt else "")

    # an assistant turn renders as "<a>text\n", i.e. the generation prompt + the completion: prefix-stable
    ex = TwoTurns(serve_http=False)
    eng = ScriptedEngine(["hello", "world!"])
    res = asyncio.run(ex.execute("hi", "lab", _sp(), 512, Tok(), eng))
    assert res["reward"] == 1.0 and res["label"] == "lab"
    (a, b), (c, d) = res["action_ranges"]
    text = CharTokenizer().decode(res["observation_tokens"])
    assert text[a:b] == "hello" and text[c:d] == "wor" and res["truncated"]
    assert text == "<u>hi\n<a>hello\n<u>again\n<a>wor"
    _check_sample(res, len("<u>hi\n<a>"))
    assert not ex.traces.buffers and not ex.traces.calls       # session state dropped

    # a prompt that does not extend the session is refused
    tr = ex.traces
    tr.prompt_for("s", [1, 2, 3])
    with pytest.raises(ValueError):
        tr.prompt_for("s", [1, 9, 3, 4])


def test_openai_shim_over_http():
    pytest.importorskip("fastapi")
    pytest.importorskip("uvicorn")
    mod_cls = load_python_object(os.path.join(EX, "agent_func_openai_server_executor.py"), "AgentExecutor")
    ex = mod_cls(serve_http=True)
    eng = ScriptedEngine(["pong"])
    try:
        res = asyncio.run(ex.execute("ping", None, _sp(), 128, CharTokenizer(), eng))
    except (RuntimeError, OSError) as e:       # no loopback sockets in this sandbox
        pytest.skip(f"local HTTP endpoint unavailable: {e}")
    text = CharTokenizer().decode(res["observation_tokens"])
    assert text.endswith("pong") and len(res["action_ranges"]) == 1


@pytest.mark.parametrize("fname", ["agent_func.py", "agent_func_gem_multiturn.py", "agent_func_openai_server_executor.py"])
def test_example_executors_pass_the_worker_type_check(fname):
    """User files import the base classes through the ``openrlhf`` alias package; the workers check them against
    ``openrlhf_b200.utils.agent``: both must be the same class objects."""
    from openrlhf_b200.utils.agent import AgentExecutorBase

    cls = load_python_object(os.path.join(EX, fname), "AgentExecutor")
    assert issubclass(cls, AgentExecutorBase)


def test_vlm_multiturn_agent_accumulates_images():
    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.vision import image_runs
    from openrlhf_b200.utils.utils import get_tokenizer
    from openrlhf_b200.datasets.utils import synthetic_dataset

    proc = get_tokenizer("tiny-qwen2-vl")
    cfg = PRESETS["tiny-qwen2-vl"]
    row = synthetic_dataset("synthetic://vlm_prompts?n=1&len=5&vocab=2000&image=56")[0]
    ex = load_python_object(os.path.join(EX, "vlm_multiturn_agent.py"), "AgentExecutor")()

    class Eng:
        calls = []

        async def generate(self, token_ids, sampling_params, multi_modal_data=None):
            self.calls.append((len(token_ids), len(multi_modal_data["image"]) if multi_modal_data else 0))
            ids = [1, 2]
            out = SimpleNamespace(token_ids=ids, text="1 2", logprobs=[-0.1, -0.2], finish_reason="stop")
            return SimpleNamespace(outputs=[out])

    eng = Eng()
    res = asyncio.run(ex.execute(row["input"], row["label"], _sp(max_tokens=8), 512, proc, eng, images=row["images"]))
    assert [c[1] for c in eng.calls] == [1, 2, 3, 4]              # one more picture every turn
    mm = res["mm_train_inputs"]
    assert mm["image_grid_thw"].tolist() == [[1, 4, 4]] * 4 and mm["pixel_values"].shape == (64, 1176)
    runs = image_runs(res["observation_tokens"], [tuple(g) for g in mm["image_grid_thw"].tolist()],
                      cfg.image_token_id, 2)
    assert len(runs) == 4 and len(res["action_ranges"]) == 4
