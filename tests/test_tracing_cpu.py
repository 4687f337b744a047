"""Span tracer: nesting, Chrome-trace JSON output, merge of spans from another process, RPC instants."""
import json

from openrlhf_b200.utils.tracing import Tracer, tracer


def test_spans_and_chrome_trace(tmp_path):
    t = Tracer().enable()
    with t.span("outer", cat="test", step=3):
        with t.span("inner", cat="test"):
            pass
    t.instant("marker", cat="test", k=1)
    t.merge([{"name": "from_worker", "cat": "w", "ph": "X", "ts": 1.0, "dur": 2.0, "pid": 1, "tid": 1, "args": {}}])
    path = t.dump(str(tmp_path / "trace.json"))
    ev = json.load(open(path))["traceEvents"]
    names = [e["name"] for e in ev]
    assert names == ["inner", "outer", "marker", "from_worker"]
    outer, inner = ev[1], ev[0]
    assert outer["ts"] <= inner["ts"] and outer["ts"] + outer["dur"] >= inner["ts"] + inner["dur"]
    assert outer["args"]["step"] == 3 and outer["ph"] == "X" and ev[2]["ph"] == "i"


def test_disabled_tracer_records_nothing():
    t = Tracer()
    with t.span("x"):
        pass
    t.instant("y")
    assert t.events() == []


def test_runtime_rpc_instants():
    from openrlhf_b200.runtime.core import WorkerHandle
    tracer.clear()
    tracer.enable()
    h = WorkerHandle("worker_stubs.EchoWorker", kwargs={"tag": "t"}, name="echo")
    try:
        h.wait_started()
        assert h.call("whoami").result(60)[0] == "t"
    finally:
        h.shutdown()
        tracer.disable()
    assert any(e["name"] == "rpc:whoami" and e["args"]["worker"] == "echo" for e in tracer.events())
    tracer.clear()
