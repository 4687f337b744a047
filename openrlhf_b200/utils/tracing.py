"""Span tracer: host wall-clock spans (optionally paired with CUDA events for device time) that can be dumped as a
Chrome-trace JSON (chrome://tracing, Perfetto) and are mirrored as NVTX ranges when CUDA is available.

The reference has no profiler integration, only host-side ``timing/*`` entries in the step status
(openrlhf/trainer/ppo_trainer.py:215-258). Those keys are kept (trainer/hybrid_engine.py times the phases with CUDA
events); this module adds what a timeline view needs: nested spans from the controller, the workers and the
runtime's RPC layer in one file.

    from openrlhf_b200.utils.tracing import tracer
    tracer.enable()
    with tracer.span("generation", cat="rl"):
        ...
    tracer.dump("trace.json")

Enabled by OPENRLHF_B200_TRACE=<path> as well: the trace is then written at interpreter exit.
"""
from __future__ import annotations

import atexit
import json
import os
import threading
import time
from contextlib import contextmanager


class Tracer:
    def __init__(self):
        self.enabled = False
        self.device_time = False
        self._events: list[dict] = []
        self._pending: list[tuple] = []      # (event dict, cuda start event, cuda end event)
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()
        self._path = None

    def enable(self, device_time: bool = False, path: str | None = None):
        self.enabled, self.device_time, self._path = True, device_time, path
        return self

    def disable(self):
        self.enabled = False

    @contextmanager
    def span(self, name: str, cat: str = "app", **args):
        if not self.enabled:
            yield
            return
        cuda = None
        try:
            import torch

            if torch.cuda.is_available():
                cuda = torch.cuda
        except Exception:  # noqa: BLE001
            cuda = None
        ev0 = ev1 = None
        if cuda is not None:
            cuda.nvtx.range_push(name)
            if self.device_time:
                ev0, ev1 = cuda.Event(enable_timing=True), cuda.Event(enable_timing=True)
                ev0.record()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            t1 = time.perf_counter()
            if ev1 is not None:
                ev1.record()
            if cuda is not None:
                cuda.nvtx.range_pop()
            ev = {"name": name, "cat": cat, "ph": "X", "ts": (t0 - self._t0) * 1e6, "dur": (t1 - t0) * 1e6,
                  "pid": os.getpid(), "tid": threading.get_ident() % 100000, "args": dict(args)}
            with self._lock:
                self._events.append(ev)
                if ev1 is not None:
                    self._pending.append((ev, ev0, ev1))

    def instant(self, name: str, cat: str = "app", **args):
        if self.enabled:
            with self._lock:
                self._events.append({"name": name, "cat": cat, "ph": "i", "s": "p",
                                     "ts": (time.perf_counter() - self._t0) * 1e6, "pid": os.getpid(),
                                     "tid": threading.get_ident() % 100000, "args": dict(args)})

    def _resolve_device_times(self):
        for ev, e0, e1 in self._pending:
            try:
                e1.synchronize()
                ev["args"]["device_ms"] = e0.elapsed_time(e1)
            except Exception:  # noqa: BLE001
                pass
        self._pending.clear()

    def events(self) -> list[dict]:
        with self._lock:
            self._resolve_device_times()
            return list(self._events)

    def merge(self, events: list[dict]):
        """Add spans recorded in another process (workers return theirs through the runtime)."""
        with self._lock:
            self._events.extend(events)

    def dump(self, path: str | None = None) -> str:
        path = path or self._path or "trace.json"
        with open(path, "w") as f:
            json.dump({"traceEvents": self.events(), "displayTimeUnit": "ms"}, f)
        return path

    def clear(self):
        with self._lock:
            self._events.clear()
            self._pending.clear()


tracer = Tracer()

_env = os.environ.get("OPENRLHF_B200_TRACE")
if _env:
    tracer.enable(device_time=os.environ.get("OPENRLHF_B200_TRACE_DEVICE", "0") == "1",
                  path=_env.replace("%p", str(os.getpid())))
    atexit.register(lambda: tracer.dump())
