"""Single-controller runtime: worker processes, RPC with futures, actor groups, heartbeats.

Plays the part Ray plays for the reference (raylet actors, ``ray.get / wait / cancel``, placement of one worker per
GPU: openrlhf/trainer/ray/launcher.py:17-373, openrlhf/cli/train_ppo_ray.py:24-50). Design:

* one OS process per worker, started with the ``spawn`` method; the worker pins its GPU, fills the torch.distributed
  environment (``MASTER_ADDR=127.0.0.1`` by default) and instantiates the worker class;
* requests and replies travel over ``torch.multiprocessing`` pipes, so CPU tensors inside any message are passed
  through shared memory (file-descriptor hand-off), not copied through the pipe;
* the worker runs an asyncio loop: coroutine methods become concurrent tasks (many outstanding generate calls feed
  one continuous batch), plain methods run inline in arrival order;
* a heartbeat thread in every worker lets the controller notice a dead or wedged process between steps; a call to a
  dead worker fails its future with ``WorkerDied`` instead of hanging the controller.
"""
from __future__ import annotations

import asyncio
import importlib
import inspect
import itertools
import os
import threading
import time
import traceback
from typing import Any, Callable

import torch.multiprocessing as mp


class RemoteError(RuntimeError):
    """An exception raised inside a worker, re-raised in the controller with the remote traceback."""


class WorkerDied(RuntimeError):
    """The worker process exited or stopped sending heartbeats before answering."""


class CancelledError(RuntimeError):
    pass


class Future:
    def __init__(self, owner: "WorkerHandle | None" = None, call_id: int = -1):
        self._ev = threading.Event()
        self._value: Any = None
        self._exc: BaseException | None = None
        self._owner, self._id = owner, call_id
        self._callbacks: list[Callable] = []

    def set_result(self, value):
        self._value = value
        self._ev.set()
        for cb in self._callbacks:
            cb(self)

    def set_exception(self, exc: BaseException):
        self._exc = exc
        self._ev.set()
        for cb in self._callbacks:
            cb(self)

    def add_done_callback(self, cb):
        self._callbacks.append(cb)
        if self._ev.is_set():
            cb(self)

    def done(self) -> bool:
        return self._ev.is_set()

    def result(self, timeout: float | None = None):
        if not self._ev.wait(timeout):
            raise TimeoutError("remote call did not finish in time")
        if self._exc is not None:
            raise self._exc
        return self._value

    def cancel(self) -> None:
        """Best effort: the controller stops waiting; a coroutine call still running in the worker is cancelled."""
        if not self._ev.is_set():
            if self._owner is not None:
                self._owner._send(("cancel", self._id, None, None, None))
            self.set_exception(CancelledError("cancelled by the controller"))


def get(x, timeout: float | None = None):
    """Resolve a future or a (nested) list of futures, like ``ray.get``."""
    if isinstance(x, Future):
        return x.result(timeout)
    if isinstance(x, (list, tuple)):
        return [get(v, timeout) for v in x]
    return x


def wait(futures: list[Future], num_returns: int = 1, timeout: float | None = None):
    """Split `futures` into (ready, pending) once `num_returns` are done or the timeout passes, like ``ray.wait``."""
    deadline = None if timeout is None else time.monotonic() + timeout
    cond = threading.Condition()

    def poke(_):
        with cond:
            cond.notify_all()

    for f in futures:
        f.add_done_callback(poke)
    with cond:
        while True:
            ready = [f for f in futures if f.done()]
            if len(ready) >= min(num_returns, len(futures)):
                break
            left = None if deadline is None else deadline - time.monotonic()
            if left is not None and left <= 0:
                break
            cond.wait(left if left is not None else 1.0)
    ready = [f for f in futures if f.done()][:max(num_returns, 0) or None]
    return ready, [f for f in futures if f not in ready]


# ---------------------------------------------------------------------------------------------------- worker side
def _resolve(spec):
    if isinstance(spec, str):
        mod, _, name = spec.rpartition(".")
        return getattr(importlib.import_module(mod), name)
    return spec


def _heartbeat(conn, interval: float, stop: threading.Event):
    while not stop.wait(interval):
        try:
            conn.send(time.time())
        except (OSError, BrokenPipeError):
            return


class _ViaRing:
    """Pipe marker: the payload of this reply travels through the worker's shared-memory ring."""


def _tensor_bytes(obj) -> int:
    import torch

    if isinstance(obj, torch.Tensor):
        return obj.numel() * obj.element_size()
    if isinstance(obj, dict):
        return sum(_tensor_bytes(v) for v in obj.values())
    if isinstance(obj, (list, tuple)):
        return sum(_tensor_bytes(v) for v in obj)
    return 0


def _worker_main(cls_spec, init_args, init_kwargs, env: dict, req, rep, hb, hb_interval: float, ring_name=None):
    os.environ.update({k: str(v) for k, v in env.items()})
    ring = None
    if ring_name:
        from .shm import ShmChannel

        ring = ShmChannel.attach(ring_name)
    stop = threading.Event()
    threading.Thread(target=_heartbeat, args=(hb, hb_interval, stop), daemon=True).start()
    try:
        obj = _resolve(cls_spec)(*init_args, **init_kwargs)
        rep.send((-1, True, None))
    except BaseException as e:  # noqa: BLE001
        rep.send((-1, False, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        return
    loop = asyncio.new_event_loop()
    asyncio.set_event_loop(loop)
    tasks: dict[int, asyncio.Task] = {}
    send_lock = threading.Lock()

    def reply(call_id, ok, payload):
        with send_lock:
            try:
                # large tensor payloads go through the native shared-memory ring (one memcpy, no pickling of the
                # bytes); the pipe only carries a marker, so ring messages and markers stay in the same order
                if ring is not None and ok and 65536 <= _tensor_bytes(payload) < ring.capacity // 2:
                    ring.send(payload, timeout=120.0)
                    payload = _ViaRing()
                rep.send((call_id, ok, payload))
            except (OSError, BrokenPipeError):
                pass

    async def run_coro(call_id, coro):
        try:
            reply(call_id, True, await coro)
        except asyncio.CancelledError:
            reply(call_id, False, "cancelled")
        except BaseException as e:  # noqa: BLE001
            reply(call_id, False, f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
        finally:
            tasks.pop(call_id, None)

    async def serve():
        while True:
            while not req.poll():
                await asyncio.sleep(0.0005)
            try:
                kind, call_id, method, args, kwargs = req.recv()
            except (EOFError, OSError):
                return
            if kind == "stop":
                return
            if kind == "cancel":
                t = tasks.get(call_id)
                if t is not None:
                    t.cancel()
                continue
            try:
                fn = getattr(obj, method)
                if inspect.iscoroutinefunction(fn):
                    tasks[call_id] = loop.create_task(run_coro(call_id, fn(*args, **kwargs)))
                else:
                    reply(call_id, True, fn(*args, **kwargs))
            except BaseException as e:  # noqa: BLE001
                reply(call_id, False, f"{type(e).__name__}: {e}\n{traceback.format_exc()}")

    try:
        loop.run_until_complete(serve())
    finally:
        stop.set()
        for t in list(tasks.values()):
            t.cancel()
        if hasattr(obj, "shutdown"):
            try:
                obj.shutdown()
            except Exception:  # noqa: BLE001
                pass


# ---------------------------------------------------------------------------------------------------- controller side
class WorkerHandle:
    """Proxy of one worker process. ``handle.call("method", ...)`` returns a Future."""

    def __init__(self, cls_spec, args=(), kwargs=None, env: dict | None = None, heartbeat_interval: float = 1.0,
                 heartbeat_timeout: float = 30.0, start_timeout: float = 600.0, name: str = "worker",
                 shm_bytes: int = 0):
        ctx = mp.get_context("spawn")
        self._ring = None
        if shm_bytes > 0:
            from .shm import ShmChannel

            self._ring = ShmChannel(capacity=shm_bytes)
        self._req_r, self._req_w = ctx.Pipe(duplex=False)
        self._rep_r, self._rep_w = ctx.Pipe(duplex=False)
        self._hb_r, self._hb_w = ctx.Pipe(duplex=False)
        self.name = name
        self.heartbeat_timeout = heartbeat_timeout
        self.last_heartbeat = time.time()
        self._ids = itertools.count()
        self._futures: dict[int, Future] = {}
        self._lock = threading.Lock()
        self._dead: str | None = None
        self.proc = ctx.Process(target=_worker_main, daemon=True,
                                args=(cls_spec, args, kwargs or {}, env or {}, self._req_r, self._rep_w, self._hb_w,
                                      heartbeat_interval, self._ring.name if self._ring is not None else None))
        self.proc.start()
        self._started = Future()
        threading.Thread(target=self._pump, daemon=True).start()
        self._start_timeout = start_timeout

    def wait_started(self):
        ok = self._started.result(self._start_timeout)
        return ok

    # -- background thread: replies + heartbeats + liveness
    def _pump(self):
        while True:
            try:
                if self._hb_r.poll():
                    self.last_heartbeat = self._hb_r.recv()
                if self._rep_r.poll(0.05):
                    call_id, ok, payload = self._rep_r.recv()
                    if isinstance(payload, _ViaRing):
                        payload = self._ring.recv(timeout=120.0)
                    if call_id == -1:
                        self.last_heartbeat = time.time()
                        if ok:
                            self._started.set_result(True)
                        else:
                            self._started.set_exception(RemoteError(payload))
                        continue
                    with self._lock:
                        fut = self._futures.pop(call_id, None)
                    if fut is not None and not fut.done():
                        fut.set_result(payload) if ok else fut.set_exception(RemoteError(payload))
                    continue
            except (EOFError, OSError):
                self._fail_all("pipe closed")
                return
            if not self.proc.is_alive():
                self._fail_all(f"process exited with code {self.proc.exitcode}")
                return
            # heartbeats are only expected once the worker has finished importing and constructing its object
            if self._started.done() and time.time() - self.last_heartbeat > self.heartbeat_timeout:
                self._fail_all(f"no heartbeat for {self.heartbeat_timeout:.0f} s")
                return

    def _fail_all(self, why: str):
        self._dead = why
        with self._lock:
            futs, self._futures = list(self._futures.values()), {}
        for f in futs + [self._started]:
            if not f.done():
                f.set_exception(WorkerDied(f"{self.name}: {why}"))

    def alive(self) -> bool:
        return self._dead is None and self.proc.is_alive()

    def _send(self, msg):
        try:
            self._req_w.send(msg)
        except (OSError, BrokenPipeError):
            pass

    def call(self, method: str, *args, **kwargs) -> Future:
        from ..utils.tracing import tracer

        tracer.instant(f"rpc:{method}", cat="runtime", worker=self.name)
        call_id = next(self._ids)
        fut = Future(self, call_id)
        if self._dead is not None:
            fut.set_exception(WorkerDied(f"{self.name}: {self._dead}"))
            return fut
        with self._lock:
            self._futures[call_id] = fut
        self._send(("call", call_id, method, args, kwargs))
        return fut

    def __getattr__(self, method):
        if method.startswith("_"):
            raise AttributeError(method)

        class _Remote:
            def __init__(s, h, m):
                s.h, s.m = h, m

            def remote(s, *a, **kw):
                return s.h.call(s.m, *a, **kw)

        return _Remote(self, method)

    def shutdown(self, timeout: float = 10.0):
        self._send(("stop", -1, None, None, None))
        self.proc.join(timeout)
        if self.proc.is_alive():
            self.proc.terminate()


def batch_engine_call(engines: list, method_name: str, *args, **kwargs) -> list:
    """Call the same method on every engine handle and gather the results (the reference's batch_vllm_engine_call,
    openrlhf/trainer/ray/vllm_engine.py:316-329)."""
    return get([e.call(method_name, *args, **kwargs) for e in engines])


def free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class ActorGroup:
    """A set of worker processes forming one torch.distributed world (one per GPU).

    ``async_run_method`` broadcasts a call; ``async_run_method_batch`` slices list arguments into one chunk per
    data-parallel replica and sends the same chunk to the ``duplicate_actors = ring_attn_size x tensor_parallel_size``
    ranks of a replica (openrlhf/trainer/ray/launcher.py:319-373)."""

    def __init__(self, cls_spec, num_workers: int, init_kwargs: dict | None = None, gpu_ids: list[int] | None = None,
                 duplicate_actors: int = 1, backend_env: dict | None = None, name: str = "group",
                 heartbeat_timeout: float = 30.0):
        self.duplicate_actors = max(1, duplicate_actors)
        port = free_port()
        self.workers: list[WorkerHandle] = []
        for r in range(num_workers):
            env = {"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": port, "WORLD_SIZE": num_workers, "RANK": r,
                   "LOCAL_RANK": gpu_ids[r] if gpu_ids else r}
            env.update(backend_env or {})
            self.workers.append(WorkerHandle(cls_spec, kwargs=dict(init_kwargs or {}), env=env, name=f"{name}[{r}]",
                                             heartbeat_timeout=heartbeat_timeout))
        for w in self.workers:
            w.wait_started()

    def __len__(self):
        return len(self.workers)

    def alive(self) -> bool:
        return all(w.alive() for w in self.workers)

    def async_run_method(self, method_name: str, *args, **kwargs) -> list[Future]:
        return [w.call(method_name, *args, **kwargs) for w in self.workers]

    def async_run_method_batch(self, method_name: str, **kwargs) -> list[Future]:
        lengths = {len(v) for v in kwargs.values()}
        if len(lengths) != 1:
            raise ValueError("all batched arguments must have the same length")
        total = lengths.pop()
        replicas = len(self.workers) // self.duplicate_actors
        if total < replicas:
            raise ValueError(f"{total} items cannot be spread over {replicas} data-parallel replicas")
        per = (total + replicas - 1) // replicas
        futs = []
        for i, w in enumerate(self.workers):
            rep = i // self.duplicate_actors
            chunk = {k: v[rep * per:(rep + 1) * per] for k, v in kwargs.items()}
            futs.append(w.call("execute_batch", method_name, chunk))
        return futs

    def shutdown(self):
        for w in self.workers:
            w.shutdown()
