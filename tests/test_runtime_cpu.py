"""Runtime tests on CPU processes: RPC, shared-memory tensors, concurrency of coroutine methods, chunked dispatch,
wait/cancel, remote exceptions, and failure detection (a worker that exits, a worker that stops answering)."""
import time

import pytest
import torch

from openrlhf_b200.runtime.core import (ActorGroup, CancelledError, RemoteError, WorkerDied, WorkerHandle, get, wait)

W = "worker_stubs.EchoWorker"


def test_rpc_tensors_and_coroutines():
    h = WorkerHandle(W, kwargs={"tag": "a"})
    h.wait_started()
    try:
        assert h.call("whoami").result(30)[0] == "a"
        t = torch.arange(1 << 16, dtype=torch.float32)
        out = h.call("add", t, k=2.0).result(30)
        assert torch.equal(out, t + 2)
        t0 = time.time()
        futs = [h.call("slow_echo", i, delay=0.3) for i in range(8)]
        assert get(futs, 30) == list(range(8))
        assert time.time() - t0 < 1.5          # ran concurrently, not 8 x 0.3 s
        with pytest.raises(RemoteError, match="intended failure"):
            h.call("boom").result(30)
        f = h.call("slow_echo", 1, delay=5.0)
        ready, pending = wait([f], num_returns=1, timeout=0.2)
        assert not ready and pending == [f]
        f.cancel()
        with pytest.raises(CancelledError):
            f.result(1)
        assert h.call("whoami").result(30)[0] == "a"      # still healthy after a cancel
    finally:
        h.shutdown()


def test_group_dispatch_and_collective():
    g = ActorGroup(W, 4, init_kwargs={"use_dist": True}, duplicate_actors=2, name="echo")
    try:
        ids = get(g.async_run_method("whoami"), 60)
        assert sorted(i[1] for i in ids) == [0, 1, 2, 3] and all(i[2] == 4 for i in ids)
        outs = get(g.async_run_method_batch("square", x=[1, 2, 3, 4, 5, 6]), 60)
        # two replicas of two duplicate ranks each: ranks 0,1 get [1,2,3]; ranks 2,3 get [4,5,6]
        assert [o[1] for o in outs[0]] == [1, 4, 9] and [o[1] for o in outs[1]] == [1, 4, 9]
        assert [o[1] for o in outs[2]] == [16, 25, 36] and outs[3] == [(3, 16), (3, 25), (3, 36)]
        assert get(g.async_run_method("all_reduce_sum", 1.5), 60) == [6.0] * 4
        with pytest.raises(ValueError):
            g.async_run_method_batch("square", x=[1])
    finally:
        g.shutdown()


def test_failure_detection_exit_and_stall():
    h = WorkerHandle(W, heartbeat_interval=0.1, heartbeat_timeout=1.0)
    h.wait_started()
    f = h.call("die")
    with pytest.raises(WorkerDied):
        f.result(20)
    assert not h.alive()
    with pytest.raises(WorkerDied):
        h.call("whoami").result(5)
    # a wedged (not dead) worker: a blocking call keeps the event loop busy but heartbeats keep coming, so a
    # call with a deadline times out on the controller instead of declaring the worker dead
    h2 = WorkerHandle(W, heartbeat_interval=0.1, heartbeat_timeout=5.0)
    h2.wait_started()
    try:
        f = h2.call("hang", 1.0)
        with pytest.raises(TimeoutError):
            f.result(0.2)
        assert h2.alive() and f.result(20) == "woke"
    finally:
        h2.shutdown()


def test_large_reply_travels_through_shared_memory_ring():
    """A worker created with shm_bytes > 0 returns big tensors through the native ring; small ones use the pipe."""
    import torch
    from openrlhf_b200.runtime.core import WorkerHandle
    from openrlhf_b200.utils import st_io
    if not st_io.available():
        pytest.skip("native library not built")
    h = WorkerHandle("worker_stubs.EchoWorker", kwargs={"tag": "ring"}, shm_bytes=8 << 20)
    try:
        h.wait_started()
        big = torch.randn(512, 1024)                      # 2 MiB reply
        out = h.call("add", big, 2.0).result(60)
        assert torch.equal(out, big + 2.0)
        small = torch.ones(4)
        assert torch.equal(h.call("add", small, 1.0).result(60), small + 1.0)
        outs = [h.call("add", big, float(i)) for i in range(6)]   # several in flight: order of markers = order in the ring
        for i, f in enumerate(outs):
            assert torch.equal(f.result(60), big + float(i))
    finally:
        h.shutdown()
