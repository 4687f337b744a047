"""Native safetensors writer / reader (interchangeable with the safetensors package) and the shared-memory ring."""
import multiprocessing as mp
import os

import pytest
import torch

from openrlhf_b200.runtime.shm import ShmChannel
from openrlhf_b200.utils import st_io

pytestmark = pytest.mark.skipif(not st_io.available(), reason="native library not built")


def test_safetensors_round_trip_and_interop(tmp_path):
    from safetensors.torch import load_file as ref_load, save_file as ref_save
    torch.manual_seed(0)
    tensors = {"a.weight": torch.randn(300, 77).to(torch.bfloat16), "b": torch.arange(10, dtype=torch.int64),
               "c": torch.randn(5, 3, 2), "empty": torch.zeros(0, 4), "big": torch.randn(40_000_000 // 4)}
    p = str(tmp_path / "native.safetensors")
    st_io.save_file(tensors, p, metadata={"format": "pt", "lo": "3"}, threads=4)
    ref = ref_load(p)                                   # the reference implementation reads our file
    got = st_io.load_file(p, threads=4)
    for k, v in tensors.items():
        assert torch.equal(ref[k], v) and torch.equal(got[k], v), k
    assert st_io.metadata(p)["lo"] == "3"
    p2 = str(tmp_path / "ref.safetensors")
    ref_save(tensors, p2)                               # and we read theirs
    got2 = st_io.load_file(p2, names=["big", "a.weight"])
    assert torch.equal(got2["big"], tensors["big"]) and torch.equal(got2["a.weight"], tensors["a.weight"])


def _producer(name, n):
    ch = ShmChannel.attach(name)
    for i in range(n):
        ch.send({"i": i, "x": torch.full((1000 + i, 7), float(i)), "nested": [torch.arange(i), ("s", 1.5)]})
    ch.send(None)
    ch.close(False)


def test_ring_between_processes():
    ch = ShmChannel(capacity=1 << 20)                  # small ring: messages wrap around and the producer has to wait
    p = mp.get_context("spawn").Process(target=_producer, args=(ch.name, 200))
    p.start()
    for i in range(200):
        m = ch.recv(timeout=60)
        assert m["i"] == i and m["x"].shape == (1000 + i, 7) and float(m["x"][0, 0]) == float(i)
        assert torch.equal(m["nested"][0], torch.arange(i)) and m["nested"][1] == ("s", 1.5)
    assert ch.recv(timeout=60) is None
    p.join(30)
    assert p.exitcode == 0
    ch.close()


def test_ring_deadlines():
    ch = ShmChannel(capacity=4096)
    with pytest.raises(TimeoutError):
        ch.recv(timeout=0.05)
    with pytest.raises(ValueError):
        ch.send(torch.zeros(10_000))
    ch.send(torch.zeros(500))
    with pytest.raises(TimeoutError):                   # ring full, nobody reads
        ch.send(torch.zeros(800), timeout=0.05)
    ch.close()
