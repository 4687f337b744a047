"""Shared-memory message channel between two processes of one node (native ring: csrc/host_io.cu).

``ShmChannel`` is single-producer / single-consumer. ``send`` takes a picklable object; tensors inside it are pulled
out and their bytes are written into the ring directly from tensor memory, next to a small pickled skeleton, so large
rollout / experience payloads cost one memcpy in and one out. Every wait has a deadline (TimeoutError).
The reference moves such payloads through Ray's object store (ray.put / ray.get in
openrlhf/trainer/ray/launcher.py:226-373).
"""
from __future__ import annotations

import ctypes
import os
import pickle
import uuid

import torch


def _lib():
    from ..ops import _lib as L

    lib = L.lib()
    lib.b200_ring_open.restype = ctypes.c_void_p
    lib.b200_ring_peek.restype = ctypes.c_longlong
    lib.b200_ring_capacity.restype = ctypes.c_longlong
    return lib


class _TensorRef:
    __slots__ = ("dtype", "shape", "nbytes")

    def __init__(self, t: torch.Tensor):
        self.dtype, self.shape, self.nbytes = t.dtype, tuple(t.shape), t.numel() * t.element_size()


def _extract(obj, out: list):
    """Replace CPU tensors by _TensorRef placeholders (depth-first order defines the byte layout)."""
    if isinstance(obj, torch.Tensor):
        t = obj.detach()
        t = (t.cpu() if t.is_cuda else t).contiguous()
        out.append(t)
        return _TensorRef(t)
    if isinstance(obj, dict):
        return {k: _extract(v, out) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        vals = [_extract(v, out) for v in obj]
        return type(obj)(vals) if not hasattr(obj, "_fields") else type(obj)(*vals)
    return obj


def _restore(obj, buf: memoryview, pos: list):
    if isinstance(obj, _TensorRef):
        raw = buf[pos[0]:pos[0] + obj.nbytes]
        pos[0] += obj.nbytes
        t = torch.frombuffer(bytearray(raw), dtype=obj.dtype) if obj.nbytes else torch.empty(0, dtype=obj.dtype)
        return t.reshape(obj.shape)
    if isinstance(obj, dict):
        return {k: _restore(v, buf, pos) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        vals = [_restore(v, buf, pos) for v in obj]
        return type(obj)(vals) if not hasattr(obj, "_fields") else type(obj)(*vals)
    return obj


class ShmChannel:
    def __init__(self, name: str | None = None, capacity: int = 256 << 20, create: bool = True):
        self.name = name or f"/b200_{os.getpid()}_{uuid.uuid4().hex[:12]}"
        self._lib = _lib()
        self._h = self._lib.b200_ring_open(self.name.encode(), ctypes.c_longlong(capacity), ctypes.c_int(int(create)))
        if not self._h:
            raise OSError(f"cannot {'create' if create else 'open'} shared-memory ring {self.name}")
        self.capacity = int(self._lib.b200_ring_capacity(ctypes.c_void_p(self._h)))

    @classmethod
    def attach(cls, name: str) -> "ShmChannel":
        return cls(name, 0, create=False)

    def send(self, obj, timeout: float = 60.0) -> None:
        tensors: list[torch.Tensor] = []
        skel = pickle.dumps(_extract(obj, tensors), protocol=pickle.HIGHEST_PROTOCOL)
        head = len(skel).to_bytes(8, "little") + skel
        parts = [head] + tensors
        k = len(parts)
        keep = ctypes.create_string_buffer(head, len(head))
        ptrs = (ctypes.c_void_p * k)(ctypes.cast(keep, ctypes.c_void_p),
                                     *[ctypes.c_void_p(t.data_ptr()) for t in tensors])
        lens = (ctypes.c_longlong * k)(len(head), *[t.numel() * t.element_size() for t in tensors])
        rc = self._lib.b200_ring_send(ctypes.c_void_p(self._h), ctypes.c_int(k), ptrs, lens,
                                      ctypes.c_int(int(timeout * 1000)))
        if rc == -1:
            raise TimeoutError("shared-memory ring: no space before the deadline")
        if rc == -2:
            raise BrokenPipeError("shared-memory ring closed by the peer")
        if rc == -3:
            raise ValueError("message larger than the ring capacity")

    def recv(self, timeout: float = 60.0):
        n = self._lib.b200_ring_peek(ctypes.c_void_p(self._h), ctypes.c_int(int(timeout * 1000)))
        if n == -1:
            raise TimeoutError("shared-memory ring: no message before the deadline")
        if n == -2:
            raise EOFError("shared-memory ring closed by the peer")
        buf = bytearray(n)
        cbuf = (ctypes.c_char * n).from_buffer(buf) if n else None
        if self._lib.b200_ring_recv(ctypes.c_void_p(self._h), cbuf, ctypes.c_longlong(n)) != 0:
            raise OSError("shared-memory ring: truncated message")
        view = memoryview(buf)
        k = int.from_bytes(view[:8], "little")
        skel = pickle.loads(view[8:8 + k])
        return _restore(skel, view, [8 + k])

    def close(self, mark_closed: bool = True) -> None:
        if self._h:
            self._lib.b200_ring_close(ctypes.c_void_p(self._h), ctypes.c_int(int(mark_closed)))
            self._h = None

    def __del__(self):
        try:
            self.close(False)
        except Exception:  # noqa: BLE001
            pass
