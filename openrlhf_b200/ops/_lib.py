"""ctypes binding of the sm_100a kernel library (``libopenrlhf_b200.so``).

The library is built in-tree by ``openrlhf_b200.csrc.build``. Tensors are passed as raw device pointers and the
current CUDA stream as an opaque handle, so no PyTorch C++ headers are involved. On a machine with a GPU a missing
library is an error, never a silent fallback.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import threading

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libopenrlhf_b200.so")

_lib = None
_lock = threading.Lock()
_status_bufs: dict[int, torch.Tensor] = {}

ERROR_NAMES = {
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free stage",
    3: "timeout waiting for an accumulator",
    4: "timeout waiting for a free accumulator",
    5: "timeout waiting for a flag",
    6: "bad argument",
}


class KernelError(RuntimeError):
    """A kernel reported a non-zero status word (for instance a bounded wait that ran out)."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    from openrlhf_b200.csrc.build import build

                    build()
                _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def available() -> bool:
    return torch.cuda.is_available()


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """One int32 per device that kernels write their error code to (0 = ok)."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    buf = _status_bufs.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _status_bufs[idx] = buf
    return buf


def check_status(device: torch.device | None = None) -> None:
    """Synchronising check of the status word; raises KernelError and clears it if a kernel failed."""
    buf = status_word(device)
    code = int(buf[0].item())
    if code != 0:
        buf.zero_()
        raise KernelError(f"kernel status {code}: {ERROR_NAMES.get(code, 'unknown')}")


@contextlib.contextmanager
def decode_chain():
    """Kernels launched inside this block form a decode chain: they carry the programmatic-dependent-launch attribute
    (a kernel's prologue overlaps its predecessor's tail) and GEMMs fetch their first weight tiles before they wait
    for the predecessor. Only valid where no kernel of the chain writes a GEMM's B operand."""
    old = lib().b200_set_pdl(ctypes.c_int(1))
    try:
        yield
    finally:
        lib().b200_set_pdl(ctypes.c_int(old))


LAUNCHES = 0  # number of kernel launches issued through this library (graph replays add their captured count)


def count_launches(n: int) -> None:
    global LAUNCHES
    LAUNCHES += n


def check_rc(rc: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise KernelError(f"{what}: launch failed with code {rc}")
