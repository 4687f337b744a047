"""Safetensors files written and read by the native parallel writer / reader (csrc/host_io.cu).

The file format is the public safetensors layout (u64 little-endian header length, JSON header padded with spaces to a
multiple of 8 bytes, then the tensors' bytes back to back), so files are interchangeable with the ``safetensors``
package; only the data movement is native: one pwrite / pread stream per thread straight from / into the tensors'
host memory. The reference writes checkpoints tensor by tensor on rank 0 through ``save_pretrained``
(openrlhf/utils/deepspeed/deepspeed.py:560-640).
"""
from __future__ import annotations

import ctypes
import json
import os
import struct

import torch

_DTYPES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.float64: "F64",
           torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
           torch.bool: "BOOL"}
_FROM = {v: k for k, v in _DTYPES.items()}


def _lib():
    from ..ops import _lib as L

    return L.lib()


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict[str, str] | None = None, threads: int = 8,
              fsync: bool = False) -> None:
    """tensors: name -> tensor (any device; device tensors are staged through host memory). Names are laid out in
    sorted order, as the safetensors package does."""
    names = sorted(tensors)
    host = []
    for n in names:
        t = tensors[n].detach()
        t = t.cpu() if t.is_cuda else t
        host.append(t.contiguous())
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    offsets, sizes = [], []
    for n, t in zip(names, host):
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _DTYPES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        offsets.append(off)
        sizes.append(nbytes)
        off += nbytes
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((-len(hb)) % 8)
    k = len(names)
    ptrs = (ctypes.c_void_p * k)(*[ctypes.c_void_p(t.data_ptr()) for t in host])
    rc = _lib().b200_st_write(path.encode(), hb, ctypes.c_longlong(len(hb)), ctypes.c_int(k), ptrs,
                              (ctypes.c_longlong * k)(*sizes), (ctypes.c_longlong * k)(*offsets), ctypes.c_int(threads),
                              ctypes.c_int(int(fsync)))
    if rc != 0:
        raise OSError(f"native safetensors write of {path} failed (code {rc})")


def read_header(path: str) -> tuple[dict, int]:
    """(header dict, byte offset of the data section)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return header, 8 + n


def load_file(path: str, names: list[str] | None = None, threads: int = 8, pin: bool = False) -> dict[str, torch.Tensor]:
    """Reads the named tensors (default: all) into freshly allocated host tensors with parallel preads."""
    header, data0 = read_header(path)
    header.pop("__metadata__", None)
    names = sorted(header) if names is None else names
    out, ptrs, sizes, offsets = {}, [], [], []
    for n in names:
        e = header[n]
        t = torch.empty(e["shape"], dtype=_FROM[e["dtype"]], pin_memory=pin)
        out[n] = t
        ptrs.append(ctypes.c_void_p(t.data_ptr()))
        sizes.append(e["data_offsets"][1] - e["data_offsets"][0])
        offsets.append(e["data_offsets"][0])
        assert sizes[-1] == t.numel() * t.element_size(), f"size mismatch for {n}"
    k = len(names)
    if k:
        rc = _lib().b200_st_read(path.encode(), ctypes.c_longlong(data0), ctypes.c_int(k), (ctypes.c_void_p * k)(*ptrs),
                                 (ctypes.c_longlong * k)(*sizes), (ctypes.c_longlong * k)(*offsets),
                                 ctypes.c_int(threads))
        if rc != 0:
            raise OSError(f"native safetensors read of {path} failed (code {rc})")
    return out


def metadata(path: str) -> dict[str, str]:
    return read_header(path)[0].get("__metadata__", {}) or {}


def available() -> bool:
    try:
        return hasattr(_lib(), "b200_st_write")
    except Exception:  # noqa: BLE001
        return False
