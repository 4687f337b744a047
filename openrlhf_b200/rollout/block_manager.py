"""KV page pool (native, reference counted) and the VMM arena that backs the KV cache.

``BlockManager`` binds the C++ ``PagePool`` of ``csrc/host_runtime.cu``; ``PyBlockManager`` is the pure-Python
restatement used where the native library is not built (CPU-only unit tests) and as the property-test oracle.
``VmmArena`` wraps a virtual address range whose physical memory can be dropped and re-created in place, so that the
rollout engine's sleep / wake keeps tensor addresses (and captured CUDA graphs) valid.
"""
from __future__ import annotations

import ctypes
import os

import torch


class PyBlockManager:
    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free_list = list(range(num_pages - 1, -1, -1))
        self.ref = [0] * num_pages

    def num_free(self) -> int:
        return len(self.free_list)

    def alloc(self) -> int:
        if not self.free_list:
            raise MemoryError("KV page pool exhausted")
        p = self.free_list.pop()
        self.ref[p] = 1
        return p

    def share(self, page: int) -> int:
        assert self.ref[page] > 0
        self.ref[page] += 1
        return page

    def free(self, page: int) -> None:
        assert self.ref[page] > 0, "double free of a KV page"
        self.ref[page] -= 1
        if self.ref[page] == 0:
            self.free_list.append(page)


def _native():
    from ..ops import _lib

    if not os.path.exists(_lib.LIB_PATH):
        return None
    L = _lib.lib()
    L.b200_pool_create.restype = ctypes.c_void_p
    L.b200_arena_create.restype = ctypes.c_void_p
    return L


class BlockManager:
    def __new__(cls, num_pages: int):
        L = _native()
        if L is None:
            return PyBlockManager(num_pages)
        self = super().__new__(cls)
        self._L = L
        self._h = ctypes.c_void_p(L.b200_pool_create(ctypes.c_int(num_pages)))
        self.num_pages = num_pages
        return self

    def num_free(self) -> int:
        return int(self._L.b200_pool_num_free(self._h))

    def alloc(self) -> int:
        p = int(self._L.b200_pool_alloc(self._h))
        if p < 0:
            raise MemoryError("KV page pool exhausted")
        return p

    def share(self, page: int) -> int:
        if self._L.b200_pool_share(self._h, ctypes.c_int(page)) < 0:
            raise AssertionError("sharing a page that is not allocated")
        return page

    def free(self, page: int) -> None:
        if self._L.b200_pool_free(self._h, ctypes.c_int(page)) < 0:
            raise AssertionError("double free of a KV page")

    def __del__(self):
        try:
            self._L.b200_pool_destroy(self._h)
        except Exception:  # noqa: BLE001
            pass


def admit(prompt_lens, max_new, n, free_rows: int, free_pages: int, page_size: int = 128, reserve_pages: int = 1) -> int:
    """How many queued requests (in order) fit into the free rows / pages (native when built, else Python)."""
    L = _native()
    cnt = len(prompt_lens)
    if L is None or cnt == 0:
        k = 0
        for p, m, s in zip(prompt_lens, max_new, n):
            pages = s * ((p + m) // page_size + 1)
            if s > free_rows or pages + reserve_pages > free_pages:
                break
            free_rows -= s
            free_pages -= pages
            k += 1
        return k
    arr = lambda x: (ctypes.c_int * cnt)(*[int(v) for v in x])
    return int(L.b200_admit(arr(prompt_lens), arr(max_new), arr(n), ctypes.c_int(cnt), ctypes.c_int(free_rows),
                            ctypes.c_int(free_pages), ctypes.c_int(page_size), ctypes.c_int(reserve_pages)))


class _RawCudaBuffer:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class VmmArena:
    """A device buffer at a fixed virtual address whose physical memory can be released (``unmap``) and re-created
    (``map``). ``tensor(dtype, shape)`` views it as a torch tensor; the view stays valid across unmap / map cycles
    (its contents do not)."""

    def __init__(self, nbytes: int, device: torch.device):
        L = _native()
        if L is None:
            raise RuntimeError("the native library is required for the VMM arena")
        self._L = L
        self.device = torch.device(device)
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        ptr, size = ctypes.c_ulonglong(0), ctypes.c_size_t(0)
        h = L.b200_arena_create(ctypes.c_size_t(nbytes), ctypes.c_int(idx), ctypes.byref(ptr), ctypes.byref(size))
        if not h:
            raise RuntimeError("could not reserve a virtual address range for the arena")
        self._h = ctypes.c_void_p(h)
        self.ptr, self.nbytes = int(ptr.value), int(size.value)
        self.map()
        self._bytes = torch.as_tensor(_RawCudaBuffer(self.ptr, self.nbytes), device=self.device)

    def map(self):
        rc = self._L.b200_arena_map(self._h)
        if rc != 0:
            raise MemoryError(f"arena map failed with code {rc}")

    def unmap(self):
        torch.cuda.synchronize(self.device)
        rc = self._L.b200_arena_unmap(self._h)
        if rc != 0:
            raise RuntimeError(f"arena unmap failed with code {rc}")

    @property
    def mapped(self) -> bool:
        return bool(self._L.b200_arena_is_mapped(self._h))

    def tensor(self, dtype: torch.dtype, shape) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty(0, dtype=dtype).element_size()
        assert nb <= self.nbytes
        return self._bytes[:nb].view(dtype).view(*shape)
