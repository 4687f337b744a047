"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of the kernel library may not allocate device memory (a decode thread that must stay out of the caching
allocator, an engine running while its memory pool is lent out, a host runtime that only holds raw device pointers).
For them ``b200_attn_decode_noalloc`` keeps the split-KV partial results in a fixed array inside the library. This
test checks it against the regular entry point (which takes a caller workspace) on two calls in a row, since every
call reuses the same built-in scratch and must not depend on what the previous call left there. The file name sorts
last so that a run stopping at the first failure has already executed every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, kc, vc, bt, sl, out, splits, scale, status):
    B, Hq, _ = q.shape
    fn = lib.b200_attn_decode_noalloc
    fn.restype = ctypes.c_int
    return fn(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(kc.data_ptr()), ctypes.c_void_p(vc.data_ptr()),
              ctypes.c_void_p(bt.data_ptr()), ctypes.c_void_p(sl.data_ptr()), ctypes.c_void_p(out.data_ptr()),
              ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(kc.shape[1]), ctypes.c_int(kc.shape[0] // 128),
              ctypes.c_int(bt.shape[1]), ctypes.c_int(splits), ctypes.c_float(scale),
              ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _case(B, Hq, Hkv, splits, lens, num_pages, max_pages, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    D, page = 128, 128
    kc = torch.randn(num_pages * page, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(num_pages * page, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    bt = torch.randperm(num_pages, device="cuda", generator=g)[: B * max_pages].reshape(B, max_pages).int()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    return q, kc, vc, bt, sl


def test_noalloc_decode_matches_regular_entry_point_twice():
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops.attention import paged_decode

    lib = _lib.lib()
    scale = 1 / math.sqrt(128)
    status = _lib.status_word(torch.device("cuda"))
    cases = [
        (4, 12, 2, 3, [1, 300, 1280, 640], 96, 10),               # ragged lengths, more splits than pages in row 0
        (6, 12, 2, 2, [129, 5, 1000, 128, 257, 900], 96, 10),     # second call reuses the scratch of the first
        (3, 12, 2, 1, [700, 1, 256], 96, 10),                     # splits == 1: the scratch is not touched at all
        (64, 32, 8, 4, [200] * 64, 130, 2),                       # B * Hq * splits == 8192: exactly the maximum
    ]
    for call, (B, Hq, Hkv, splits, lens, num_pages, max_pages) in enumerate(cases):
        q, kc, vc, bt, sl = _case(B, Hq, Hkv, splits, lens, num_pages, max_pages, seed=call)
        expect = paged_decode(q, kc, vc, bt, sl, scale, splits=splits)
        got = torch.empty_like(q)
        torch.cuda.synchronize()
        # the driver's own view of device memory: a cudaMalloc inside the library would show up here, which
        # torch.cuda.memory_allocated() (the caching allocator's bookkeeping) cannot see. The first call is excluded
        # because it may load the kernel's module lazily.
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, q, kc, vc, bt, sl, got, splits, scale, status)
        assert rc == 0, f"call {call}: rc {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == torch_before
        if call > 0:
            assert torch.cuda.mem_get_info()[0] >= free_before, f"call {call}: device memory was allocated"
        _lib.check_status()
        err = (got.float() - expect.float()).abs().max().item()
        ref = expect.float().abs().max().item()
        assert err <= 2e-2 * ref + 2e-2, f"call {call}: max err {err} (scale {ref})"
        # same kernel, same inputs, fixed merge order: the two entry points agree bit for bit
        assert torch.equal(got, expect), f"call {call}: outputs differ (max err {err})"


def test_noalloc_rejects_oversized_problem():
    from openrlhf_b200.ops import _lib

    lib = _lib.lib()
    B, Hq, Hkv, splits = 64, 32, 8, 8          # 64 * 32 * 8 = 16384 partial rows > 8192
    q = torch.zeros(B, Hq, 128, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(2 * 128, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    bt = torch.zeros(B, 1, device="cuda", dtype=torch.int32)
    sl = torch.ones(B, device="cuda", dtype=torch.int32)
    rc = _call_noalloc(lib, q, kc, kc, bt, sl, torch.empty_like(q), splits, 1.0, _lib.status_word(torch.device("cuda")))
    assert rc == -20
