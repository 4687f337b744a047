"""Single-GPU checks of the collective kernels' host-visible behaviour (no peer process involved)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_symm_barrier_times_out_with_a_status_instead_of_hanging():
    """A peer that never arrives: the bounded wait runs out, the kernel returns, and the status word names the error
    and the missing peer. Both pad pointers are local and slot [channel][1] is never written, so nothing else is
    needed to make the wait expire; the context stays usable afterwards."""
    from openrlhf_b200.ops import _lib

    lib = _lib.lib()
    pad = torch.zeros(1024, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(ctypes.c_void_p(pad.data_ptr()), ctypes.c_void_p(pad.data_ptr()))
    rc = lib.b200_symm_barrier(ptrs, ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(0), ctypes.c_uint(1),
                               ctypes.c_double(0.02), ctypes.c_void_p(status.data_ptr()),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    assert st[0] == 5, st            # ERR_TIMEOUT_FLAG: "timeout waiting for a flag"
    assert st[1] == 1, st            # the peer whose slot never reached the epoch
    assert int(pad[0]) == 1          # this rank's own arrival was published
    # once the missing slot is written the same barrier passes and leaves the status untouched
    status.zero_()
    pad[1] = 1
    rc = lib.b200_symm_barrier(ptrs, ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(0), ctypes.c_uint(1),
                               ctypes.c_double(0.02), ctypes.c_void_p(status.data_ptr()),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert status.cpu().tolist()[:2] == [0, 0]
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0
