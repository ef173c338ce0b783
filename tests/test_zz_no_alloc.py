"""GPU: the allocation-free VM entry point against the regular one.

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
Hosts that own the whole device through their own arena, or that cannot afford the device-wide synchronisation of an
allocation inside a latency-critical loop, cannot call cudaMalloc from a plug-in; pimb200_gemv_vm_static serves them
from a fixed scratch inside the library image.  It must give the regular entry point's result, call after call,
although every call reuses the same scratch."""
import pytest
import torch

from tests.util import assert_close, h16, to_dev

pytestmark = pytest.mark.gpu


def _lib():
    from pimaicompiler_b200 import _lib, ops
    ops.init()   # only the regular entry point needs it
    return _lib.lib(), _lib


@pytest.mark.parametrize("K,N", [(1024, 4096), (320, 1280), (2048, 1024), (64, 32768), (2048, 32768), (1024, 16384)])
def test_static_scratch_vm_matches_regular_entry_point_twice_in_a_row(K, N):
    lib, L = _lib()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(K + N)
    A = to_dev(h16((torch.rand(K, N, generator=g) * 2 - 1) / K ** 0.5))
    b = to_dev(h16(torch.randn(N, generator=g)))
    for call in range(2):   # two calls in a row: the second starts from the scratch the first one left behind
        x = to_dev(h16(torch.randn(K, generator=g)))
        act = L.ACT_RELU if call == 0 else L.ACT_NONE
        y_ref = torch.empty(N, dtype=torch.float16, device="cuda")
        y_new = torch.full((N,), 7.0, dtype=torch.float16, device="cuda")
        assert lib.pimb200_gemv_vm(x.data_ptr(), A.data_ptr(), b.data_ptr(), y_ref.data_ptr(), K, N, act, st) == L.OK
        assert lib.pimb200_gemv_vm_static(x.data_ptr(), A.data_ptr(), b.data_ptr(), y_new.data_ptr(), K, N, act,
                                          st) == L.OK
        torch.cuda.synchronize()
        # same kernel; only the K split (hence the fp32 summation order) may differ: the GEMV tolerance of the suite
        assert_close(y_new, y_ref.float().cpu(), 2e-3, 1e-3, f"static VM call {call} {K}x{N}")
        # and directly against the C oracle (the largest widths run the widest K splits the scratch is sized for:
        # 5 partial rows of 32768 columns, 10 of 16384)
        from oracle import c_oracle as co
        ref = co.vm(x.float().cpu().numpy(), A.float().cpu().numpy(), b.float().cpu().numpy(), call == 0)
        assert_close(y_new, ref, 2e-3, 1e-3, f"static VM vs oracle, call {call} {K}x{N}")


def test_static_scratch_vm_refuses_what_does_not_fit():
    lib, L = _lib()
    t = torch.zeros(64, dtype=torch.float16, device="cuda")
    p = t.data_ptr()
    assert lib.pimb200_gemv_vm_static(p, p, None, p, 8, 32768 + 8, 0, None) == L.ERR_UNSUPPORTED   # N beyond the scratch
    assert lib.pimb200_gemv_vm_static(p, p, None, p, 8, 29, 0, None) == L.ERR_UNSUPPORTED          # N not a multiple of 8
    assert lib.pimb200_gemv_vm_static(p, p + 2, None, p, 8, 8, 0, None) == L.ERR_UNSUPPORTED       # unaligned matrix
    assert lib.pimb200_gemv_vm_static(None, p, None, p, 8, 8, 0, None) == L.ERR_BAD_ARG
    assert b"unsupported" in lib.pimb200_status_string(L.ERR_UNSUPPORTED)
