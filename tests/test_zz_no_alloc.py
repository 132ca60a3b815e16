"""The allocation-free channel mean (`paro_channel_mean_noalloc`) against the regular entry point.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  The entry point exists for callers that may not allocate device memory (a frozen memory pool,
a host without an allocator, a loop that cannot afford a cudaMalloc stall); its scratch is a fixed
array inside the library that every call shares, so the test calls it twice in a row with different
problems and checks that nothing of the first call leaks into the second.  Both entry points are
called through the C ABI with ctypes; equality is exact, as in the other channel-mean tests.
"""
import ctypes

import pytest
import torch

from paroatten_b200 import _lib

pytestmark = pytest.mark.gpu


def _mean(fn_name, x, with_scratch):
    L = _lib.lib()
    B, H, N, D = x.shape
    out = torch.empty(B, H, D, dtype=x.dtype, device=x.device)
    out32 = torch.empty(B, H, D, dtype=torch.float32, device=x.device)
    args = [x.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, x.stride(0), x.stride(1), x.stride(2),
            out.data_ptr(), out32.data_ptr()]
    if with_scratch:
        need = L.paro_channel_stats_scratch_bytes(B, H, N, D)
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
        args += [scratch.data_ptr(), need]
    rc = getattr(L, fn_name)(*args, _lib.stream_ptr())
    assert rc == 0, L.paro_last_error().decode()
    torch.cuda.synchronize()
    return out, out32


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    g = torch.Generator().manual_seed(123)
    first = (torch.randn(2, 6, 5000, 128, generator=g) * 3 + 1).to(torch.bfloat16).cuda()
    second = (torch.randn(1, 3, 700, 64, generator=g) - 2).to(torch.float16).cuda()   # smaller: stale partials remain
    for x in (first, second, first):
        want, want32 = _mean("paro_channel_mean", x, True)
        got, got32 = _mean("paro_channel_mean_noalloc", x, False)
        assert torch.equal(got, want) and torch.equal(got32, want32)
        assert torch.equal(got32, (x.double().sum(2) / x.shape[2]).float())


def test_noalloc_strided_input_and_limit():
    L = _lib.lib()
    x = torch.randn(1, 300, 4, 64, device="cuda").to(torch.float16)            # [B,N,H,D] storage
    xv = x.transpose(1, 2)                                                      # HND view with strides
    want, _ = _mean("paro_channel_mean", xv, True)
    got, _ = _mean("paro_channel_mean_noalloc", xv, False)
    assert torch.equal(got, want)
    # beyond the built-in scratch: refused with a clear message, nothing launched
    before = L.paro_launch_count()
    rc = L.paro_channel_mean_noalloc(x.data_ptr(), _lib.F16, 64, 64, 1 << 20, 128, 0, 0, 128, x.data_ptr(), None,
                                     _lib.stream_ptr())
    assert rc == _lib.PARO_ECAP and b"built-in scratch" in L.paro_last_error()
    assert L.paro_launch_count() == before
