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


def test_noalloc_capacity_edge_and_no_allocation():
    """At the limit of the built-in array (1,048,576 partial sums of 16 bytes) the call runs, one chunk of
    tokens more is refused; and a call takes no device memory: what the driver reports as free and what
    torch's allocator holds are the same before and after (after a first call, which is when the driver
    places the library's array).  Batch and head strides of 0 make a large problem out of one small tensor."""
    L = _lib.lib()
    D, B, H = 128, 64, 128                       # B*H*D = 1,048,576: exactly one 512-token chunk fits
    row = (torch.arange(D, dtype=torch.float32, device="cuda") / 8 - 3).to(torch.float16).reshape(1, D)
    rows = row.expand(513, D).contiguous()       # 513 equal tokens, shared by every (batch entry, head)
    out32 = torch.empty(B, H, D, dtype=torch.float32, device="cuda")

    def call(n_tokens):
        return L.paro_channel_mean_noalloc(rows.data_ptr(), _lib.F16, B, H, n_tokens, D, 0, 0, D, None, out32.data_ptr(),
                                           _lib.stream_ptr())
    assert call(512) == 0, L.paro_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(out32, row.float().reshape(1, 1, D).expand(B, H, D))     # the mean of equal rows is the row
    before = L.paro_launch_count()
    assert call(513) == _lib.PARO_ECAP and b"built-in scratch" in L.paro_last_error()
    assert L.paro_launch_count() == before
    # no device memory is taken by a call
    x = torch.randn(2, 4, 3000, 64, device="cuda").to(torch.bfloat16)
    out = torch.empty(2, 4, 64, dtype=torch.bfloat16, device="cuda")
    args = (x.data_ptr(), _lib.BF16, 2, 4, 3000, 64, x.stride(0), x.stride(1), x.stride(2), out.data_ptr(), None,
            _lib.stream_ptr())
    assert L.paro_channel_mean_noalloc(*args) == 0
    torch.cuda.synchronize()
    free0, held0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    for _ in range(3):
        assert L.paro_channel_mean_noalloc(*args) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == held0
