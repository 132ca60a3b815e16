"""The C-ABI library builds, loads and exports every symbol the header declares (no GPU)."""
import ctypes
import os
import re

import pytest

from paroatten_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "paro_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(paro_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    handle = _lib.lib()
    names = declared_symbols()
    assert "paro_sparse_attn" in names and len(names) >= 12
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/paro_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of sync with the header"


def test_version_and_argument_errors_without_gpu():
    handle = _lib.lib()
    assert handle.paro_version() == 100
    # argument validation happens before any CUDA call, so it can be exercised on a CPU box
    rc = handle.paro_quant_int8(None, 0, 1, 1, 64, 64, 0, 0, 64, None, 0.0, 32, None, None, None)
    assert rc == _lib.PARO_EINVAL and b"null" in handle.paro_last_error()
    buf = ctypes.create_string_buffer(64 * 96 * 2 + 64)
    addr = (ctypes.addressof(buf) + 15) & ~15
    rc = handle.paro_quant_int8(addr, 0, 1, 1, 64, 96, 0, 0, 96, None, 0.0, 32, addr, addr, None)
    assert rc == _lib.PARO_ESHAPE and b"head_dim" in handle.paro_last_error()
    rc = handle.paro_quant_int8(addr, 0, 1, 1, 64, 64, 0, 0, 64, None, 0.0, 48, addr, addr, None)
    assert rc == _lib.PARO_EINVAL and b"group" in handle.paro_last_error()
    rc = handle.paro_rope_permute(addr, addr + 16, 1, 1, 1, 10, 64, 0, 0, 64, 0, 1, 2, 3, None, 0, 0, None, None, 0, 0, None)
    assert rc == _lib.PARO_ESHAPE and b"!= N" in handle.paro_last_error()
    rc = handle.paro_plan_schedule(addr, addr, 1, 4, 70000, addr, addr, None)
    assert rc == _lib.PARO_ESHAPE and b"16 bits" in handle.paro_last_error()
    rc = handle.paro_rope_permute_norm(addr, addr + 16, 1, 1, 1, 6, 64, 0, 0, 64, 0, 1, 2, 3, None, 0, None, None, 0, 0,
                                       7, None, None, None, 1e-6, None)
    assert rc == _lib.PARO_EINVAL and b"norm_mode" in handle.paro_last_error()
    rc = handle.paro_rope_permute_norm(addr, addr + 16, 1, 1, 1, 6, 64, 0, 0, 64, 0, 1, 2, 3, None, 0, None, None, 0, 0,
                                       2, addr, None, None, 1e-6, None)
    assert rc == _lib.PARO_EINVAL and b"inv_rms" in handle.paro_last_error()
    assert handle.paro_channel_stats_scratch_bytes(1, 2, 1000, 128) == 2 * 2 * 128 * 16 + 2 * 2 * 128 * 4
    with pytest.raises(ValueError):
        _lib.check(rc)


def test_ops_refuse_cpu_tensors():
    import torch
    import paroatten_b200 as pb
    x = torch.zeros(1, 1, 64, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pb.per_warp_int8(x, x, BLKQ=64, WARPQ=32, BLKK=64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pb.compact_plan(torch.ones(1, 2, 2, dtype=torch.bool))
