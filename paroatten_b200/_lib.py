"""Loader (and in-tree builder) of libparo_b200.so, the C-ABI CUDA library.

There is no fallback: if the library cannot be built or loaded, every operator of this
package raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libparo_b200.so")
SOURCES = ("common.cu", "perm_plan.cu", "rope_permute.cu", "quant.cu", "sparse_attn.cu", "attn_aux.cu")
NVCC_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared")

PARO_OK, PARO_EINVAL, PARO_ESHAPE, PARO_EALIGN, PARO_ETIMEOUT, PARO_ECUDA, PARO_ECAP = 0, -1, -2, -3, -4, -5, -6
F16, BF16 = 0, 1
ROPE_NONE, ROPE_REAL_F32, ROPE_COMPLEX_F64 = 0, 1, 2
NORM_NONE, NORM_LAYER_HEAD, NORM_RMS_ALL = 0, 1, 2
ATTN_FAST, ATTN_EXACT = 0, 1

_lock = threading.Lock()
_lib = None


def _nvcc():
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


HASH_PATH = LIB_PATH + ".srchash"


def _source_hash() -> str:
    """Digest of everything the library is built from (file times do not survive copying a tree)."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    files = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)) + [os.path.join(HERE, "..", "include", "paro_b200.h")]
    for f in files:
        with open(f, "rb") as fh:
            h.update(os.path.basename(f).encode() + b"\0" + fh.read())
    return h.hexdigest()


def _stale() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(HASH_PATH)):
        return True
    with open(HASH_PATH) as fh:
        return fh.read().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/*.cu for sm_100a into libparo_b200.so next to this file.  Safe against
    several processes building at once (each writes its own temporary file, renames are atomic)."""
    with _lock:
        if not force and not _stale():
            return LIB_PATH
        nvcc = _nvcc()
        if nvcc is None:
            raise RuntimeError("libparo_b200.so is missing or out of date and nvcc was not found to build it")
        tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []),
               *[os.path.join(CSRC, s) for s in SOURCES], "-o", tmp]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        os.replace(tmp, LIB_PATH)
        with open(f"{HASH_PATH}.{os.getpid()}.tmp", "w") as fh:
            fh.write(_source_hash())
        os.replace(f"{HASH_PATH}.{os.getpid()}.tmp", HASH_PATH)
        if verbose:
            print(res.stderr)
        return LIB_PATH


_i32, _i64, _f32, _vp, _sz = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

SIGNATURES = {
    "paro_version": (ctypes.c_int, []),
    "paro_last_error": (ctypes.c_char_p, []),
    "paro_launch_count": (ctypes.c_longlong, []),
    "paro_build_perm_index": (_i32, [_vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "paro_rope_permute": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32,
                                 _vp, _i32, _i32, _vp, _vp, _i32, _i32, _vp]),
    "paro_channel_stats_scratch_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "paro_channel_mean": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    "paro_channel_mean_noalloc": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _vp, _vp]),
    "paro_quant_int8": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _f32, _i32, _vp, _vp, _vp]),
    "paro_quant_v_fp8": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _f32, _vp, _vp, _vp, _vp,
                                _vp, _sz, _vp]),
    "paro_prep_qk_int8": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp,
                                 _i32, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _sz, _vp]),
    "paro_prep_v_fp8": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp,
                               _i32, _f32, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "paro_row_inv_rms": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _f32, _vp, _vp]),
    "paro_rope_permute_norm": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32,
                                      _vp, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _f32, _vp]),
    "paro_prep_qk_int8_norm": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp,
                                      _i32, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _f32, _vp]),
    "paro_plan_count": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "paro_plan_fill": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp, _i64, _vp, _vp, _i64, _vp]),
    "paro_plan_schedule": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "paro_sparse_attn_redo_bytes": (_sz, [_i32, _i32, _i32]),
    "paro_sparse_attn": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i32, _vp, _i32,
                                _i64, _i64, _i64, _vp, _i32, _i32, _i32, _i32, _f32, _i32, _vp, _sz, _vp, _vp]),
    "paro_status_poll": (_i32, [_vp, _vp, _vp]),
    "paro_plan_validate": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _vp, _vp]),
    "paro_merge_attn_states": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _vp]),
}


def lib() -> ctypes.CDLL:
    """The loaded library; builds it first when the sources are newer and nvcc is present."""
    global _lib
    if _lib is None:
        if _stale():
            build()
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = a symbol of the header is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


class ParoError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libparo_b200 error {code}: {message}")
        self.code = code


def check(rc: int) -> None:
    """Raises like the reference's extensions do: ValueError for rejected arguments
    (csrc/dispatch_utils.h:30-33), RuntimeError otherwise (csrc/utils.cuh:20-37)."""
    if rc == PARO_OK:
        return
    msg = lib().paro_last_error().decode()
    if rc in (PARO_EINVAL, PARO_ESHAPE, PARO_EALIGN, PARO_ECAP):
        raise ValueError(f"libparo_b200 error {rc}: {msg}")
    raise ParoError(rc, msg)


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("paroatten_b200 operators run on CUDA tensors only; there is no CPU path")


def dtype_code(dt) -> int:
    import torch
    if dt == torch.float16:
        return F16
    if dt == torch.bfloat16:
        return BF16
    raise ValueError(f"unsupported dtype {dt}: fp16 or bf16 expected")


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()
