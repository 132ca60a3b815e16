"""INT8 / FP8 quantisers with the reference's Python signatures (paroattention/quant.py)."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

_scratch = {}


def _hnd(x: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    if tensor_layout == "HND":
        v = x
    elif tensor_layout == "NHD":
        v = x.transpose(1, 2)
    else:
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    return v if v.stride(-1) == 1 else v.contiguous()


def _stats_scratch(B, H, N, D, device) -> torch.Tensor:
    need = _lib.lib().paro_channel_stats_scratch_bytes(B, H, N, D)
    # one buffer per device AND stream: two streams reducing at once must not share partial sums
    key = (device.index if device.index is not None else torch.cuda.current_device(), _lib.stream_ptr())
    buf = _scratch.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def channel_mean(x: torch.Tensor, tensor_layout: str = "HND", out_dtype=None) -> torch.Tensor:
    """Mean over tokens -> [B,H,D] (the `km` argument of per_block_int8 / per_warp_int8);
    deterministic fp64 accumulation.  out_dtype: x.dtype (default) or torch.float32."""
    _lib.require_cuda(x)
    xv = _hnd(x, tensor_layout)
    B, H, N, D = xv.shape
    f32 = out_dtype == torch.float32
    with torch.cuda.device(x.device):
        out = torch.empty(B, H, D, dtype=torch.float32 if f32 else x.dtype, device=x.device)
        scr = _stats_scratch(B, H, N, D, x.device)
        _lib.check(_lib.lib().paro_channel_mean(
            xv.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, xv.stride(0), xv.stride(1), xv.stride(2),
            0 if f32 else out.data_ptr(), out.data_ptr() if f32 else 0, scr.data_ptr(), scr.numel(),
            _lib.stream_ptr()))
    return out


def _quant_int8(x, tensor_layout, group, km=None, fold=0.0):
    _lib.require_cuda(x, km)
    xv = _hnd(x, tensor_layout)
    B, H, N, D = xv.shape
    nb = (N + 63) // 64
    with torch.cuda.device(x.device):
        out = torch.empty(B, H, N, D, dtype=torch.int8, device=x.device)
        scale = torch.empty(B, H, nb * (64 // group), dtype=torch.float32, device=x.device)
        if km is not None:
            km = km.reshape(B, H, D).to(x.dtype).contiguous()
        _lib.check(_lib.lib().paro_quant_int8(
            xv.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, xv.stride(0), xv.stride(1), xv.stride(2),
            _lib.ptr(km), float(fold), group, out.data_ptr(), scale.data_ptr(), _lib.stream_ptr()))
    if tensor_layout == "NHD":
        out = out.transpose(1, 2)  # logical [B,N,H,D] view of the HND buffer
    return out, scale


def _quant_int8_blocks_of(x, tensor_layout, block, km=None, fold=0.0):
    """Per-`block`-token INT8 for block sizes the CUDA pass does not take (the reference's default
    BLKQ = 128), with torch elementwise ops and the same arithmetic (fused.cu:95-197): a compatibility
    route for callers of the quantisers alone -- the attention path of this library always uses 64-token
    blocks, the sparse plan's granularity.  Returns (int8 like x, fp32 scale [B,H,ceil(N/block)])."""
    _lib.require_cuda(x, km)
    xv = _hnd(x, tensor_layout)
    B, H, N, D = xv.shape
    xf = xv.float()
    if km is not None:
        xf = xf - km.reshape(B, H, 1, D).to(x.dtype).float()
    if fold:
        xf = xf * torch.tensor(fold, dtype=torch.float32, device=x.device)
    nblk = (N + block - 1) // block
    pad = nblk * block - N
    if pad:
        xf = torch.nn.functional.pad(xf, (0, 0, 0, pad))
    g = xf.reshape(B, H, nblk, block * D)
    amax = g.abs().amax(dim=-1).clamp_min(1e-7)
    scale = torch.div(amax, torch.full_like(amax, 127.0))    # (a tensor / scalar division multiplies by the reciprocal)
    inv = torch.div(torch.full_like(amax, 127.0), amax)     # one IEEE division (scalar / tensor would be reciprocal * scalar)
    q8 = torch.round(g * inv.unsqueeze(-1)).clamp_(-128, 127).to(torch.int8)
    q8 = q8.reshape(B, H, nblk * block, D)[:, :, :N].contiguous()
    return (q8.transpose(1, 2) if tensor_layout == "NHD" else q8), scale.contiguous()


def per_block_int8(q, k, km: Optional[torch.Tensor] = None, BLKQ: int = 128, BLKK: int = 64,
                   sm_scale: Optional[float] = None, tensor_layout: str = "HND"):
    """Reference signature and defaults of paroattention/quant.py:22-103: Q per block of BLKQ tokens with
    sm_scale*log2(e) folded in, K per block of BLKK tokens (optionally mean-smoothed).  64-token blocks
    run in the CUDA quantiser; 128-token blocks (the reference's default BLKQ) take the torch route of
    _quant_int8_blocks_of.  The attention entry points of this library quantise with 64-token blocks."""
    if BLKQ not in (64, 128) or BLKK not in (64, 128):
        raise ValueError("per_block_int8: BLKQ and BLKK must be 64 or 128")
    D = q.shape[-1]
    if sm_scale is None:
        sm_scale = D ** -0.5
    fold = sm_scale * 1.44269504
    q8, qs = (_quant_int8(q, tensor_layout, 64, fold=fold) if BLKQ == 64
              else _quant_int8_blocks_of(q, tensor_layout, BLKQ, fold=fold))
    k8, ks = (_quant_int8(k, tensor_layout, 64, km=km) if BLKK == 64
              else _quant_int8_blocks_of(k, tensor_layout, BLKK, km=km))
    return q8, qs, k8, ks


def per_warp_int8(q, k, km: Optional[torch.Tensor] = None, BLKQ: int = 128, WARPQ: int = 32, BLKK: int = 64,
                  tensor_layout: str = "HND"):
    """Reference signature and defaults of paroattention/quant.py:105-180: Q per WARPQ = 32 rows, K per
    block of BLKK tokens (optionally mean-smoothed).  BLKQ only sets how far the Q scale array is padded:
    (ceil(N/BLKQ) * BLKQ/32) entries, the trailing ones belonging to groups past the end of the sequence
    (quant.py:169).  The processors call it with BLKQ=64, WARPQ=32, BLKK=64 (cogvideox.py:186); that is also
    the layout the attention kernel reads.  WARPQ = 16 is not supported."""
    if BLKQ not in (64, 128) or WARPQ != 32 or BLKK not in (64, 128):
        raise ValueError("per_warp_int8: BLKQ and BLKK must be 64 or 128, WARPQ must be 32")
    q8, qs = _quant_int8(q, tensor_layout, 32)
    if BLKQ == 128:
        n = q.shape[2] if tensor_layout == "HND" else q.shape[1]
        want = (n + 127) // 128 * 4
        if want != qs.shape[-1]:       # two more 32-row groups of padding: all zeros, amax floor 1e-7
            qs = torch.cat([qs, torch.full((*qs.shape[:-1], want - qs.shape[-1]), 1e-7 / 127.0,
                                           dtype=qs.dtype, device=qs.device)], dim=-1)
    k8, ks = (_quant_int8(k, tensor_layout, 64, km=km) if BLKK == 64
              else _quant_int8_blocks_of(k, tensor_layout, BLKK, km=km))
    return q8, qs, k8, ks


def sub_mean(v: torch.Tensor, tensor_layout: str = "HND"):
    """Reference signature paroattention/quant.py:182-222: (v - mean over tokens) as fp16 and
    the mean in v.dtype.  The mean comes from the deterministic reduction kernel; the
    subtraction is one elementwise torch op (this helper is not on the attention path here:
    V smoothing is part of per_channel_fp8)."""
    vm = channel_mean(v, tensor_layout)
    expand = vm.unsqueeze(2) if tensor_layout == "HND" else vm.unsqueeze(1)
    return (v.float() - expand.float()).to(torch.float16), vm


def per_channel_fp8(v: torch.Tensor, tensor_layout: str = "HND", scale_max: float = 448.0, smooth_v: bool = True,
                    return_16: bool = False):
    """Reference signature paroattention/quant.py:224-293: V transposed to token-contiguous
    [B,H,D,ceil64(N)] float8_e4m3fn (zero padded; no 16-token shuffle), per-channel scale
    [B,H,D] and mean [B,H,D] (None without smoothing).  return_16=True appends the same values
    widened to bf16 (exact), which is what the attention kernel consumes."""
    _lib.require_cuda(v)
    vv = _hnd(v, tensor_layout)
    B, H, N, D = vv.shape
    npad = (N + 63) // 64 * 64
    with torch.cuda.device(v.device):
        v8 = torch.empty(B, H, D, npad, dtype=torch.float8_e4m3fn, device=v.device)
        v16 = torch.empty(B, H, D, npad, dtype=torch.bfloat16, device=v.device) if return_16 else None
        scale = torch.empty(B, H, D, dtype=torch.float32, device=v.device)
        vm = torch.empty(B, H, D, dtype=torch.float32, device=v.device) if smooth_v else None
        scr = _stats_scratch(B, H, N, D, v.device)
        _lib.check(_lib.lib().paro_quant_v_fp8(
            vv.data_ptr(), _lib.dtype_code(v.dtype), B, H, N, D, vv.stride(0), vv.stride(1), vv.stride(2),
            int(bool(smooth_v)), float(scale_max), v8.data_ptr(), _lib.ptr(v16), scale.data_ptr(), _lib.ptr(vm),
            scr.data_ptr(), scr.numel(), _lib.stream_ptr()))
    if tensor_layout == "NHD":
        v8 = v8.transpose(1, 2)  # [B,D,H,Npad] view, the reference's NHD output shape
    return (v8, scale, vm, v16) if return_16 else (v8, scale, vm)


def prep_qk_int8(x: torch.Tensor, order_ids: Optional[torch.Tensor], grid, n_text: int = 0, rope=None, group: int = 32,
                 smooth: bool = False, tensor_layout: str = "HND", norm=None):
    """[normalisation +] RoPE + per-head reordering + INT8 quantisation of Q (group=32) or K (group=64,
    smooth=True for mean smoothing) straight from the natural-order tensor: no reordered 16-bit copy
    is written.  Returns (int8 [B,H,N,D], scale, km or None), equal bit for bit to
    per_warp_int8(rope_permute(x, ...)).  `norm` (a rope.QKNorm) cannot be combined with smooth."""
    _lib.require_cuda(x, order_ids)
    xv = _hnd(x, tensor_layout)
    B, H, N, D = xv.shape
    nb = (N + 63) // 64
    F, Hh, W = (int(g) for g in grid)
    with torch.cuda.device(x.device):
        if order_ids is not None:
            order_ids = order_ids.to(device=x.device, dtype=torch.int32).contiguous()
        out = torch.empty(B, H, N, D, dtype=torch.int8, device=x.device)
        scale = torch.empty(B, H, nb * (64 // group), dtype=torch.float32, device=x.device)
        km = torch.empty(B, H, D, dtype=x.dtype, device=x.device) if smooth else None
        scr = _stats_scratch(B, H, N, D, x.device) if smooth else None
        r = rope
        if norm is not None:
            if smooth:
                raise ValueError("prep_qk_int8: norm and smooth cannot be combined (use rope_permute(norm=...) first)")
            from .rope import _norm_call_args
            mode, w, b, inv, eps, _keep = _norm_call_args(norm, xv)
            _lib.check(_lib.lib().paro_prep_qk_int8_norm(
                xv.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, xv.stride(0), xv.stride(1), xv.stride(2),
                int(n_text), F, Hh, W, _lib.ptr(order_ids), r.mode if r is not None else _lib.ROPE_NONE,
                _lib.ptr(r.cos if r else None), _lib.ptr(r.sin if r else None), r.pairs_f if r else 0,
                r.pairs_h if r else 0, int(group), out.data_ptr(), scale.data_ptr(),
                mode, _lib.ptr(w), _lib.ptr(b), _lib.ptr(inv), eps, _lib.stream_ptr()))
            return out, scale, None
        _lib.check(_lib.lib().paro_prep_qk_int8(
            xv.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, xv.stride(0), xv.stride(1), xv.stride(2),
            int(n_text), F, Hh, W, _lib.ptr(order_ids), r.mode if r is not None else _lib.ROPE_NONE,
            _lib.ptr(r.cos if r else None), _lib.ptr(r.sin if r else None), r.pairs_f if r else 0,
            r.pairs_h if r else 0, int(group), int(bool(smooth)), _lib.ptr(km), out.data_ptr(), scale.data_ptr(),
            _lib.ptr(scr), scr.numel() if scr is not None else 0, _lib.stream_ptr()))
    return out, scale, km


def prep_v_fp8(v: torch.Tensor, order_ids: Optional[torch.Tensor], grid, n_text: int = 0, smooth_v: bool = True,
               scale_max: float = 448.0, tensor_layout: str = "HND", want_fp8: bool = False):
    """Per-head reordering + per-channel FP8 quantisation of V from the natural-order tensor.
    Returns (v16: bf16 [B,H,D,ceil64(N)] holding the e4m3 values, v_scale, vm, v_fp8 or None), equal
    bit for bit to per_channel_fp8(rope_permute(v, ...), return_16=True)."""
    _lib.require_cuda(v, order_ids)
    vv = _hnd(v, tensor_layout)
    B, H, N, D = vv.shape
    npad = (N + 63) // 64 * 64
    F, Hh, W = (int(g) for g in grid)
    with torch.cuda.device(v.device):
        if order_ids is not None:
            order_ids = order_ids.to(device=v.device, dtype=torch.int32).contiguous()
        v16 = torch.empty(B, H, D, npad, dtype=torch.bfloat16, device=v.device)
        v8 = torch.empty(B, H, D, npad, dtype=torch.float8_e4m3fn, device=v.device) if want_fp8 else None
        scale = torch.empty(B, H, D, dtype=torch.float32, device=v.device)
        vm = torch.empty(B, H, D, dtype=torch.float32, device=v.device) if smooth_v else None
        scr = _stats_scratch(B, H, N, D, v.device)
        _lib.check(_lib.lib().paro_prep_v_fp8(
            vv.data_ptr(), _lib.dtype_code(v.dtype), B, H, N, D, vv.stride(0), vv.stride(1), vv.stride(2),
            int(n_text), F, Hh, W, _lib.ptr(order_ids), int(bool(smooth_v)), float(scale_max), _lib.ptr(v8),
            v16.data_ptr(), scale.data_ptr(), _lib.ptr(vm), scr.data_ptr(), scr.numel(), _lib.stream_ptr()))
    return v16, scale, vm, v8
