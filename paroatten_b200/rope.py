"""Fused 3D-RoPE + per-head token permutation (replaces paroattention._rope.rope_permutation,
csrc/rope/rope.cu:14-48, and the torch loops permute_qk / permute_attn_out of
paroattention/cogvideox.py:22-110)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib


class RopeTables:
    """Per-axis angle tables: row = axis base + coordinate, column = channel pair.  Built from cos and sin
    tables [F+H+W, D/2] and handed to the kernels as ONE table [F+H+W, D/2, 2] with cos and sin of a pair side
    by side (a single load fetches both): `.cos` is that table, `.sin` is None."""

    def __init__(self, mode: int, cos: torch.Tensor, sin: torch.Tensor, pairs_f: int, pairs_h: int):
        self.mode = mode            # _lib.ROPE_REAL_F32 or _lib.ROPE_COMPLEX_F64
        self.cos = torch.stack([cos, sin], dim=-1).contiguous()
        self.sin = None
        self.pairs_f, self.pairs_h = pairs_f, pairs_h


@dataclass
class QKNorm:
    """The normalisation the processors apply to Q or K between the projection and RoPE
    (paroattention/cogvideox.py:161-164, wan.py:150-153), folded into the pre-attention passes.
    kind "layer": LayerNorm over the head dimension, weight/bias [D];
    kind "rms":   RMSNorm over all heads' channels of a token, weight [H*D], no bias.
    Parameters are cast to the activations' dtype when used."""
    kind: str
    weight: torch.Tensor
    bias: Optional[torch.Tensor] = None
    eps: float = 1e-6

    @classmethod
    def from_module(cls, mod, heads: int, head_dim: int) -> Optional["QKNorm"]:
        """QKNorm for a torch.nn.LayerNorm over head_dim or an RMS-norm module over heads*head_dim
        (anything with a 1-D `weight` of that size, an `eps` and no bias); None if `mod` is neither."""
        w = getattr(mod, "weight", None)
        eps = getattr(mod, "eps", None)
        if w is None or eps is None or w.dim() != 1:
            return None
        if isinstance(mod, torch.nn.LayerNorm) and w.numel() == head_dim:
            return cls("layer", w.detach(), None if mod.bias is None else mod.bias.detach(), float(eps))
        if "rms" in type(mod).__name__.lower() and w.numel() == heads * head_dim and getattr(mod, "bias", None) is None:
            return cls("rms", w.detach(), None, float(eps))
        return None


def _norm_call_args(norm: Optional[QKNorm], xv: torch.Tensor):
    """(mode, weight, bias, inv_rms, eps, keep-alive list) for an entry point that takes a norm;
    xv is the [B,H,N,D] view of the activations.  For "rms" the per-token statistic is computed here."""
    if norm is None:
        return _lib.NORM_NONE, None, None, None, 0.0, []
    B, H, N, D = xv.shape
    w = norm.weight.to(device=xv.device, dtype=xv.dtype).contiguous()
    if norm.kind == "layer":
        if w.numel() != D:
            raise ValueError("layer norm weight must have head_dim entries")
        b = None if norm.bias is None else norm.bias.to(device=xv.device, dtype=xv.dtype).contiguous()
        return _lib.NORM_LAYER_HEAD, w, b, None, float(norm.eps), [w, b]
    if norm.kind == "rms":
        if w.numel() != H * D:
            raise ValueError("rms norm weight must have heads*head_dim entries")
        inv = torch.empty(B, N, dtype=torch.float32, device=xv.device)
        _lib.check(_lib.lib().paro_row_inv_rms(
            xv.data_ptr(), _lib.dtype_code(xv.dtype), B, H, N, D, xv.stride(0), xv.stride(1), xv.stride(2),
            float(norm.eps), inv.data_ptr(), _lib.stream_ptr()))
        return _lib.NORM_RMS_ALL, w, None, inv, float(norm.eps), [w, inv]
    raise ValueError(f"unknown norm kind {norm.kind!r}")


def axis_pairs(head_dim: int, family: str) -> Tuple[int, int, int]:
    """Channel pairs rotated by the f / h / w coordinate: CogVideoX D/4, 3D/8, 3D/8 channels;
    Wan h = w = 2*(D//6) channels, the rest for f (paroattention/wan.py:492-493)."""
    if family == "cogvideox":
        t, h = head_dim // 4, head_dim // 8 * 3
        return t // 2, h // 2, h // 2
    if family == "wan":
        hw = 2 * (head_dim // 6)
        return (head_dim - 2 * hw) // 2, hw // 2, hw // 2
    raise ValueError(f"unknown rope family {family!r}")


def rope_tables(grid, head_dim: int, family: str, theta: float = 10000.0, device="cuda") -> RopeTables:
    """Angle of pair i of an axis with n pairs at coordinate p: p * theta^(-i/n).
    fp32 tables and fp32 rotation for "cogvideox" (diffusers' real-valued apply_rotary_emb,
    call site paroattention/cogvideox.py:167-172); fp64 for "wan" (wan.py:161-164,497-500)."""
    F, H, W = (int(g) for g in grid)
    pairs = axis_pairs(head_dim, family)
    dt = torch.float32 if family == "cogvideox" else torch.float64
    cos = torch.ones(F + H + W, head_dim // 2, dtype=dt)
    sin = torch.zeros(F + H + W, head_dim // 2, dtype=dt)
    row0 = col0 = 0
    for n_pos, n_pair in zip((F, H, W), pairs):
        dim = 2 * n_pair
        freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=dt)[:n_pair] / dim))
        ang = torch.outer(torch.arange(n_pos, dtype=dt), freqs)
        cos[row0:row0 + n_pos, col0:col0 + n_pair] = ang.cos()
        sin[row0:row0 + n_pos, col0:col0 + n_pair] = ang.sin()
        row0 += n_pos
        col0 += n_pair
    mode = _lib.ROPE_REAL_F32 if family == "cogvideox" else _lib.ROPE_COMPLEX_F64
    return RopeTables(mode, cos.to(device).contiguous(), sin.to(device).contiguous(), pairs[0], pairs[1])


def tables_from_embedding(emb, grid, head_dim: int, family: str, device=None) -> RopeTables:
    """Per-axis tables taken from the rotary embedding a pipeline hands to the processor, so that the
    processor rotates by exactly the angles it was given (another theta, a cropped or rescaled grid):
      "cogvideox": emb = (cos, sin), each [F*H*W, D] fp32 with every angle repeated for its channel pair
                   (diffusers' real layout; paroattention/cogvideox.py:167-172 passes it on unchanged);
      "wan":       emb = complex128 [1, 1, F*H*W, D/2] (WanRotaryPosEmbed, paroattention/wan.py:482-522).
    A 3-D table depends on one coordinate per channel pair, so the rows of tokens (f,0,0), (0,y,0), (0,0,x)
    hold everything; the result is checked by rebuilding the full table from the per-axis rows and
    comparing it with `emb` exactly -- ValueError if the embedding is not of that separable form."""
    F, Hh, W = (int(g) for g in grid)
    n_img, half = F * Hh * W, head_dim // 2
    if family == "cogvideox":
        cos_full, sin_full = (t.reshape(n_img, head_dim)[:, 0::2].to(torch.float32) for t in emb)
        mode = _lib.ROPE_REAL_F32
    elif family == "wan":
        e = emb.reshape(n_img, half)
        cos_full, sin_full = e.real.to(torch.float64), e.imag.to(torch.float64)
        mode = _lib.ROPE_COMPLEX_F64
    else:
        raise ValueError(f"unknown rope family {family!r}")
    device = cos_full.device if device is None else torch.device(device)
    cos_full, sin_full = cos_full.to(device), sin_full.to(device)
    pf, ph, pw = axis_pairs(head_dim, family)
    rows = (torch.arange(F, device=device) * (Hh * W), torch.arange(Hh, device=device) * W, torch.arange(W, device=device))
    cols = ((0, pf), (pf, pf + ph), (pf + ph, half))
    cos = torch.ones(F + Hh + W, half, dtype=cos_full.dtype, device=device)
    sin = torch.zeros(F + Hh + W, half, dtype=cos_full.dtype, device=device)
    r0 = 0
    for idx, (c0, c1) in zip(rows, cols):
        cos[r0:r0 + idx.numel(), c0:c1] = cos_full[idx, c0:c1]
        sin[r0:r0 + idx.numel(), c0:c1] = sin_full[idx, c0:c1]
        r0 += idx.numel()
    # rebuild and compare
    n = torch.arange(n_img, device=device)
    f, y, x = n // (Hh * W), (n // W) % Hh, n % W
    for full, tab in ((cos_full, cos), (sin_full, sin)):
        back = torch.cat([tab[f, 0:pf], tab[F + y, pf:pf + ph], tab[F + Hh + x, pf + ph:half]], dim=1)
        if not torch.equal(back, full):
            raise ValueError(f"the rotary embedding is not a per-axis 3-D table over the grid {tuple(grid)} with "
                             f"{pf}/{ph}/{pw} channel pairs per axis; set processor.grid_fhw to the latent grid")
    return RopeTables(mode, cos.contiguous(), sin.contiguous(), pf, ph)


def rope_permute(x: torch.Tensor, order_ids: Optional[torch.Tensor], grid, n_text: int = 0,
                 rope: Optional[RopeTables] = None, inverse: bool = False,
                 tensor_layout: str = "HND", norm: Optional[QKNorm] = None) -> torch.Tensor:
    """One pass over x ([B,H,N,D], or [B,N,H,D] when tensor_layout="NHD"): optional normalisation
    of every token (`norm`), optional RoPE on the video tokens, then head h's tokens gathered in its
    axis order (`order_ids` int32 [H] on the GPU; None = keep the order).  inverse=True undoes the
    permutation (no RoPE, no norm).  Returns a new contiguous [B,H,N,D] tensor."""
    _lib.require_cuda(x, order_ids)
    if tensor_layout == "NHD":
        x = x.transpose(1, 2)
    elif tensor_layout != "HND":
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    B, H, N, D = x.shape
    if x.stride(-1) != 1:
        x = x.contiguous()
    F, Hh, W = (int(g) for g in grid)
    if order_ids is not None:
        order_ids = order_ids.to(device=x.device, dtype=torch.int32).contiguous()
        if order_ids.numel() != H:
            raise ValueError("order_ids must hold one id per head")
    with torch.cuda.device(x.device):
        out = torch.empty(B, H, N, D, dtype=x.dtype, device=x.device)
        r = rope
        if norm is not None:
            if inverse:
                raise ValueError("the inverse permutation does not normalise")
            mode, w, b, inv, eps, _keep = _norm_call_args(norm, x)
            _lib.check(_lib.lib().paro_rope_permute_norm(
                x.data_ptr(), out.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, x.stride(0), x.stride(1), x.stride(2),
                int(n_text), F, Hh, W, _lib.ptr(order_ids), r.mode if r is not None else _lib.ROPE_NONE,
                _lib.ptr(r.cos if r else None), _lib.ptr(r.sin if r else None), r.pairs_f if r else 0,
                r.pairs_h if r else 0, mode, _lib.ptr(w), _lib.ptr(b), _lib.ptr(inv), eps, _lib.stream_ptr()))
            return out
        _lib.check(_lib.lib().paro_rope_permute(
            x.data_ptr(), out.data_ptr(), _lib.dtype_code(x.dtype), B, H, N, D, x.stride(0), x.stride(1), x.stride(2),
            int(n_text), F, Hh, W, _lib.ptr(order_ids), int(bool(inverse)),
            r.mode if r is not None else _lib.ROPE_NONE, _lib.ptr(r.cos if r else None),
            _lib.ptr(r.sin if r else None), r.pairs_f if r else 0, r.pairs_h if r else 0, _lib.stream_ptr()))
    return out


def rope_permutation(Q: torch.Tensor, K: torch.Tensor, freq, permutation: bool, *, order_ids=None, grid=None,
                     n_text: int = 0):
    """Same call shape as the reference op `_rope.rope_permutation(Q, K, freq, permutation) ->
    (QO, KO)` (csrc/rope/rope.h:6).  `freq` is a RopeTables (the reference's position-independent
    128-float table, rope.cuh:36-39, is a placeholder and has no meaning here).  Q, K are
    [B,H,N,D]; with permutation=True each head is reordered by `order_ids` (default: id 1, the
    H<->W swap the reference op performs, rope.cuh:41-50) over `grid` (default (1, H, W) is not
    inferable from a flat token axis, so grid is required)."""
    if grid is None:
        raise ValueError("grid=(F,H,W) is required")
    H = Q.shape[1]
    ids = None
    if permutation:
        ids = order_ids if order_ids is not None else torch.full((H,), 1, dtype=torch.int32, device=Q.device)
    return (rope_permute(Q, ids, grid, n_text, freq), rope_permute(K, ids, grid, n_text, freq))
