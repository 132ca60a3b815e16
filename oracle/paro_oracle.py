"""CPU restatement of PAROAttention's quantized block-sparse attention path.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA library is
compared against.  Nothing in the shipped package imports it; only the test
suite, the smoke check and the benchmark's CPU-baseline leg may call it.

Parity status: the token permutation and its inverse are pinned against the
reference's own Python (`paroattention/cogvideox.py:22-110`, run on CPU by
`tests/golden/make_golden.py`).  Everything else (RoPE, INT8/FP8 quantisers,
sparse attention) is "parity unpinned": the reference implements those only as
sm80 CUDA kernels with no stored expected values, so this file restates their
arithmetic from the sources cited on each function.

All arithmetic is IEEE fp32 (or fp64 where stated) on the host via torch CPU
ops; integer work uses exact integer ops.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

LOG2E = 1.44269504  # the constant the reference multiplies sm_scale by (quant.py:94, core.py:214)

# Axis orders of the (F, H, W) latent grid, by plan id.  cogvideox.py:38-45 / wan.py:40-47.
ORDERS = (
    (0, 1, 2),  # 0: FHW
    (0, 2, 1),  # 1: FWH
    (1, 2, 0),  # 2: HWF
    (1, 0, 2),  # 3: HFW
    (2, 1, 0),  # 4: WHF
    (2, 0, 1),  # 5: WFH
)


# --------------------------------------------------------------------------- permutation
def perm_index(order_id: int, grid: Tuple[int, int, int]) -> torch.Tensor:
    """idx[new] = old for one head: the flat gather index that
    `x.reshape(F,H,W,D).permute(order).reshape(-1,D)` performs on the video tokens
    (cogvideox.py:54, wan.py:54)."""
    F, H, W = grid
    base = torch.arange(F * H * W, dtype=torch.int64).reshape(F, H, W)
    return base.permute(*ORDERS[int(order_id)]).reshape(-1).to(torch.int32)


def perm_index_table(order_ids: Sequence[int], grid: Tuple[int, int, int]) -> torch.Tensor:
    """[H, F*H*W] int32 table, one row per head."""
    return torch.stack([perm_index(int(o), grid) for o in order_ids], dim=0)


def permute_tokens(x: torch.Tensor, order_ids: Sequence[int], grid, n_text: int = 0) -> torch.Tensor:
    """Forward permutation of [B,H,N,D]; text tokens stay (cogvideox.py:22-62)."""
    out = x.clone()
    for h, o in enumerate(order_ids):
        idx = perm_index(int(o), grid).long()
        out[:, h, n_text:, :] = x[:, h, n_text:, :][:, idx, :]
    return out


def inverse_permute_tokens(x: torch.Tensor, order_ids: Sequence[int], grid, n_text: int = 0) -> torch.Tensor:
    """Inverse of `permute_tokens` (cogvideox.py:64-110): out[idx[j]] = x[j]."""
    out = x.clone()
    for h, o in enumerate(order_ids):
        idx = perm_index(int(o), grid).long()
        tmp = torch.empty_like(x[:, h, n_text:, :])
        tmp[:, idx, :] = x[:, h, n_text:, :]
        out[:, h, n_text:, :] = tmp
    return out


# --------------------------------------------------------------------------- RoPE
def rope_axis_pairs(head_dim: int, family: str) -> Tuple[int, int, int]:
    """Number of rotated channel PAIRS driven by the f, h and w coordinate.
    CogVideoX: channels D/4, 3D/8, 3D/8 (diffusers 3-D table used at cogvideox.py:167-172).
    Wan: h_dim = w_dim = 2*(D//6), t_dim = the rest (wan.py:492-493)."""
    if family == "cogvideox":
        t, h = head_dim // 4, head_dim // 8 * 3
        return t // 2, h // 2, h // 2
    if family == "wan":
        hw = 2 * (head_dim // 6)
        return (head_dim - 2 * hw) // 2, hw // 2, hw // 2
    raise ValueError(family)


def rope_axis_tables(grid, head_dim: int, family: str, theta: float = 10000.0):
    """Per-axis (cos, sin) tables laid out [F+H+W, D/2]; row = axis base + coordinate,
    column = pair index.  Only the columns owned by the row's axis are meaningful
    (others hold cos=1, sin=0).  fp32 for cogvideox, fp64 for wan (wan.py:497-500)."""
    F, H, W = grid
    pairs = rope_axis_pairs(head_dim, family)
    dt = torch.float32 if family == "cogvideox" else torch.float64
    cos = torch.ones(F + H + W, head_dim // 2, dtype=dt)
    sin = torch.zeros(F + H + W, head_dim // 2, dtype=dt)
    row0, col0 = 0, 0
    for n_pos, n_pair in zip((F, H, W), pairs):
        dim = 2 * n_pair
        freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=dt)[:n_pair] / dim))
        ang = torch.outer(torch.arange(n_pos, dtype=dt), freqs)
        cos[row0:row0 + n_pos, col0:col0 + n_pair] = ang.cos()
        sin[row0:row0 + n_pos, col0:col0 + n_pair] = ang.sin()
        row0 += n_pos
        col0 += n_pair
    return cos, sin


def rope_full_tables(grid, head_dim: int, family: str, theta: float = 10000.0):
    """Per-token (cos, sin) [F*H*W, D/2] gathered from the axis tables."""
    F, H, W = grid
    cos_a, sin_a = rope_axis_tables(grid, head_dim, family, theta)
    pairs = rope_axis_pairs(head_dim, family)
    n = torch.arange(F * H * W)
    coord = (n // (H * W), (n // W) % H, n % W)
    base = (0, F, F + H)
    cos = torch.empty(F * H * W, head_dim // 2, dtype=cos_a.dtype)
    sin = torch.empty_like(cos)
    c0 = 0
    for ax in range(3):
        rows = base[ax] + coord[ax]
        cos[:, c0:c0 + pairs[ax]] = cos_a[rows, c0:c0 + pairs[ax]]
        sin[:, c0:c0 + pairs[ax]] = sin_a[rows, c0:c0 + pairs[ax]]
        c0 += pairs[ax]
    return cos, sin


def apply_rope_real(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_text: int = 0) -> torch.Tensor:
    """CogVideoX flavour (call site cogvideox.py:167-172; arithmetic of diffusers'
    apply_rotary_emb with interleaved pairs): on tokens >= n_text,
    out = x*cos + rot(x)*sin in fp32 with rot(x)[2i] = -x[2i+1], rot(x)[2i+1] = x[2i];
    each product and the sum rounded separately; result rounded to x.dtype."""
    out = x.clone()
    xv = x[:, :, n_text:, :].float()
    c = cos.float().repeat_interleave(2, dim=-1)
    s = sin.float().repeat_interleave(2, dim=-1)
    x0, x1 = xv[..., 0::2], xv[..., 1::2]
    rot = torch.stack([-x1, x0], dim=-1).flatten(-2)
    out[:, :, n_text:, :] = (xv * c + rot * s).to(x.dtype)
    return out


def apply_rope_complex(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_text: int = 0) -> torch.Tensor:
    """Wan flavour (wan.py:161-164): pairs as complex numbers times cos+i*sin in fp64,
    then cast to x.dtype (double -> float -> x.dtype, which is what torch's cast does)."""
    out = x.clone()
    xv = x[:, :, n_text:, :].to(torch.float64)
    x0, x1 = xv[..., 0::2], xv[..., 1::2]
    c, s = cos.double(), sin.double()
    re = x0 * c - x1 * s
    im = x0 * s + x1 * c
    out[:, :, n_text:, :] = torch.stack([re, im], dim=-1).flatten(-2).float().to(x.dtype)
    return out


# --------------------------------------------------------------------------- QK normalisation
# The processors normalise Q and K between the projection and RoPE (cogvideox.py:161-164,
# wan.py:150-153) with modules of the third-party `diffusers` package, which is not vendored in the
# reference and not pinned to a version: LayerNorm over the head dimension with affine parameters
# for CogVideoX, RMSNorm over all heads' channels ("rms_norm_across_heads", wan.py:531) for Wan.
# Parity unpinned: the arithmetic below is this project's definition (sums in fp64, every other
# operation a separately rounded IEEE fp32 operation, result rounded to the input dtype), not a
# transcript of that package.
def _sqrt_f32(t: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 square root.  torch's vectorised CPU sqrt is off by one unit in the last
    place for a fraction of a percent of inputs; the fp64 root rounded to fp32 is exact (53 >= 2*24+2)."""
    return torch.sqrt(t.double()).float()


def layer_norm_heads(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x [..., D] -> (x - mean) * rstd * weight + bias over the last dimension."""
    xd = x.double()
    D = x.shape[-1]
    mean = (xd.sum(-1, keepdim=True) / D).float()
    dev = xd - mean.double()
    var = ((dev * dev).sum(-1, keepdim=True) / D).float()
    rstd = 1.0 / _sqrt_f32(var + torch.tensor(eps, dtype=torch.float32))
    y = (x.float() - mean) * rstd
    y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def row_inv_rms(x_bnc: torch.Tensor, eps: float) -> torch.Tensor:
    """x [B, N, C] -> 1/sqrt(mean(x^2) + eps) per token, fp32 [B, N]."""
    xd = x_bnc.double()
    ms = ((xd * xd).sum(-1) / x_bnc.shape[-1]).float()
    return 1.0 / _sqrt_f32(ms + torch.tensor(eps, dtype=torch.float32))


def rms_norm_across_heads(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x [B, H, N, D], weight [H*D]: y = dtype(dtype(x * inv_rms[token]) * weight), the statistic taken
    over all H*D channels of a token."""
    B, H, N, D = x.shape
    inv = row_inv_rms(x.permute(0, 2, 1, 3).reshape(B, N, H * D), eps)          # [B, N]
    y = (x.float() * inv.reshape(B, 1, N, 1)).to(x.dtype)
    return (y.float() * weight.float().reshape(1, H, 1, D)).to(x.dtype)


def apply_qk_norm(x: torch.Tensor, norm) -> torch.Tensor:
    """norm = None | ("layer", weight [D], bias [D] or None, eps) | ("rms", weight [H*D], eps)."""
    if norm is None:
        return x
    if norm[0] == "layer":
        return layer_norm_heads(x, norm[1], norm[2], norm[3])
    if norm[0] == "rms":
        return rms_norm_across_heads(x, norm[1], norm[2])
    raise ValueError(f"unknown norm kind {norm[0]!r}")


# --------------------------------------------------------------------------- quantisers
def channel_mean(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Mean over tokens of [B,H,N,D] -> [B,H,D].  The reference takes `k.mean(dim=-2)` in the
    input dtype (quant.py:46-48) whose summation order is unspecified; here the sum is taken in
    fp64 (exact for 16-bit inputs of sane range), divided by N in fp64, rounded to fp32 and
    then to `out_dtype`."""
    m = x.double().sum(dim=2) / x.shape[2]
    return m.float().to(out_dtype)


def quant_int8(x: torch.Tensor, group: int, km: Optional[torch.Tensor] = None,
               fold_scale: Optional[float] = None):
    """Per-group symmetric INT8 of [B,H,N,D] (fused.cu:95-197).
    x = float(in) [- float(km)] [* fold_scale]; rows >= N count as 0;
    amax = max(1e-7, max|x|) over group*D values; scale = amax/127;
    q = sat_s8(round_half_even(x * (127/amax))).  Groups tile the sequence padded up to a
    multiple of max(64, group) tokens, so `group`=32 yields 2 scales per 64-token block (quant.py:169).
    Returns (int8 [B,H,N,D], fp32 scale [B,H,ceil(N/64)*(64/group)] (group <= 64) or [B,H,ceil(N/group)])."""
    B, H, N, D = x.shape
    xf = x.float()
    if km is not None:
        xf = xf - km.float().reshape(B, H, 1, D)
    if fold_scale is not None:
        xf = xf * torch.tensor(fold_scale, dtype=torch.float32)
    tile = max(64, group)
    npad = (N + tile - 1) // tile * tile
    if npad != N:
        xf = torch.cat([xf, torch.zeros(B, H, npad - N, D)], dim=2)
    g = xf.reshape(B, H, npad // group, group * D)
    amax = g.abs().amax(dim=-1).clamp_min(1e-7)
    scale = amax / torch.tensor(127.0)
    inv = torch.div(torch.full_like(amax, 127.0), amax)
    q = torch.round(g * inv.unsqueeze(-1)).clamp(-128, 127).to(torch.int8)
    q = q.reshape(B, H, npad, D)[:, :, :N, :].contiguous()
    return q, scale.contiguous()


def quant_v_fp8(v: torch.Tensor, smooth: bool = True, scale_max: float = 448.0, mean_divisor: Optional[int] = None):
    """Per-channel FP8-e4m3 of V, stored token-contiguous (fused.cu:316-427 with the
    transposed, 64-padded layout of fused.cu:262-313 minus its 16-token shuffle).
    vm = fp32(sum_fp64(v)/N) when smoothing (the reference divides by N rounded up to 16,
    fused.cu:335,381: the true N is used here); amax = max(1e-7, max|v - vm|);
    v_scale = amax/scale_max; v8 = e4m3_rn_satfinite((v - vm) * (scale_max/amax)).
    mean_divisor: only for comparisons with the reference kernel's own output -- its divisor (N rounded up
    to 16) instead of N.
    Returns (fp8 [B,H,D,ceil64(N)] zero padded, v_scale [B,H,D] fp32, vm [B,H,D] fp32 or None)."""
    B, H, N, D = v.shape
    vf = v.float()
    vm = None
    if smooth:
        vm = (v.double().sum(dim=2) / (N if mean_divisor is None else mean_divisor)).float()
        vf = vf - vm.reshape(B, H, 1, D)
    amax = vf.abs().amax(dim=2).clamp_min(1e-7)
    scale = amax / torch.tensor(scale_max)
    inv = torch.div(torch.full_like(amax, scale_max), amax)
    y = (vf * inv.reshape(B, H, 1, D)).clamp(-scale_max, scale_max)
    npad = (N + 63) // 64 * 64
    out = torch.zeros(B, H, D, npad, dtype=torch.float8_e4m3fn)
    out[:, :, :, :N] = y.transpose(2, 3).to(torch.float8_e4m3fn)
    return out, scale.contiguous(), vm


# --------------------------------------------------------------------------- plan compaction
def compact_plan(mask: torch.Tensor):
    """mask [..., nbq, nbk] bool -> CSR over rows in row-major order:
    row_ptr int32 [rows+1], cols int32 [nnz] ascending within a row (the blocks the
    reference kernel visits, qk_int_sv_f16_cuda_sm80.cu:222,268)."""
    m = mask.reshape(-1, mask.shape[-1]).bool()
    counts = m.sum(dim=1)
    row_ptr = torch.zeros(m.shape[0] + 1, dtype=torch.int64)
    row_ptr[1:] = counts.cumsum(0)
    cols = m.nonzero()[:, 1]
    return row_ptr.to(torch.int32), cols.to(torch.int32)


def pair_union_plan(mask: torch.Tensor):
    """Merged walk list for pairs of adjacent q-blocks (2p, 2p+1):
    entry = kb*4 + (keep(2p,kb) | keep(2p+1,kb)<<1), ascending kb, only entries with a
    non-zero flag.  An odd trailing q-block pairs with an absent (all-false) row.
    Returns (pair_ptr int32 [slices*npairs+1], entries int32)."""
    nbq, nbk = mask.shape[-2:]
    m = mask.reshape(-1, nbq, nbk).bool()
    if nbq % 2:
        m = torch.cat([m, torch.zeros(m.shape[0], 1, nbk, dtype=torch.bool)], dim=1)
    flags = m[:, 0::2, :].to(torch.int32) + 2 * m[:, 1::2, :].to(torch.int32)
    flat = flags.reshape(-1, nbk)
    nz = flat != 0
    counts = nz.sum(dim=1)
    ptr = torch.zeros(flat.shape[0] + 1, dtype=torch.int64)
    ptr[1:] = counts.cumsum(0)
    pos = nz.nonzero()
    ent = pos[:, 1].to(torch.int32) * 4 + flat[nz]
    return ptr.to(torch.int32), ent.to(torch.int32)


# --------------------------------------------------------------------------- attention
def pair_schedule(mask: torch.Tensor):
    """Walk order of the attention kernel for every pair of adjacent q-blocks (2p, 2p+1) of a mask
    [slices, nbq, nbk]: first the k-blocks both keep (ascending), then the r-th block only 2p keeps
    beside the r-th block only 2p+1 keeps.  Returns (entries int32 in the slots of the pair's merged
    list -- kbA | kbB << 16 with 0xFFFF for "none", unused slots all ones -- and counts int32
    [slices*npairs, 2] = steps of q-block 2p, of 2p+1)."""
    m = mask.reshape(-1, mask.shape[-2], mask.shape[-1]).bool()
    slices, nbq, nbk = m.shape
    npairs = (nbq + 1) // 2
    ent, cnt = [], []
    for sl in range(slices):
        for p in range(npairs):
            a = m[sl, 2 * p]
            b = m[sl, 2 * p + 1] if 2 * p + 1 < nbq else torch.zeros(nbk, dtype=torch.bool)
            both = torch.nonzero(a & b).flatten().tolist()
            only_a = torch.nonzero(a & ~b).flatten().tolist()
            only_b = torch.nonzero(b & ~a).flatten().tolist()
            union = int((a | b).sum())
            steps = [(k, k) for k in both]
            for r in range(max(len(only_a), len(only_b))):
                steps.append((only_a[r] if r < len(only_a) else 0xFFFF, only_b[r] if r < len(only_b) else 0xFFFF))
            words = [ka | (kb << 16) for ka, kb in steps] + [0xFFFFFFFF] * (union - len(steps))
            ent.extend(words)
            cnt.append((len(both) + len(only_a), len(both) + len(only_b)))
    e = torch.tensor(ent, dtype=torch.int64)
    e = torch.where(e >= 2 ** 31, e - 2 ** 32, e).to(torch.int32)
    return e, torch.tensor(cnt, dtype=torch.int32).reshape(-1, 2)


def sparse_attention(q_i8, q_scale, k_i8, k_scale, v8, v_scale, vm, mask, sm_scale: float,
                     q_group: int = 32, out_dtype=torch.bfloat16, return_lse: bool = False,
                     heads: Optional[Sequence[int]] = None, q_blocks: Optional[Sequence[int]] = None):
    """Fake-quant block-sparse attention in fp32 on dequantised operands.

    S = (Qi8 . Ki8^T) * q_scale[row group] * k_scale[col block] * sm_scale * log2e
    (qk_int_sv_f16_cuda_sm80.cu:91,248-253); blocks whose mask entry is false and columns
    >= N are excluded (:268, attn_utils.cuh:355-381); P = 2^(S - rowmax); O = P.Vhat / sum(P)
    with Vhat = float(v8) * v_scale (+ vm).  A row with no kept block gives 0 (:166-167).
    LSE = (log2(sum P) + rowmax)/log2e (:721, core.py:214).

    mask: [Hm or B*H..., nb, nb] with leading dims broadcast over batch when it has H slices.
    `heads` / `q_blocks` restrict the computed rows (used for bounded CPU timing); rows not
    computed are left 0."""
    B, H, N, D = q_i8.shape
    nb = (N + 63) // 64
    m = mask.reshape(-1, nb, nb).bool()
    out = torch.zeros(B, H, N, D, dtype=out_dtype)
    # a row without a kept block has an empty sum: output 0, LSE = log 0 = -inf
    lse = torch.full((B, H, N), float("-inf"), dtype=torch.float32) if return_lse else None
    c = torch.tensor(sm_scale, dtype=torch.float32) * torch.tensor(LOG2E, dtype=torch.float32)
    per64 = 64 // q_group
    for b in range(B):
        for h in (range(H) if heads is None else heads):
            mk = m[(b * H + h) % m.shape[0]]
            qf = q_i8[b, h].float()
            kf = k_i8[b, h].float()
            vhat = v8[b, h, :, :N].float().t() * v_scale[b, h].reshape(1, D)
            if vm is not None:
                vhat = vhat + vm[b, h].reshape(1, D)
            for qb in (range(nb) if q_blocks is None else q_blocks):
                r0, r1 = qb * 64, min(qb * 64 + 64, N)
                kept = mk[qb].nonzero().flatten()
                if kept.numel() == 0:
                    continue
                cols = (kept.reshape(-1, 1) * 64 + torch.arange(64).reshape(1, -1)).flatten()
                colscale = k_scale[b, h][kept].repeat_interleave(64)
                valid = cols < N
                cols, colscale = cols[valid], colscale[valid]
                rows = torch.arange(r0, r1)
                rowscale = q_scale[b, h][qb * per64 + (rows - r0) // q_group]
                s = qf[r0:r1] @ kf[cols].t()
                s = s * rowscale.reshape(-1, 1) * colscale.reshape(1, -1) * c
                mx = s.amax(dim=1, keepdim=True)
                p = torch.exp2(s - mx)
                l = p.sum(dim=1, keepdim=True)
                out[b, h, r0:r1] = ((p @ vhat[cols]) / l).to(out_dtype)
                if return_lse:
                    lse[b, h, r0:r1] = ((torch.log2(l) + mx) / LOG2E).flatten()
    return (out, lse) if return_lse else out


def merge_attention_states(o_a, lse_a, o_b, lse_b):
    """Two partial attention results over disjoint key sets -> the result over their union (what the
    reference returns the LSE for, core.py:55-57): lse = log(e^lse_a + e^lse_b),
    o = o_a * e^(lse_a - lse) + o_b * e^(lse_b - lse) in fp32, rounded to o_a's dtype.  o_*: [B,H,N,D];
    lse_*: [B,H,N] natural log, -inf where a side kept no block for the row (that side is then ignored)."""
    m = torch.maximum(lse_a, lse_b)
    safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    ea, eb = torch.exp(lse_a - safe), torch.exp(lse_b - safe)
    ssum = ea + eb
    wa = torch.where(ssum > 0, ea / ssum.clamp_min(1e-38), torch.zeros_like(ea)).unsqueeze(-1)
    wb = torch.where(ssum > 0, eb / ssum.clamp_min(1e-38), torch.zeros_like(eb)).unsqueeze(-1)
    va = torch.where(wa != 0, wa * o_a.float(), torch.zeros_like(o_a, dtype=torch.float32))
    vb = torch.where(wb != 0, wb * o_b.float(), torch.zeros_like(o_b, dtype=torch.float32))
    lse = torch.where(ssum > 0, safe + torch.log(ssum.clamp_min(1e-38)), torch.full_like(m, float("-inf")))
    return (va + vb).to(o_a.dtype), lse


def apply_empty_heads(mask, empty, n_text_blocks=0):
    """The video-to-video blocks of the heads flagged in `empty` ([H] bool) switched off; text rows and
    columns stay (the mask multiply of example/pipeline_cogvideox.py:76-77, before its text padding)."""
    if empty is None:
        return mask
    out = mask.clone()
    t = int(n_text_blocks)
    for h in torch.as_tensor(empty).bool().nonzero().flatten().tolist():
        out[..., h, t:, t:] = False
    return out


def paro_attention(q, k, v, order_ids, mask, grid, n_text=0, rope=None, sm_scale=None,
                   smooth_k=True, smooth_v=True, q_group=32, return_lse=False, q_norm=None, k_norm=None,
                   empty=None, empty_mode="zero"):
    """The composed path as the processors run it (cogvideox.py:167-227): RoPE on Q,K ->
    permute Q,K,V -> INT8 Q (per 32 rows), INT8 K (per 64 rows, mean-smoothed), FP8 V ->
    block-sparse attention -> inverse permute.  `rope` = None | ("real"|"complex", cos, sin)
    with per-token tables [F*H*W, D/2]; q_norm / k_norm as in `apply_qk_norm` (applied first).
    empty ([H] bool, the permute plan's 'empty' flags; bench/check.py:116-128): "zero" removes the flagged
    heads' video-to-video blocks; "uniform" (n_text == 0 only) sets their output to the mean of V over the
    tokens (fp64 sum, rounded to fp32, then to the output dtype)."""
    D = q.shape[-1]
    mask = apply_empty_heads(mask, empty, (n_text + 63) // 64)
    if sm_scale is None:
        sm_scale = D ** -0.5
    q, k = apply_qk_norm(q, q_norm), apply_qk_norm(k, k_norm)
    if rope is not None:
        kind, cos, sin = rope
        fn = apply_rope_real if kind == "real" else apply_rope_complex
        q, k = fn(q, cos, sin, n_text), fn(k, cos, sin, n_text)
    qp = permute_tokens(q, order_ids, grid, n_text)
    kp = permute_tokens(k, order_ids, grid, n_text)
    vp = permute_tokens(v, order_ids, grid, n_text)
    km = channel_mean(kp, kp.dtype) if smooth_k else None
    q8, qs = quant_int8(qp, q_group)
    k8, ks = quant_int8(kp, 64, km=km)
    v8, vs, vm = quant_v_fp8(vp, smooth=smooth_v)
    res = sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask, sm_scale, q_group=q_group,
                           out_dtype=q.dtype, return_lse=return_lse)
    o, lse = res if return_lse else (res, None)
    o = inverse_permute_tokens(o, order_ids, grid, n_text)
    if empty is not None and empty_mode == "uniform":
        assert n_text == 0, "uniform treatment is defined for sequences without text tokens"
        hs = torch.as_tensor(empty).bool().nonzero().flatten()
        mean_v = (v.double().sum(dim=2) / v.shape[2]).float()          # [B,H,D]
        o[:, hs] = mean_v[:, hs].to(o.dtype).unsqueeze(2).expand(-1, -1, o.shape[2], -1)
    if return_lse:
        lse = inverse_permute_tokens(lse.unsqueeze(-1), order_ids, grid, n_text).squeeze(-1)
        return o, lse
    return o


# --------------------------------------------------------------------------- metrics
def cosine_per_head(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    a2, b2 = a.double().flatten(2), b.double().flatten(2)
    return (a2 * b2).sum(-1) / (a2.norm(dim=-1) * b2.norm(dim=-1)).clamp_min(1e-30)


def rel_l1_per_head(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    a2, b2 = a.double().flatten(2), b.double().flatten(2)
    return (a2 - b2).abs().sum(-1) / b2.abs().sum(-1).clamp_min(1e-30)


# --------------------------------------------------------------------------- synthetic workloads
CONFIGS = {
    # name: B, H, D, grid (F,H,W), n_text, dtype, density, rope family
    "c1_plumbing": dict(B=1, H=2, D=64, grid=(4, 16, 16), n_text=0, dtype=torch.float16, density=0.5, rope=None),
    "c2_cogvideox": dict(B=2, H=48, D=64, grid=(13, 30, 45), n_text=226, dtype=torch.bfloat16, density=0.3, rope="cogvideox"),
    "c3_wan_1p3b": dict(B=2, H=12, D=128, grid=(21, 30, 52), n_text=0, dtype=torch.bfloat16, density=0.3, rope="wan"),
    "c4_wan_14b": dict(B=1, H=40, D=128, grid=(21, 45, 80), n_text=0, dtype=torch.bfloat16, density=0.2, rope="wan"),
}


def make_mask(H: int, nb: int, density: float, seed: int, text_blocks: int = 0, window: int = 0) -> torch.Tensor:
    """Bernoulli(density) block mask [H, nb, nb] from a seeded CPU generator, shared over the
    batch (cogvideox.py:191-193), with diagonal blocks, the first `text_blocks` rows/columns and
    a +-`window` band forced on."""
    g = torch.Generator().manual_seed(seed)
    m = torch.rand(H, nb, nb, generator=g) < density
    i = torch.arange(nb)
    m[:, i, i] = True
    if text_blocks:
        m[:, :text_blocks, :] = True
        m[:, :, :text_blocks] = True
    if window:
        band = (i.reshape(-1, 1) - i.reshape(1, -1)).abs() <= window
        m |= band.unsqueeze(0)
    return m


def make_inputs(B, H, N, D, dtype, seed=0, orders_seed=None):
    """Q,K,V ~ N(0,1); K gets a per-channel offset ~ N(0,2) (variance 2); per-head order ids
    uniform over the 6 orders."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, N, D, generator=g)
    k = torch.randn(B, H, N, D, generator=g) + math.sqrt(2.0) * torch.randn(1, H, 1, D, generator=g)
    v = torch.randn(B, H, N, D, generator=g)
    orders = torch.randint(0, 6, (H,), generator=g)
    return q.to(dtype), k.to(dtype), v.to(dtype), orders.tolist()


def sha256_of(t: torch.Tensor) -> str:
    import hashlib
    a = t.contiguous()
    if a.dtype == torch.bfloat16:
        a = a.view(torch.int16)
    if a.dtype == torch.float8_e4m3fn:
        a = a.view(torch.uint8)
    return hashlib.sha256(np.ascontiguousarray(a.numpy()).tobytes()).hexdigest()
