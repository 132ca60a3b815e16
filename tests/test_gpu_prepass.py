"""Parity of the pre-attention kernels (permutation tables, plan compaction, RoPE+reorder, INT8 and
FP8 quantisers) with the CPU oracle, through the C-ABI library.  Integer/byte results are compared
bit for bit."""
import os

import numpy as np
import pytest
import torch

import paroatten_b200 as pb
from oracle import paro_oracle as po

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"


def rand(shape, dtype, seed, offset=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) + offset).to(dtype)


@pytest.mark.parametrize("grid", [(13, 30, 45), (4, 16, 16), (1, 1, 7), (3, 5, 2)])
def test_perm_index(grid):
    ids = torch.tensor([0, 1, 2, 3, 4, 5, 5, 2], dtype=torch.int32)
    got = pb.perm_index(ids.to(DEV), grid).cpu()
    assert torch.equal(got, po.perm_index_table(ids.tolist(), grid))


def test_perm_index_reference_fixture():
    ref = torch.from_numpy(np.load(os.path.join(GOLD, "perm_cogvideox_ref.npz"))["table"])
    got = pb.perm_index(torch.arange(6, dtype=torch.int32, device=DEV), (13, 30, 45)).cpu()
    assert torch.equal(got + 226, ref[:, 226:])


@pytest.mark.parametrize("slices,nb,density", [(1, 1, 1.0), (3, 7, 0.4), (2, 33, 0.3), (48, 278, 0.3), (2, 64, 0.0)])
def test_compact_plan(slices, nb, density):
    g = torch.Generator().manual_seed(nb)
    mask = torch.rand(slices, nb, nb, generator=g) < density
    plan = pb.compact_plan(mask.to(DEV))
    ptr, cols = po.compact_plan(mask)
    pptr, pent = po.pair_union_plan(mask)
    assert torch.equal(plan.row_ptr.cpu(), ptr) and torch.equal(plan.cols.cpu(), cols)
    assert torch.equal(plan.pair_ptr.cpu(), pptr) and torch.equal(plan.pair_ent.cpu(), pent)
    assert plan.kept_blocks == int(mask.sum()) and plan.pair_tiles == pent.numel()
    # the schedule the attention kernel walks: shared blocks first, then the rest side by side
    sched, cnt = po.pair_schedule(mask)
    assert torch.equal(plan.sched.cpu(), sched) and torch.equal(plan.sched_cnt.cpu(), cnt)
    both = int((pent & 3).eq(3).sum())
    assert plan.shared_tiles == both and plan.tiles == plan.kept_blocks - both
    assert plan.steps == int(cnt.max(dim=1).values.sum())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D,family,grid,n_text", [(64, "cogvideox", (3, 6, 10), 17), (128, "wan", (2, 5, 9), 0),
                                                  (64, "cogvideox", (13, 30, 45), 226)])
def test_rope_permute(dtype, D, family, grid, n_text):
    H = 6 if grid[0] < 13 else 2
    N = n_text + grid[0] * grid[1] * grid[2]
    x = rand((2, H, N, D), dtype, 11)
    orders = [(h * 5 + 1) % 6 for h in range(H)]
    cos, sin = po.rope_full_tables(grid, D, family)
    fn = po.apply_rope_real if family == "cogvideox" else po.apply_rope_complex
    want = po.permute_tokens(fn(x, cos, sin, n_text), orders, grid, n_text)
    tabs = pb.rope_tables(grid, D, family)
    ids = torch.tensor(orders, dtype=torch.int32, device=DEV)
    got = pb.rope_permute(x.to(DEV), ids, grid, n_text, tabs)
    assert torch.equal(got.cpu(), want)
    # permutation only, RoPE only, inverse, NHD input
    assert torch.equal(pb.rope_permute(x.to(DEV), ids, grid, n_text).cpu(), po.permute_tokens(x, orders, grid, n_text))
    assert torch.equal(pb.rope_permute(x.to(DEV), None, grid, n_text, tabs).cpu(), fn(x, cos, sin, n_text))
    back = pb.rope_permute(pb.rope_permute(x.to(DEV), ids, grid, n_text), ids, grid, n_text, inverse=True)
    assert torch.equal(back.cpu(), x)
    nhd = x.transpose(1, 2).contiguous().to(DEV)
    assert torch.equal(pb.rope_permute(nhd, ids, grid, n_text, tabs, tensor_layout="NHD").cpu(), want)


def test_rope_permutation_reference_signature():
    grid = (2, 6, 8)
    q, k = rand((1, 2, 96, 64), torch.float16, 1), rand((1, 2, 96, 64), torch.float16, 2)
    tabs = pb.rope_tables(grid, 64, "cogvideox")
    qo, ko = pb.rope_permutation(q.to(DEV), k.to(DEV), tabs, True, grid=grid)
    cos, sin = po.rope_full_tables(grid, 64, "cogvideox")
    assert torch.equal(qo.cpu(), po.permute_tokens(po.apply_rope_real(q, cos, sin), [1, 1], grid))
    qo2, _ = pb.rope_permutation(q.to(DEV), k.to(DEV), tabs, False, grid=grid)
    assert torch.equal(qo2.cpu(), po.apply_rope_real(q, cos, sin))
    assert torch.equal(ko.cpu(), po.permute_tokens(po.apply_rope_real(k, cos, sin), [1, 1], grid))


def test_kat_ramp():
    g = np.load(os.path.join(GOLD, "kat_ramp_int8.npz"))
    rows = torch.arange(-256, 256, dtype=torch.bfloat16).unsqueeze(1).repeat(1, 64).reshape(1, 1, 512, 64).to(DEV)
    q8, qs, k8, ks = pb.per_warp_int8(rows, rows, BLKQ=64, WARPQ=32, BLKK=64)
    assert np.array_equal(q8[0, 0, :, 0].cpu().numpy(), g["q_col0"]) and np.array_equal(qs.cpu().numpy(), g["q_scale"])
    assert np.array_equal(k8[0, 0, :, 0].cpu().numpy(), g["k_col0"]) and np.array_equal(ks.cpu().numpy(), g["k_scale"])
    assert (q8 == q8[..., :1]).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,D", [(64, 64), (1024, 64), (1008, 128), (1016, 128), (976, 64), (1, 128), (17776, 64)])
def test_quant_int8(dtype, N, D):
    B, H = (2, 3) if N < 10000 else (1, 2)
    q = rand((B, H, N, D), dtype, N)
    k = rand((B, H, N, D), dtype, N + 1, offset=1.5)
    km_want = po.channel_mean(k, dtype)
    km = pb.channel_mean(k.to(DEV))
    assert torch.equal(km.cpu(), km_want)
    assert torch.equal(pb.channel_mean(k.to(DEV), out_dtype=torch.float32).cpu(), (k.double().sum(2) / N).float())
    q8, qs, k8, ks = pb.per_warp_int8(q.to(DEV), k.to(DEV), km, BLKQ=64, WARPQ=32, BLKK=64)
    wq, wqs = po.quant_int8(q, 32)
    wk, wks = po.quant_int8(k, 64, km=km_want)
    assert torch.equal(q8.cpu(), wq) and torch.equal(qs.cpu(), wqs)
    assert torch.equal(k8.cpu(), wk) and torch.equal(ks.cpu(), wks)
    # per-block Q with the softmax scale folded in, K unsmoothed
    q8b, qsb, k8b, ksb = pb.per_block_int8(q.to(DEV), k.to(DEV), BLKQ=64, BLKK=64, sm_scale=0.2)
    wqb, wqsb = po.quant_int8(q, 64, fold_scale=0.2 * 1.44269504)
    wkb, wksb = po.quant_int8(k, 64)
    assert torch.equal(q8b.cpu(), wqb) and torch.equal(qsb.cpu(), wqsb)
    assert torch.equal(k8b.cpu(), wkb) and torch.equal(ksb.cpu(), wksb)


def test_quant_int8_nhd_layout():
    q = rand((2, 200, 3, 64), torch.float16, 5)  # [B,N,H,D]
    q8, qs, _, _ = pb.per_warp_int8(q.to(DEV), q.to(DEV), BLKQ=64, WARPQ=32, BLKK=64, tensor_layout="NHD")
    wq, wqs = po.quant_int8(q.transpose(1, 2).contiguous(), 32)
    assert q8.shape == q.shape
    assert torch.equal(q8.cpu().transpose(1, 2), wq) and torch.equal(qs.cpu(), wqs)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,D,smooth", [(64, 64, True), (1000, 128, True), (1000, 128, False), (976, 64, True),
                                        (5, 64, True), (17776, 64, True)])
def test_quant_v_fp8(dtype, N, D, smooth):
    B, H = (2, 3) if N < 10000 else (1, 2)
    v = rand((B, H, N, D), dtype, N + 7, offset=0.3) * 2.0
    v8, vs, vm, v16 = pb.per_channel_fp8(v.to(DEV), smooth_v=smooth, return_16=True)
    w8, ws, wm = po.quant_v_fp8(v, smooth=smooth)
    assert torch.equal(vs.cpu(), ws)
    if smooth:
        assert torch.equal(vm.cpu(), wm)
    else:
        assert vm is None
    assert torch.equal(v8.cpu().view(torch.uint8), w8.view(torch.uint8))
    assert torch.equal(v16.cpu(), w8.to(torch.bfloat16))


def test_quant_v_fp8_zero_channel_and_nhd():
    v = rand((1, 100, 2, 64), torch.bfloat16, 3)  # NHD
    v[..., 5] = 0
    v8, vs, vm = pb.per_channel_fp8(v.to(DEV), tensor_layout="NHD")
    w8, ws, wm = po.quant_v_fp8(v.transpose(1, 2).contiguous())
    assert v8.shape == (1, 64, 2, 128)
    assert torch.equal(v8.cpu().transpose(1, 2).contiguous().view(torch.uint8), w8.view(torch.uint8))
    assert torch.equal(vs.cpu(), ws) and torch.isfinite(v8.float()).all()


def test_argument_errors():
    x = torch.zeros(1, 1, 64, 96, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError, match="head_dim"):
        pb.per_warp_int8(x, x, BLKQ=64, WARPQ=32, BLKK=64)
    with pytest.raises(ValueError):
        pb.per_warp_int8(x[..., :64].contiguous(), x[..., :64].contiguous(), WARPQ=16)
    y = torch.zeros(1, 1, 64, 64, dtype=torch.float32, device=DEV)
    with pytest.raises(ValueError, match="dtype"):
        pb.per_channel_fp8(y)
    z = torch.zeros(1, 2, 50, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError, match="!= N"):
        pb.rope_permute(z, None, (1, 7, 7))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D,family,grid,n_text", [(64, "cogvideox", (3, 6, 10), 17), (128, "wan", (2, 5, 9), 0),
                                                  (128, "wan", (3, 7, 11), 40)])
def test_fused_prep_equals_separate_passes(dtype, D, family, grid, n_text):
    """RoPE + reorder + quantise in one pass gives the very same bytes as the separate kernels and
    as the oracle."""
    B, H = 2, 6
    N = n_text + grid[0] * grid[1] * grid[2]
    q, k, v = rand((B, H, N, D), dtype, 31), rand((B, H, N, D), dtype, 32, offset=1.0), rand((B, H, N, D), dtype, 33)
    orders = [(h * 5 + 2) % 6 for h in range(H)]
    ids = torch.tensor(orders, dtype=torch.int32, device=DEV)
    tabs = pb.rope_tables(grid, D, family)
    cos, sin = po.rope_full_tables(grid, D, family)
    fn = po.apply_rope_real if family == "cogvideox" else po.apply_rope_complex
    qp = po.permute_tokens(fn(q, cos, sin, n_text), orders, grid, n_text)
    kp = po.permute_tokens(fn(k, cos, sin, n_text), orders, grid, n_text)
    vp = po.permute_tokens(v, orders, grid, n_text)
    km = po.channel_mean(kp, dtype)
    wq, wqs = po.quant_int8(qp, 32)
    wk, wks = po.quant_int8(kp, 64, km=km)
    w8, wvs, wvm = po.quant_v_fp8(vp)
    q8, qs, none = pb.prep_qk_int8(q.to(DEV), ids, grid, n_text, tabs, group=32)
    assert none is None and torch.equal(q8.cpu(), wq) and torch.equal(qs.cpu(), wqs)
    k8, ks, gkm = pb.prep_qk_int8(k.to(DEV), ids, grid, n_text, tabs, group=64, smooth=True)
    assert torch.equal(gkm.cpu(), km) and torch.equal(k8.cpu(), wk) and torch.equal(ks.cpu(), wks)
    v16, vs, vm, v8 = pb.prep_v_fp8(v.to(DEV), ids, grid, n_text, want_fp8=True)
    assert torch.equal(v8.cpu().view(torch.uint8), w8.view(torch.uint8)) and torch.equal(v16.cpu(), w8.to(torch.bfloat16))
    assert torch.equal(vs.cpu(), wvs) and torch.equal(vm.cpu(), wvm)
    # NHD input, no fp8 copy
    v16b, _, _, none8 = pb.prep_v_fp8(v.transpose(1, 2).contiguous().to(DEV), ids, grid, n_text, tensor_layout="NHD")
    assert none8 is None and torch.equal(v16b, v16)


def _norm_case(kind, H, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "layer":
        w = (1.0 + 0.2 * torch.randn(D, generator=g)).to(dtype)
        b = (0.1 * torch.randn(D, generator=g)).to(dtype)
        return pb.QKNorm("layer", w.to(DEV), b.to(DEV), 1e-6), ("layer", w, b, 1e-6)
    w = (1.0 + 0.2 * torch.randn(H * D, generator=g)).to(dtype)
    return pb.QKNorm("rms", w.to(DEV), None, 1e-6), ("rms", w, 1e-6)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kind,D,family,grid,n_text", [("layer", 64, "cogvideox", (3, 6, 10), 17),
                                                       ("layer", 128, "wan", (2, 5, 9), 0),
                                                       ("rms", 128, "wan", (3, 7, 11), 0),
                                                       ("rms", 64, "cogvideox", (2, 5, 9), 40)])
def test_qk_norm_folded_into_the_passes(kind, D, family, grid, n_text, dtype):
    """norm_q / norm_k applied inside the RoPE + reorder (+ quantise) passes: the same bytes as the
    oracle's normalise -> rotate -> reorder -> quantise, text tokens included."""
    B, H = 2, 6
    N = n_text + grid[0] * grid[1] * grid[2]
    x = rand((B, H, N, D), dtype, 51, offset=0.3) * 3.0
    orders = [(h * 5 + 3) % 6 for h in range(H)]
    ids = torch.tensor(orders, dtype=torch.int32, device=DEV)
    norm, onorm = _norm_case(kind, H, D, dtype, 52)
    tabs = pb.rope_tables(grid, D, family)
    cos, sin = po.rope_full_tables(grid, D, family)
    fn = po.apply_rope_real if family == "cogvideox" else po.apply_rope_complex
    xn = po.apply_qk_norm(x, onorm)
    want = po.permute_tokens(fn(xn, cos, sin, n_text), orders, grid, n_text)
    got = pb.rope_permute(x.to(DEV), ids, grid, n_text, tabs, norm=norm)
    assert torch.equal(got.cpu(), want)
    # norm only (no rotation, no reordering) and NHD input
    assert torch.equal(pb.rope_permute(x.to(DEV), None, grid, n_text, norm=norm).cpu(), xn)
    nhd = x.transpose(1, 2).contiguous().to(DEV)
    assert torch.equal(pb.rope_permute(nhd, ids, grid, n_text, tabs, tensor_layout="NHD", norm=norm).cpu(), want)
    # fused with the INT8 quantiser
    for group in (32, 64):
        w8, ws = po.quant_int8(want, group)
        q8, qs, _ = pb.prep_qk_int8(x.to(DEV), ids, grid, n_text, tabs, group=group, norm=norm)
        assert torch.equal(q8.cpu(), w8) and torch.equal(qs.cpu(), ws)
    q8n, qsn, _ = pb.prep_qk_int8(nhd, ids, grid, n_text, tabs, group=32, tensor_layout="NHD", norm=norm)
    w8, ws = po.quant_int8(want, 32)
    assert torch.equal(q8n.cpu(), w8) and torch.equal(qsn.cpu(), ws)
    with pytest.raises(ValueError):
        pb.prep_qk_int8(x.to(DEV), ids, grid, n_text, tabs, group=64, smooth=True, norm=norm)


def test_qk_norm_argument_errors():
    x = torch.zeros(1, 2, 64, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        pb.rope_permute(x, None, (1, 8, 8), norm=pb.QKNorm("layer", torch.ones(32, device=DEV)))
    with pytest.raises(ValueError):
        pb.rope_permute(x, None, (1, 8, 8), norm=pb.QKNorm("rms", torch.ones(64, device=DEV)))
    with pytest.raises(ValueError):
        pb.rope_permute(x, None, (1, 8, 8), norm=pb.QKNorm("batch", torch.ones(64, device=DEV)))
    with pytest.raises(ValueError):
        pb.rope_permute(x, None, (1, 8, 8), inverse=True, norm=pb.QKNorm("layer", torch.ones(64, device=DEV)))


@pytest.mark.parametrize("N,D,dtype", [(300, 64, torch.float16), (1000, 128, torch.bfloat16)])
def test_reference_default_block_sizes(N, D, dtype):
    """per_warp_int8 / per_block_int8 called with the reference's defaults (BLKQ=128,
    paroattention/quant.py:22-30,105-112): same values as the oracle's per-128 quantiser; per-warp Q
    only differs from the BLKQ=64 call in the padding of its scale array."""
    B, H = 2, 3
    q, k = rand((B, H, N, D), dtype, 61), rand((B, H, N, D), dtype, 62, offset=0.5)
    q8, qs, k8, ks = pb.per_warp_int8(q.to(DEV), k.to(DEV))                      # BLKQ=128, WARPQ=32, BLKK=64
    w8, ws = po.quant_int8(q, 32)
    assert torch.equal(q8.cpu(), w8) and qs.shape[-1] == (N + 127) // 128 * 4
    assert torch.equal(qs.cpu()[..., :ws.shape[-1]], ws)
    assert torch.equal(k8.cpu(), po.quant_int8(k, 64)[0])
    sm = D ** -0.5
    q8b, qsb, k8b, ksb = pb.per_block_int8(q.to(DEV), k.to(DEV), sm_scale=sm)     # BLKQ=128, BLKK=64
    w8b, wsb = po.quant_int8(q, 128, fold_scale=sm * 1.44269504)
    assert qsb.shape == wsb.shape == (B, H, (N + 127) // 128)
    assert torch.equal(q8b.cpu(), w8b) and torch.equal(qsb.cpu(), wsb)
    assert torch.equal(k8b.cpu(), po.quant_int8(k, 64)[0]) and torch.equal(ksb.cpu(), po.quant_int8(k, 64)[1])
