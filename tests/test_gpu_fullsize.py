"""The model-shaped workloads at their full sizes: size-independent properties over the whole result plus
spot checks of one head against the CPU oracle (whole-tensor oracle runs would take hours)."""
import math

import pytest
import torch

import paroatten_b200 as pb
from oracle import paro_oracle as po

pytestmark = pytest.mark.gpu
DEV = "cuda"

FULL = {
    "cogvideox_5b": dict(B=2, H=48, D=64, grid=(13, 30, 45), n_text=226, density=0.3, family="cogvideox", window=0),
    "wan1p3b_480p": dict(B=2, H=12, D=128, grid=(21, 30, 52), n_text=0, density=0.3, family="wan", window=1),
    "wan14b_720p": dict(B=1, H=40, D=128, grid=(21, 45, 80), n_text=0, density=0.2, family="wan", window=0),
}


def gpu_inputs(B, H, N, D, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.randn(B, H, N, D, generator=g, device=DEV).to(torch.bfloat16)
    k = (torch.randn(B, H, N, D, generator=g, device=DEV) + math.sqrt(2.0) * torch.randn(1, H, 1, D, generator=g, device=DEV)).to(torch.bfloat16)
    v = torch.randn(B, H, N, D, generator=g, device=DEV).to(torch.bfloat16)
    return q, k, v


@pytest.mark.parametrize("name", list(FULL))
def test_full_size_workload(name):
    wl = FULL[name]
    B, H, D, grid, n_text = wl["B"], wl["H"], wl["D"], wl["grid"], wl["n_text"]
    N = n_text + grid[0] * grid[1] * grid[2]
    nb = (N + 63) // 64
    q, k, v = gpu_inputs(B, H, N, D, seed=len(name))
    orders = torch.randint(0, 6, (H,), generator=torch.Generator().manual_seed(1)).tolist()
    mask = po.make_mask(H, nb, wl["density"], seed=2, text_blocks=(n_text + 63) // 64, window=wl["window"])
    ids = torch.tensor(orders, dtype=torch.int32, device=DEV)
    tabs = pb.rope_tables(grid, D, wl["family"])

    # --- walk lists: counts, ordering, flags (whole plan)
    plan = pb.compact_plan(mask.to(DEV))
    assert plan.kept_blocks == int(mask.sum())
    counts = (plan.row_ptr[1:] - plan.row_ptr[:-1]).cpu()
    assert torch.equal(counts, mask.reshape(-1, nb).sum(1).to(torch.int32))
    d = plan.cols[1:] - plan.cols[:-1]
    row_start = torch.zeros(plan.cols.numel(), dtype=torch.bool, device=DEV)
    row_start[plan.row_ptr[:-1][counts.to(DEV) > 0].long()] = True
    assert bool(((d > 0) | row_start[1:]).all())
    flags = plan.pair_ent & 3
    assert int(((flags & 1) != 0).sum() + ((flags & 2) != 0).sum()) == plan.kept_blocks
    # the kernel's schedule covers every kept block once: per pair, steps of 2p + steps of 2p+1 = its kept blocks
    per_pair = torch.zeros(plan.slices * ((nb + 1) // 2), dtype=torch.int64, device=DEV)
    rows = torch.arange(plan.slices * nb, device=DEV)
    per_pair.index_add_(0, (rows // nb) * ((nb + 1) // 2) + (rows % nb) // 2, counts.to(DEV).long())
    assert torch.equal(plan.sched_cnt.long().sum(1), per_pair)
    assert plan.tiles + plan.shared_tiles == plan.kept_blocks and plan.steps <= plan.tiles

    # --- reordering: inverse(forward(x)) == x over the whole tensor, text rows untouched
    fwd = pb.rope_permute(v, ids, grid, n_text)
    assert torch.equal(pb.rope_permute(fwd, ids, grid, n_text, inverse=True), v)
    assert torch.equal(fwd[:, :, :n_text], v[:, :, :n_text])
    del fwd

    # --- whole path
    out, lse = pb.paro_attention(q, k, v, ids, plan, grid_fhw=grid, n_text=n_text, rope=tabs, return_lse=True)
    pb.check_status()
    assert out.shape == q.shape and bool(torch.isfinite(out.float()).all()) and bool(torch.isfinite(lse).all())
    # every output row is a convex combination of (de-quantised) value rows
    vmax = v.float().abs().amax(dim=2, keepdim=True)
    assert bool((out.float().abs() <= vmax * 1.02 + 0.05).all())

    # --- one head against the oracle: quantiser outputs bit for bit, attention rows within tolerance
    b, h = B - 1, H // 2
    qh, kh, vh = (t[b:b + 1, h:h + 1].cpu() for t in (q, k, v))
    cos, sin = po.rope_full_tables(grid, D, wl["family"])
    fn = po.apply_rope_real if wl["family"] == "cogvideox" else po.apply_rope_complex
    qp = po.permute_tokens(fn(qh, cos, sin, n_text), [orders[h]], grid, n_text)
    kp = po.permute_tokens(fn(kh, cos, sin, n_text), [orders[h]], grid, n_text)
    vp = po.permute_tokens(vh, [orders[h]], grid, n_text)
    km = po.channel_mean(kp, kp.dtype)
    q8, qs = po.quant_int8(qp, 32)
    k8, ks = po.quant_int8(kp, 64, km=km)
    v8, vs, vm = po.quant_v_fp8(vp)
    g_qp = pb.rope_permute(q[b:b + 1], ids, grid, n_text, tabs)[:, h:h + 1]
    g_kp = pb.rope_permute(k[b:b + 1], ids, grid, n_text, tabs)[:, h:h + 1]
    g_vp = pb.rope_permute(v[b:b + 1], ids, grid, n_text)[:, h:h + 1]
    assert torch.equal(g_qp.cpu(), qp) and torch.equal(g_kp.cpu(), kp)
    g_km = pb.channel_mean(g_kp)
    assert torch.equal(g_km.cpu(), km)
    g_q8, g_qs, g_k8, g_ks = pb.per_warp_int8(g_qp, g_kp, g_km, BLKQ=64, WARPQ=32, BLKK=64)
    assert torch.equal(g_q8.cpu(), q8) and torch.equal(g_qs.cpu(), qs)
    assert torch.equal(g_k8.cpu(), k8) and torch.equal(g_ks.cpu(), ks)
    g_v8, g_vs, g_vm = pb.per_channel_fp8(g_vp)
    assert torch.equal(g_v8.cpu().view(torch.uint8), v8.view(torch.uint8)) and torch.equal(g_vs.cpu(), vs)
    assert torch.equal(g_vm.cpu(), vm)

    blocks = sorted({0, 1, nb // 2, nb - 2, nb - 1})
    want = po.sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask[h:h + 1], D ** -0.5, out_dtype=torch.bfloat16,
                               q_blocks=blocks)
    idx = po.perm_index(orders[h], grid).long()
    rows = torch.cat([torch.arange(qb * 64, min(qb * 64 + 64, N)) for qb in blocks])
    dst = torch.where(rows < n_text, rows, n_text + idx[(rows - n_text).clamp_min(0)])
    got = out[b, h].cpu()[dst]
    ref = want[0, 0][rows]
    cosv = torch.nn.functional.cosine_similarity(got.double().flatten(), ref.double().flatten(), dim=0).item()
    rl1 = ((got.double() - ref.double()).abs().sum() / ref.double().abs().sum()).item()
    assert cosv >= 0.9995 and rl1 <= 1e-2, f"{name}: cosine {cosv:.6f} rel-L1 {rl1:.3e}"
