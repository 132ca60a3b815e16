"""Parity of the block-sparse attention kernel (and of the composed path) with the CPU
fake-quant oracle.  Tolerance: cosine similarity >= 0.9995 and relative L1 <= 1e-2 per head."""
import os

import numpy as np
import pytest
import torch

import paroatten_b200 as pb
from oracle import paro_oracle as po

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"
COS_MIN, RL1_MAX = 0.9995, 1e-2


def assert_close(got, want, what=""):
    c = po.cosine_per_head(got.cpu(), want).min().item()
    r = po.rel_l1_per_head(got.cpu(), want).max().item()
    assert c >= COS_MIN and r <= RL1_MAX, f"{what}: min cosine {c:.6f}, max rel-L1 {r:.3e}"


def quantised(q, k, v, orders, grid, n_text=0):
    qp, kp, vp = (po.permute_tokens(t, orders, grid, n_text) for t in (q, k, v))
    km = po.channel_mean(kp, kp.dtype)
    q8, qs = po.quant_int8(qp, 32)
    k8, ks = po.quant_int8(kp, 64, km=km)
    v8, vs, vm = po.quant_v_fp8(vp)
    return q8, qs, k8, ks, v8, vs, vm


@pytest.mark.parametrize("D,N,H,density,dtype", [
    (64, 1024, 2, 0.5, torch.float16),
    (128, 1024, 2, 0.5, torch.bfloat16),
    (128, 64, 1, 1.0, torch.bfloat16),      # single block, odd block count
    (64, 200, 3, 1.0, torch.float16),       # ragged tail 8, dense
    (128, 1008, 2, 0.4, torch.bfloat16),    # tail 48
    (128, 1016, 2, 0.4, torch.float16),     # tail 56, 16 blocks
    (64, 976, 2, 0.3, torch.bfloat16),      # tail 16, odd block count (pair with a missing half)
    (128, 4160, 2, 0.2, torch.bfloat16),    # 65 blocks: long lists, ring wrap-around
])
@pytest.mark.parametrize("mode,pairing", [("fast", "adjacent"), ("exact", "adjacent"), ("fast", "overlap")])
def test_kernel_on_oracle_quantised_operands(D, N, H, density, dtype, mode, pairing):
    """The kernel alone: operands quantised by the ORACLE, so only the attention differs.  Both
    walks: the fast one (fixed reference exponent per row) and the exact one (running maximum)."""
    B = 2
    q, k, v, _ = po.make_inputs(B, H, N, D, dtype, seed=N + D)
    nb = (N + 63) // 64
    mask = po.make_mask(H, nb, density, seed=N)
    q8, qs, k8, ks, v8, vs, vm = quantised(q, k, v, [0] * H, (1, 1, N))
    want, want_lse = po.sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask, D ** -0.5, out_dtype=dtype, return_lse=True)
    plan = pb.compact_plan(mask.to(DEV), pairing=pairing)   # "overlap": q-blocks paired by the k-blocks they share
    got, lse = pb.sparse_attn_quantized(q8.to(DEV), qs.to(DEV), k8.to(DEV), ks.to(DEV), v8.to(torch.bfloat16).to(DEV),
                                        vs.to(DEV), vm.to(DEV), plan, D ** -0.5, out_dtype=dtype, return_lse=True,
                                        mode=mode)
    pb.check_status()
    if mode == "fast":
        assert pb.last_redo_count() == 0      # N(0,1) data never leaves the fast walk's exponent range
    assert_close(got, want, f"D={D} N={N} {mode}")
    assert (lse.cpu() - want_lse).abs().max().item() < 2e-3


@pytest.mark.parametrize("D,growth,mode", [(128, 1.0, "exact"), (64, 1.0, "exact"), (128, -1.0, "exact"),
                                           (128, 0.25, "exact"), (128, 1.0, "fast"), (64, 0.25, "fast"),
                                           (128, 6.0, "fast"), (64, 6.0, "fast"), (128, -6.0, "fast")])
def test_row_maximum_that_keeps_growing(D, growth, mode):
    """Keys of later blocks are scaled up (or down), so that along every row's list the running
    maximum rises by more than the lazy-rescaling threshold again and again.  Exact walk: the
    accumulator is rescaled by the warp set whose step saw the rise, and the other set picks the new
    maximum up.  Fast walk: moderate growth stays inside its exponent range; with growth 6 the scores
    of late blocks lie hundreds of powers of two above a row's first block, so pairs of q-blocks are
    handed to the exact walk (the redo count says so) and the result is still the oracle's."""
    B, H, N = 1, 2, 1024
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.bfloat16, seed=77)
    nb = N // 64
    j = torch.arange(nb, dtype=torch.float32)
    f = (1.0 + growth * j) if growth > 0 else (1.0 + (-growth) * (nb - 1 - j))
    k = (k.float() * f.repeat_interleave(64).reshape(1, 1, N, 1)).to(torch.bfloat16)
    mask = po.make_mask(H, nb, 0.7, seed=5)
    q8, qs, k8, ks, v8, vs, vm = quantised(q, k, v, [0] * H, (1, 1, N))
    want, want_lse = po.sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask, D ** -0.5, out_dtype=torch.bfloat16,
                                         return_lse=True)
    plan = pb.compact_plan(mask.to(DEV))
    got, lse = pb.sparse_attn_quantized(q8.to(DEV), qs.to(DEV), k8.to(DEV), ks.to(DEV), v8.to(torch.bfloat16).to(DEV),
                                        vs.to(DEV), vm.to(DEV), plan, D ** -0.5, out_dtype=torch.bfloat16,
                                        return_lse=True, mode=mode)
    pb.check_status()
    if mode == "fast":
        redone = pb.last_redo_count()
        assert (redone > 0) if growth >= 6.0 else (redone >= 0)
    assert torch.isfinite(got.float()).all()
    assert_close(got, want, f"D={D} growth={growth} {mode}")
    assert ((lse.cpu() - want_lse).abs() / want_lse.abs().clamp_min(1.0)).max().item() < 2e-3


def test_c1_plumbing_fixture():
    """The small CPU-runnable configuration end to end against the committed oracle output."""
    cfg = po.CONFIGS["c1_plumbing"]
    N = 1024
    q, k, v, orders = po.make_inputs(cfg["B"], cfg["H"], N, cfg["D"], cfg["dtype"], seed=0)
    mask = po.make_mask(cfg["H"], 16, cfg["density"], seed=0)
    g = np.load(os.path.join(GOLD, "c1_plumbing_out.npz"))
    want = torch.from_numpy(g["out"]).view(torch.float16)
    got, lse = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(orders), mask.to(DEV),
                                 grid_fhw=cfg["grid"], return_lse=True)
    pb.check_status()
    assert_close(got, want, "c1")
    assert (lse.cpu() - torch.from_numpy(g["lse"])).abs().max().item() < 2e-3


@pytest.mark.parametrize("family,D,grid,n_text,dtype", [
    ("cogvideox", 64, (3, 10, 15), 226, torch.bfloat16),
    ("wan", 128, (3, 6, 13), 0, torch.bfloat16),
    ("wan", 128, (2, 9, 8), 40, torch.float16),
])
def test_composed_path(family, D, grid, n_text, dtype):
    """RoPE + reorder + quantisers + attention + inverse reorder, all on the GPU, against the
    composed oracle; also checks the intermediate integer tensors bit for bit."""
    B, H = 2, 6
    N = n_text + grid[0] * grid[1] * grid[2]
    q, k, v, orders = po.make_inputs(B, H, N, D, dtype, seed=sum(grid))
    nb = (N + 63) // 64
    mask = po.make_mask(H, nb, 0.4, seed=1, text_blocks=(n_text + 63) // 64)
    cos, sin = po.rope_full_tables(grid, D, family)
    kind = "real" if family == "cogvideox" else "complex"
    want, want_lse = po.paro_attention(q, k, v, orders, mask, grid, n_text=n_text, rope=(kind, cos, sin), return_lse=True)
    tabs = pb.rope_tables(grid, D, family)
    got, lse = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), {"permute": torch.tensor([orders])},
                                 mask.to(DEV).reshape(1, 1, H, nb, nb), i_block=0, i_timestep=0, grid_fhw=grid,
                                 n_text=n_text, rope=tabs, return_lse=True)
    pb.check_status()
    assert_close(got, want, family)
    assert (lse.cpu() - want_lse).abs().max().item() < 2e-3
    # NHD in, NHD out
    got2 = pb.paro_attention(*(t.transpose(1, 2).contiguous().to(DEV) for t in (q, k, v)), torch.tensor(orders),
                             mask.to(DEV), grid_fhw=grid, n_text=n_text, rope=tabs, tensor_layout="NHD")
    assert torch.equal(got2.transpose(1, 2), got)


def test_mask_per_batch_entry():
    """A [B, H, nb, nb] mask gives every batch entry its own plan slices."""
    B, H, N, D = 2, 3, 700, 64
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.bfloat16, seed=12)
    nb = (N + 63) // 64
    masks = torch.stack([po.make_mask(H, nb, 0.3, seed=40), po.make_mask(H, nb, 0.8, seed=41)])   # [B, H, nb, nb]
    got = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.zeros(H, dtype=torch.int32), masks.to(DEV),
                            grid_fhw=(1, 1, N))
    pb.check_status()
    for b in range(B):
        want = po.paro_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], [0] * H, masks[b], (1, 1, N))
        assert_close(got[b:b + 1], want, f"batch entry {b}")


def test_reference_operator_signature():
    """paroattn_qk_int8_pv_fp16_cuda(q, k, v, sparse): already reordered inputs, bool mask."""
    B, H, N, D = 2, 3, 520, 96   # head_dim padded to 128 like the reference
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.float16, seed=2)
    nb = (N + 63) // 64
    mask = po.make_mask(H, nb, 0.5, seed=2)
    pad = lambda t: torch.nn.functional.pad(t, (0, 128 - D))
    q8, qs = po.quant_int8(pad(q), 32)
    k8, ks = po.quant_int8(pad(k), 64)
    v8, vs, vm = po.quant_v_fp8(pad(v))
    want = po.sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask, D ** -0.5, out_dtype=torch.float16)[..., :D]
    sparse = torch.stack([mask, mask]).to(DEV)  # [B,H,nb,nb] as the processors build it
    got = pb.paroattn_qk_int8_pv_fp16_cuda(q.to(DEV), k.to(DEV), v.to(DEV), sparse)
    pb.check_status()
    assert got.shape == (B, H, N, D)
    assert_close(got, want, "per_warp")
    got_nhd = pb.paroattn(*(t.transpose(1, 2).contiguous().to(DEV) for t in (q, k, v)), tensor_layout="NHD", sparse=sparse)
    assert torch.equal(got_nhd.transpose(1, 2), got)
    # "per_thread": per-block Q with the scale folded in
    q8b, qsb = po.quant_int8(pad(q), 64, fold_scale=D ** -0.5 * 1.44269504)
    want_b = po.sparse_attention(q8b, qsb, k8, ks, v8, vs, vm, mask, 1.0 / 1.44269504, q_group=64,
                                 out_dtype=torch.float16)[..., :D]
    got_b = pb.paroattn_qk_int8_pv_fp16_cuda(q.to(DEV), k.to(DEV), v.to(DEV), sparse, qk_quant_gran="per_thread")
    assert_close(got_b, want_b, "per_thread")
    with pytest.raises(ValueError):
        pb.paroattn_qk_int8_pv_fp16_cuda(q.to(DEV), k.to(DEV), v.to(DEV), sparse, is_causal=True)


def test_dense_mask_matches_sdpa():
    B, H, N, D = 1, 2, 1500, 128
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.bfloat16, seed=9)
    mask = torch.ones(H, 24, 24, dtype=torch.bool, device=DEV)
    got = pb.paroattn_qk_int8_pv_fp16_cuda(q.to(DEV), k.to(DEV), v.to(DEV), mask, smooth_k=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    assert po.cosine_per_head(got.cpu(), ref).min().item() > 0.998


def test_empty_rows_give_zero():
    B, H, N, D = 1, 1, 256, 64
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.float16, seed=3)
    mask = torch.zeros(H, 4, 4, dtype=torch.bool)
    mask[0, 0, 1] = mask[0, 3, 3] = True      # q-blocks 1 and 2 keep nothing
    got = pb.paroattn_qk_int8_pv_fp16_cuda(q.to(DEV), k.to(DEV), v.to(DEV), mask.to(DEV))
    pb.check_status()
    assert (got[0, 0, 64:192] == 0).all() and got[0, 0, :64].abs().sum() > 0 and got[0, 0, 192:].abs().sum() > 0


def test_processors_on_a_stand_in_attention_module():
    """The two processors driven by a minimal module with the attributes they read."""
    import torch.nn as nn

    class Attn(nn.Module):
        def __init__(self, dim, heads):
            super().__init__()
            self.heads = heads
            self.to_q, self.to_k, self.to_v = (nn.Linear(dim, dim) for _ in range(3))
            self.to_out = nn.ModuleList([nn.Linear(dim, dim), nn.Dropout(0.0)])
            self.norm_q = self.norm_k = None

    torch.manual_seed(0)
    heads, D, grid, n_text = 2, 64, (2, 4, 8), 32
    attn = Attn(heads * D, heads).to(DEV, torch.bfloat16)
    proc = pb.PARO_CogVideoXAttnProcessor2_0()
    proc.grid_fhw = grid
    proc.permute_plan = {"permute": torch.tensor([[4, 2]])}
    nb = (n_text + 64 + 63) // 64
    proc.sparse_mask = torch.ones(1, 1, heads, nb, nb, dtype=torch.bool, device=DEV)
    proc.i_block, proc.i_timestep = 0, 0
    hs = torch.randn(1, 64, heads * D, device=DEV, dtype=torch.bfloat16)
    enc = torch.randn(1, n_text, heads * D, device=DEV, dtype=torch.bfloat16)
    h_out, e_out = proc(attn, hs, enc, image_rotary_emb=None)
    assert h_out.shape == hs.shape and e_out.shape == enc.shape
    x = torch.cat([enc, hs], 1)
    qkv = [f(x).view(1, -1, heads, D).transpose(1, 2).float() for f in (attn.to_q, attn.to_k, attn.to_v)]
    ref = torch.nn.functional.scaled_dot_product_attention(*qkv).transpose(1, 2).reshape(1, -1, heads * D)
    ref = attn.to_out[0](ref.to(torch.bfloat16))
    got = torch.cat([e_out, h_out], 1)
    assert torch.nn.functional.cosine_similarity(got.float().flatten(), ref.float().flatten(), dim=0) > 0.99
    assert proc.get_time_stats()["total_ms"] > 0 and proc.call_count == 1

    wan = pb.PARO_WanAttnProcessor2_0()
    wan.grid_fhw = (2, 4, 12)
    wan.permute_plan = {"permute": torch.tensor([[1, 5]])}
    wan.sparse_mask = torch.ones(1, 1, heads, 2, 2, dtype=torch.bool, device=DEV)
    hs = torch.randn(1, 96, heads * D, device=DEV, dtype=torch.bfloat16)
    out = wan(attn, hs, rotary_emb=None)
    qkv = [f(hs).view(1, -1, heads, D).transpose(1, 2).float() for f in (attn.to_q, attn.to_k, attn.to_v)]
    ref = attn.to_out[0](torch.nn.functional.scaled_dot_product_attention(*qkv).transpose(1, 2).reshape(1, -1, heads * D).to(torch.bfloat16))
    assert torch.nn.functional.cosine_similarity(out.float().flatten(), ref.float().flatten(), dim=0) > 0.99


def test_processors_fold_qk_norm():
    """norm_q / norm_k of the two known forms are folded into the pre-attention passes; the result
    agrees with calling the modules (the reference's order of operations) within the attention
    tolerance, and the composed call with norms matches the oracle."""
    import torch.nn as nn

    class RMSNorm(nn.Module):   # stand-in with the attribute shape of an across-heads RMS norm
        def __init__(self, dim, eps=1e-6):
            super().__init__()
            self.weight, self.eps, self.bias = nn.Parameter(torch.ones(dim)), eps, None

        def forward(self, x):
            v = x.float().pow(2).mean(-1, keepdim=True)
            return (x.float() * torch.rsqrt(v + self.eps)).to(x.dtype) * self.weight

    class Attn(nn.Module):
        def __init__(self, dim, heads, kind):
            super().__init__()
            self.heads = heads
            self.to_q, self.to_k, self.to_v = (nn.Linear(dim, dim) for _ in range(3))
            self.to_out = nn.ModuleList([nn.Linear(dim, dim), nn.Dropout(0.0)])
            mk = (lambda: nn.LayerNorm(dim // heads, eps=1e-6)) if kind == "layer" else (lambda: RMSNorm(dim))
            self.norm_q, self.norm_k = mk(), mk()

    torch.manual_seed(1)
    heads, D = 2, 64
    for kind, proc, grid, n_text in (("layer", pb.PARO_CogVideoXAttnProcessor2_0(), (2, 4, 8), 32),
                                     ("rms", pb.PARO_WanAttnProcessor2_0(), (2, 4, 12), 0)):
        attn = Attn(heads * D, heads, kind).to(DEV, torch.bfloat16)
        with torch.no_grad():
            for m in (attn.norm_q, attn.norm_k):
                m.weight.add_(0.2 * torch.randn_like(m.weight))
        n_img = grid[0] * grid[1] * grid[2]
        nb = (n_text + n_img + 63) // 64
        proc.grid_fhw = grid
        proc.permute_plan = {"permute": torch.tensor([[4, 2]])}
        proc.sparse_mask = torch.ones(1, 1, heads, nb, nb, dtype=torch.bool, device=DEV)
        hs = torch.randn(1, n_img, heads * D, device=DEV, dtype=torch.bfloat16)
        enc = torch.randn(1, n_text, heads * D, device=DEV, dtype=torch.bfloat16)
        outs = []
        for fuse in (True, False):
            proc.fuse_qk_norm = fuse
            with torch.no_grad():
                o = proc(attn, hs, enc, image_rotary_emb=None) if kind == "layer" else proc(attn, hs, rotary_emb=None)
            outs.append(torch.cat([o[1], o[0]], 1) if kind == "layer" else o)
        pb.check_status()
        cos = torch.nn.functional.cosine_similarity(outs[0].float().flatten(), outs[1].float().flatten(), dim=0)
        assert cos > 0.999, (kind, cos)
        assert pb.QKNorm.from_module(attn.norm_q, heads, D).kind == kind
    assert pb.QKNorm.from_module(nn.Identity(), heads, D) is None

    # composed call against the oracle
    B, H, D, grid, n_text = 1, 2, 128, (2, 6, 10), 8
    N = n_text + grid[0] * grid[1] * grid[2]
    q, k, v, orders = po.make_inputs(B, H, N, D, torch.bfloat16, seed=31)
    mask = po.make_mask(H, (N + 63) // 64, 0.7, seed=31)
    g = torch.Generator().manual_seed(2)
    wq, wk = ((1 + 0.2 * torch.randn(H * D, generator=g)).to(torch.bfloat16) for _ in range(2))
    cos_t, sin_t = po.rope_full_tables(grid, D, "wan")
    want = po.paro_attention(q, k, v, orders, mask, grid, n_text, rope=("complex", cos_t, sin_t),
                             q_norm=("rms", wq, 1e-6), k_norm=("rms", wk, 1e-6))
    got = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(orders), mask.to(DEV), grid_fhw=grid,
                            n_text=n_text, rope=pb.rope_tables(grid, D, "wan"),
                            q_norm=pb.QKNorm("rms", wq.to(DEV), None, 1e-6), k_norm=pb.QKNorm("rms", wk.to(DEV), None, 1e-6))
    pb.check_status()
    assert_close(got, want, "composed path with rms norms")


def test_host_pipelined_matches_device_call():
    """Pinned host tensors through the head-group pipeline give bit-identical results."""
    B, H, D, grid, n_text = 2, 6, 64, (2, 6, 10), 8
    N = n_text + grid[0] * grid[1] * grid[2]
    q, k, v, orders = po.make_inputs(B, H, N, D, torch.bfloat16, seed=21)
    nb = (N + 63) // 64
    mask = po.make_mask(H, nb, 0.6, seed=21, text_blocks=1)
    tabs = pb.rope_tables(grid, D, "cogvideox")
    want = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(orders), mask.to(DEV), grid_fhw=grid,
                             n_text=n_text, rope=tabs)
    pipe = pb.HostPipelinedAttention(orders, mask, (B, H, N, D), torch.bfloat16, grid_fhw=grid, n_text=n_text, rope=tabs,
                                     heads_per_group=4)
    hq, hk = (t.pin_memory() for t in (q, k))
    hv = pb.pinned_like(v.shape, v.dtype)      # pinned pages allocated next to the GPU
    hv.copy_(v)
    assert hv.is_pinned() and not hv.is_cuda
    for _ in range(2):
        got = pipe(hq, hk, hv)
        torch.cuda.synchronize()
        pb.check_status()
        assert torch.equal(got, want.cpu())
    with pytest.raises(ValueError):
        pipe(q, k, v)   # not pinned


def test_plan_store_prefetch_and_roundtrip(tmp_path):
    """Pre-compacted plan store: lists equal the oracle's, prefetching alternates buffers without
    corrupting a plan in use, save/load round trip, and attention through it equals the direct call."""
    T, L, H, nb = 2, 3, 2, 9
    g = torch.Generator().manual_seed(8)
    sparse = torch.rand(T, L, H, nb, nb, generator=g) < 0.4
    sparse[..., torch.arange(nb), torch.arange(nb)] = True
    store = pb.PlanStore(sparse.to(DEV))
    store.save(str(tmp_path / "plan.pt"))
    store2 = pb.PlanStore.load(str(tmp_path / "plan.pt"))
    for st in (store, store2):
        for t in range(T):
            for l in range(L):
                st.prefetch(t, l + 1)
                plan = st.get(t, l)
                # the store pairs q-blocks by overlap: its step counts carry the pairs' q-block ids (+1) in their
                # high halves, and its lists are the oracle's lists of the mask with the rows in that order
                words = plan.sched_cnt.cpu()
                ids = ((words >> 16) & 0xFFFF) - 1
                m = sparse[t, l]
                if (ids >= 0).any():
                    order = ids.view(H, -1)[:, :nb].long()
                    assert all(sorted(order[h].tolist()) == list(range(nb)) for h in range(H))
                    m = torch.gather(m, 1, order.unsqueeze(-1).expand(-1, -1, nb))
                sched, cnt = po.pair_schedule(m)
                assert torch.equal(plan.sched.cpu(), sched) and torch.equal(words & 0xFFFF, cnt)
                assert plan.kept_blocks == int(sparse[t, l].sum())
    N, D = nb * 64 - 20, 64
    q, k, v, orders = po.make_inputs(1, H, N, D, torch.float16, seed=4)
    args = dict(grid_fhw=(1, 1, N))
    want = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(orders), sparse.to(DEV), i_timestep=1, i_block=2, **args)
    got = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(orders), store, i_timestep=1, i_block=2, **args)
    pb.check_status()
    assert torch.equal(got, want)
