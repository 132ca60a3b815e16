"""The CPU oracle against the committed fixtures and against first principles."""
import json
import os
from fractions import Fraction

import numpy as np
import pytest
import torch

from oracle import paro_oracle as po

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_perm_index_matches_reference_cogvideox():
    ref = torch.from_numpy(np.load(os.path.join(GOLD, "perm_cogvideox_ref.npz"))["table"])
    n_text = 226
    assert torch.equal(ref[:, :n_text], torch.arange(n_text, dtype=torch.int32).expand(6, -1))
    mine = po.perm_index_table(range(6), (13, 30, 45)) + n_text
    assert torch.equal(ref[:, n_text:], mine)


def test_perm_index_matches_reference_wan():
    with open(os.path.join(GOLD, "perm_wan_ref_sha256.json")) as f:
        g = json.load(f)
    mine = po.perm_index_table(range(6), tuple(g["grid"]))
    assert po.sha256_of(mine) == g["sha256_int32_table_6xN"]
    assert mine[:, :8].tolist() == g["first8"] and mine[:, -8:].tolist() == g["last8"]


@pytest.mark.parametrize("grid,n_text", [((2, 3, 4), 0), ((3, 4, 5), 7)])
def test_permute_roundtrip(grid, n_text):
    n = n_text + grid[0] * grid[1] * grid[2]
    x = torch.randn(2, 6, n, 4)
    y = po.permute_tokens(x, range(6), grid, n_text)
    assert torch.equal(po.inverse_permute_tokens(y, range(6), grid, n_text), x)
    assert torch.equal(y[:, :, :n_text], x[:, :, :n_text])
    assert torch.equal(y[:, 0], x[:, 0])


def test_kat_ramp_fixture_and_exact_rational():
    g = np.load(os.path.join(GOLD, "kat_ramp_int8.npz"))
    rows = torch.arange(-256, 256, dtype=torch.bfloat16).unsqueeze(1).repeat(1, 64).reshape(1, 1, 512, 64)
    q8, qs = po.quant_int8(rows, 32)
    k8, ks = po.quant_int8(rows, 64)
    assert np.array_equal(q8[0, 0, :, 0].numpy(), g["q_col0"]) and np.array_equal(qs.numpy(), g["q_scale"])
    assert np.array_equal(k8[0, 0, :, 0].numpy(), g["k_col0"]) and np.array_equal(ks.numpy(), g["k_scale"])
    # exact rational arithmetic agrees to within one code (fp32 products may sit on the other
    # side of a rounding boundary) and exactly at the block extremes
    vals = list(range(-256, 256))
    for grp, q in ((32, q8), (64, k8)):
        for b0 in range(0, 512, grp):
            amax = max(abs(v) for v in vals[b0:b0 + grp])
            for r in range(b0, b0 + grp):
                exact = Fraction(vals[r] * 127, amax)
                assert abs(int(q[0, 0, r, 0]) - exact) <= Fraction(1, 2) + Fraction(1, 1000)
            assert max(abs(int(q[0, 0, r, 0])) for r in range(b0, b0 + grp)) == 127
    assert torch.equal(qs.flatten()[:1], torch.tensor([256.0]) / 127.0)


def test_quant_int8_tail_and_smoothing():
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(1, 2, 100, 64, generator=g) + 3.0).to(torch.bfloat16)
    km = po.channel_mean(x, x.dtype)
    q, s = po.quant_int8(x, 64, km=km)
    assert q.shape == x.shape and s.shape == (1, 2, 2)
    deq = q.float() * s.repeat_interleave(64, dim=-1)[:, :, :100].unsqueeze(-1) + km.float().unsqueeze(2)
    assert (deq - x.float()).abs().max() <= s.max() * 0.5 + 1e-6
    q32, s32 = po.quant_int8(x, 32)
    assert s32.shape == (1, 2, 4)
    q96, s96 = po.quant_int8(x[:, :, :96], 32)
    assert s96.shape == (1, 2, 4) and s96[0, 0, 3] == torch.tensor(1e-7) / 127  # rows 96..127 all padding
    assert torch.equal(q96, q32[:, :, :96]) and torch.equal(s96[..., :3], s32[..., :3])


def test_quant_v_fp8_layout_and_range():
    g = torch.Generator().manual_seed(2)
    v = (torch.randn(1, 2, 70, 64, generator=g) * 3 + 1).to(torch.float16)
    v8, vs, vm = po.quant_v_fp8(v, smooth=True)
    assert v8.shape == (1, 2, 64, 128) and vs.shape == (1, 2, 64) and vm.shape == (1, 2, 64)
    assert (v8[..., 70:].view(torch.uint8) == 0).all()
    assert v8.float().abs().max() == 448.0
    deq = v8[..., :70].float().transpose(2, 3) * vs.unsqueeze(2) + vm.unsqueeze(2)
    assert ((deq - v.float()).abs() <= 0.0625 * (v.float() - vm.unsqueeze(2)).abs() + 2e-3 * vs.unsqueeze(2) * 448).all()
    z8, zs, _ = po.quant_v_fp8(torch.zeros(1, 1, 64, 64, dtype=torch.float16), smooth=False)
    assert torch.isfinite(z8.float()).all() and (z8.view(torch.uint8) == 0).all()


def test_compact_and_pair_plans():
    m = po.make_mask(3, 7, 0.4, seed=5)
    ptr, cols = po.compact_plan(m)
    flat = m.reshape(-1, 7)
    for r in range(flat.shape[0]):
        assert cols[ptr[r]:ptr[r + 1]].tolist() == flat[r].nonzero().flatten().tolist()
    pptr, pent = po.pair_union_plan(m)
    npairs = 4
    assert pptr.numel() == 3 * npairs + 1
    for s in range(3):
        for p in range(npairs):
            ent = pent[pptr[s * npairs + p]:pptr[s * npairs + p + 1]].tolist()
            want = []
            for kb in range(7):
                f = int(m[s, 2 * p, kb]) + (2 * int(m[s, 2 * p + 1, kb]) if 2 * p + 1 < 7 else 0)
                if f:
                    want.append(kb * 4 + f)
            assert ent == want


def test_attention_dense_matches_sdpa():
    g = torch.Generator().manual_seed(3)
    B, H, N, D = 1, 2, 200, 64
    q = torch.randn(B, H, N, D, generator=g).to(torch.float16)
    k = (torch.randn(B, H, N, D, generator=g) + 1.0).to(torch.float16)
    v = torch.randn(B, H, N, D, generator=g).to(torch.float16)
    mask = torch.ones(H, 4, 4, dtype=torch.bool)
    out, lse = po.paro_attention(q, k, v, [0, 0], mask, (1, 10, 20), return_lse=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    assert po.cosine_per_head(out, ref).min() > 0.999
    s = (q.float() @ k.float().transpose(-1, -2)) * D ** -0.5
    # K smoothing leaves O unchanged up to quantisation noise but shifts every score of a row by
    # q.km, so the LSE is only comparable without it
    out2, lse2 = po.paro_attention(q, k, v, [0, 0], mask, (1, 10, 20), smooth_k=False, return_lse=True)
    assert po.cosine_per_head(out2, ref).min() > 0.995
    assert (lse2 - torch.logsumexp(s, dim=-1)).abs().max() < 0.05


def test_attention_permutation_invariance_when_dense():
    """With every block kept the permutation must cancel out of the result."""
    g = torch.Generator().manual_seed(4)
    q, k, v, _ = po.make_inputs(1, 6, 4 * 4 * 8, 64, torch.bfloat16, seed=4)
    mask = torch.ones(6, 2, 2, dtype=torch.bool)
    a = po.paro_attention(q, k, v, [0] * 6, mask, (4, 4, 8))
    b = po.paro_attention(q, k, v, list(range(6)), mask, (4, 4, 8))
    assert po.cosine_per_head(a, b).min() > 0.9995


def test_rope_tables_and_rotation():
    cos, sin = po.rope_full_tables((2, 3, 4), 64, "cogvideox")
    assert cos.shape == (24, 32) and cos.dtype == torch.float32
    assert po.rope_axis_pairs(64, "cogvideox") == (8, 12, 12)
    assert po.rope_axis_pairs(128, "wan") == (22, 21, 21)
    x = torch.randn(1, 1, 5 + 24, 64).to(torch.bfloat16)
    y = po.apply_rope_real(x, cos, sin, n_text=5)
    assert torch.equal(y[:, :, :5], x[:, :, :5])
    assert torch.equal(y[:, :, 5], x[:, :, 5])  # position (0,0,0): zero angle
    n0 = x[:, :, 5:].float().reshape(1, 1, 24, 32, 2).norm(dim=-1)
    n1 = y[:, :, 5:].float().reshape(1, 1, 24, 32, 2).norm(dim=-1)
    assert (n0 - n1).abs().max() < 0.05
    cw, sw = po.rope_full_tables((2, 3, 4), 128, "wan")
    assert cw.dtype == torch.float64
    xw = torch.randn(1, 1, 24, 128).to(torch.bfloat16)
    yw = po.apply_rope_complex(xw, cw, sw)
    assert yw.shape == xw.shape and yw.dtype == xw.dtype


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_wan_rotation_equals_the_reference_expression(dtype):
    """The Wan rotation is pure torch in the reference (paroattention/wan.py:161-164):
    view_as_complex(x.to(float64).unflatten(3, (-1, 2))) * freqs -> view_as_real -> flatten -> type_as.
    That expression is evaluated here literally, with freqs = cos + i*sin from the oracle's table, on
    more than a million elements; the oracle (four separately rounded fp64 products, which the CUDA
    kernel follows bit for bit) must give the same 16-bit values."""
    grid, D, H = (6, 15, 12), 128, 9
    n_img = grid[0] * grid[1] * grid[2]
    cos, sin = po.rope_full_tables(grid, D, "wan")
    assert cos.dtype == torch.float64 and cos.shape == (n_img, D // 2)
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(1, H, n_img, D, generator=g) * 3).to(dtype)
    assert x.numel() > 1_000_000
    freqs = torch.complex(cos, sin).reshape(1, 1, n_img, D // 2)

    def apply_rotary_emb(hidden_states, freqs):          # wan.py:161-164
        x_rotated = torch.view_as_complex(hidden_states.to(torch.float64).unflatten(3, (-1, 2)))
        x_out = torch.view_as_real(x_rotated * freqs).flatten(3, 4)
        return x_out.type_as(hidden_states)

    assert torch.equal(apply_rotary_emb(x, freqs), po.apply_rope_complex(x, cos, sin))


def test_wan_rope_table_equals_the_reference_construction():
    """WanRotaryPosEmbed (wan.py:482-522): per-axis tables of D/2 - 2*(D//6), D//6, D//6 complex
    frequencies, theta 10000, angles position * theta^(-2i/dim) in fp64 (what diffusers'
    get_1d_rotary_pos_embed(use_real=False, freqs_dtype=float64) computes: polar(1, outer(pos, freq))),
    expanded over the (f, h, w) grid and concatenated.  Rebuilt here with plain torch."""
    grid, D = (3, 4, 5), 128
    h_dim = w_dim = 2 * (D // 6)
    t_dim = D - h_dim - w_dim
    parts = []
    for dim in (t_dim, h_dim, w_dim):
        freq = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float64)[: dim // 2] / dim))
        ang = torch.outer(torch.arange(1024, dtype=torch.float64), freq)
        parts.append(torch.polar(torch.ones_like(ang), ang))
    f, h, w = grid
    ff = parts[0][:f].view(f, 1, 1, -1).expand(f, h, w, -1)
    fh = parts[1][:h].view(1, h, 1, -1).expand(f, h, w, -1)
    fw = parts[2][:w].view(1, 1, w, -1).expand(f, h, w, -1)
    freqs = torch.cat([ff, fh, fw], dim=-1).reshape(f * h * w, -1)
    cos, sin = po.rope_full_tables(grid, D, "wan")
    assert torch.equal(cos, freqs.real) and torch.equal(sin, freqs.imag)


def test_c1_fixture():
    with open(os.path.join(GOLD, "c1_plumbing_sha256.json")) as f:
        g = json.load(f)
    cfg = po.CONFIGS["c1_plumbing"]
    N = 4 * 16 * 16
    q, k, v, orders = po.make_inputs(cfg["B"], cfg["H"], N, cfg["D"], cfg["dtype"], seed=0)
    assert orders == g["orders"]
    mask = po.make_mask(cfg["H"], 16, cfg["density"], seed=0)
    d = g["digests"]
    assert po.sha256_of(q) == d["q"] and po.sha256_of(mask.to(torch.uint8)) == d["mask"]
    qp = po.permute_tokens(q, orders, cfg["grid"])
    q8, qs = po.quant_int8(qp, 32)
    assert po.sha256_of(q8) == d["q_int8"] and po.sha256_of(qs) == d["q_scale"]
    ptr, cols = po.compact_plan(mask)
    assert po.sha256_of(ptr) == d["row_ptr"] and po.sha256_of(cols) == d["cols"]
    out = po.paro_attention(q, k, v, orders, mask, cfg["grid"])
    gold = torch.from_numpy(np.load(os.path.join(GOLD, "c1_plumbing_out.npz"))["out"]).view(torch.float16)
    assert torch.equal(out, gold)


def test_qk_norm_restatement_against_torch():
    """The oracle's normalisations agree with torch's own fp32 formulas up to the rounding of the
    16-bit result (their arithmetic is this project's definition; the diffusers modules the
    processors call are not available to pin them)."""
    torch.manual_seed(3)
    x = (torch.randn(2, 3, 50, 64) * 2 + 0.5).bfloat16()
    w, b = (1 + 0.1 * torch.randn(64)).bfloat16(), (0.1 * torch.randn(64)).bfloat16()
    y = po.layer_norm_heads(x, w, b, 1e-6)
    ref = torch.nn.functional.layer_norm(x.float(), (64,), w.float(), b.float(), 1e-6)
    assert y.dtype == x.dtype and (y.float() - ref).abs().max() <= 2 ** -7 * ref.abs().max()
    w2 = (1 + 0.1 * torch.randn(192)).bfloat16()
    y2 = po.rms_norm_across_heads(x, w2, 1e-6)
    xf = x.float().permute(0, 2, 1, 3).reshape(2, 50, 192)
    ref2 = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w2.float()).reshape(2, 50, 3, 64).permute(0, 2, 1, 3)
    assert (y2.float() - ref2).abs().max() <= 2 ** -6 * ref2.abs().max()
    assert po.apply_qk_norm(x, None) is x
    # the composed oracle takes the norms first
    q, k, v, orders = po.make_inputs(1, 2, 128, 64, torch.float16, seed=4)
    mask = po.make_mask(2, 2, 1.0, seed=0)
    wn = torch.ones(64, dtype=torch.float16)
    a = po.paro_attention(q, k, v, orders, mask, (2, 8, 8), q_norm=("layer", wn, None, 1e-6), k_norm=("layer", wn, None, 1e-6))
    b2 = po.paro_attention(po.layer_norm_heads(q, wn, None, 1e-6), po.layer_norm_heads(k, wn, None, 1e-6), v, orders, mask,
                           (2, 8, 8))
    assert torch.equal(a, b2)


def test_pair_schedule_covers_every_kept_block_once():
    """Shared blocks first (one tile for both q-blocks), then the remaining blocks side by side; each
    q-block's steps are contiguous from 0 and list exactly its kept blocks."""
    for nb, density in ((1, 1.0), (5, 0.5), (8, 0.3), (9, 0.9), (6, 0.0)):
        mask = torch.rand(3, nb, nb, generator=torch.Generator().manual_seed(nb)) < density
        sched, cnt = po.pair_schedule(mask)
        pptr, pent = po.pair_union_plan(mask)
        assert sched.numel() == pent.numel() and cnt.shape == (3 * ((nb + 1) // 2), 2)
        npairs = (nb + 1) // 2
        for r in range(3 * npairs):
            sl, p = divmod(r, npairs)
            words = [w & 0xFFFFFFFF for w in sched[pptr[r]:pptr[r + 1]].tolist()]
            na, nb_ = cnt[r].tolist()
            a = [w & 0xFFFF for w in words[:na]]
            b = [w >> 16 for w in words[:nb_]]
            assert sorted(a) == mask[sl, 2 * p].nonzero().flatten().tolist()
            want_b = mask[sl, 2 * p + 1].nonzero().flatten().tolist() if 2 * p + 1 < nb else []
            assert sorted(b) == want_b
            shared = [w for w in words if (w & 0xFFFF) == (w >> 16) and w != 0xFFFFFFFF]
            assert words[:len(shared)] == shared                      # shared tiles come first
            assert all(w == 0xFFFFFFFF for w in words[max(na, nb_):])  # unused slots
            assert all((w & 0xFFFF) == 0xFFFF for w in words[na:max(na, nb_)])
            assert all((w >> 16) == 0xFFFF for w in words[nb_:max(na, nb_)])
