"""Walk-list validation, the bounded-wait expiry path, merging of partial attention results and the
permute plan's empty heads."""
import pytest
import torch

import paroatten_b200 as pb
from paroatten_b200 import _lib, core
from oracle import paro_oracle as po

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, RL1_MAX = 0.9995, 1e-2


def assert_close(got, want, what=""):
    c = po.cosine_per_head(got.cpu(), want).min().item()
    r = po.rel_l1_per_head(got.cpu(), want).max().item()
    assert c >= COS_MIN and r <= RL1_MAX, f"{what}: min cosine {c:.6f}, max rel-L1 {r:.3e}"


def _plan(H=3, nb=9, density=0.5, seed=3):
    mask = po.make_mask(H, nb, density, seed=seed)
    return mask, pb.compact_plan(mask.to(DEV))


def _with(plan, **kw):
    import dataclasses
    return dataclasses.replace(plan, **kw)


def test_validator_accepts_built_plans_and_names_the_fault_in_malformed_ones():
    """Malformed lists go to the validator only, never to the attention kernel."""
    for nb, density in ((1, 1.0), (9, 0.5), (16, 0.2), (7, 0.0)):
        _, plan = _plan(nb=nb, density=density, seed=nb)
        pb.validate_plan(plan)
    assert pb.compact_plan(po.make_mask(2, 5, 0.5, seed=1).to(DEV), validate=True).slices == 2
    mask, plan = _plan()
    npairs = (plan.nbq + 1) // 2
    cnt, sched, ptr = plan.sched_cnt.clone(), plan.sched.clone(), plan.pair_ptr.clone()
    # a pair whose upper q-block has own blocks, i.e. free slots after its steps
    free = ((ptr[1:] - ptr[:-1]) - cnt[:, 0] > 0).nonzero().flatten()
    r = int(free[0])
    # (1) one step too many for a q-block: the slot holds the filler, not a block id
    bad = cnt.clone(); bad[r, 0] += 1
    with pytest.raises(ValueError, match="k-block id out of range"):
        pb.validate_plan(_with(plan, sched_cnt=bad))
    # (2) more steps than the pair has slots
    bad = cnt.clone(); bad[r, 1] = int(ptr[r + 1] - ptr[r]) + 1
    with pytest.raises(ValueError, match="step count"):
        pb.validate_plan(_with(plan, sched_cnt=bad))
    # (3) a k-block id beyond the sequence
    bad = sched.clone(); bad[int(ptr[r])] = (int(bad[int(ptr[r])]) & ~0xFFFF) | (plan.nbk + 3)
    with pytest.raises(ValueError, match="out of range"):
        pb.validate_plan(_with(plan, sched=bad))
    # (4) offsets that go backwards
    bad = ptr.clone(); bad[2] = bad[1] - 1
    with pytest.raises(ValueError, match="offsets"):
        pb.validate_plan(_with(plan, pair_ptr=bad))
    # (5) a repeated block inside a section
    rows = ((cnt[:, 0] >= 2) & (cnt[:, 1] >= 2)).nonzero().flatten()
    r2 = int(rows[0]); e0 = int(ptr[r2])
    bad = sched.clone(); bad[e0 + 1] = bad[e0]
    with pytest.raises(ValueError, match="ascending"):
        pb.validate_plan(_with(plan, sched=bad))
    # (6) steps for a q-block past the end (odd block count: the last pair has no second q-block)
    bad = cnt.clone(); bad[npairs - 1, 1] = 1
    with pytest.raises(ValueError):
        pb.validate_plan(_with(plan, sched_cnt=bad))


def test_plan_store_rejects_a_tampered_file(tmp_path):
    T, L, H, nb = 1, 2, 2, 6
    sparse = torch.rand(T, L, H, nb, nb, generator=torch.Generator().manual_seed(5)) < 0.5
    store = pb.PlanStore(sparse.to(DEV))
    path = str(tmp_path / "plan.pt")
    store.save(path)
    pb.PlanStore.load(path)
    blob = torch.load(path)
    ptr, sched, cnt = blob["lists"]["0,1"]
    sched[0] = (int(sched[0]) & ~0xFFFF) | 0x7000
    torch.save(blob, path)
    with pytest.raises(ValueError, match=r"slice .0, 1."):
        pb.PlanStore.load(path)
    with pytest.raises(KeyError, match="holds no slice"):
        store.get(3, 0)


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """A plan that claims one more step for a q-block than its schedule holds (the slot is the filler, so
    neither issuer ever produces that step's scores): the softmax warps of that q-block wait for scores that
    never come, the bounded wait gives up after its limit (~0.2 s), the work item is reported through the
    status words, every role of the CTA leaves, later CTAs and the second launch drain, and the next call
    with the intact plan is correct again.  Nothing faults or hangs: this is the wait's own time-out."""
    B, H, N, D = 1, 2, 1024, 128
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.bfloat16, seed=9)
    mask = po.make_mask(H, N // 64, 0.5, seed=9)
    q8, qs = po.quant_int8(q, 32); k8, ks = po.quant_int8(k, 64, km=po.channel_mean(k, k.dtype)); v8, vs, vm = po.quant_v_fp8(v)
    args = [t.to(DEV) for t in (q8, qs, k8, ks, v8.to(torch.bfloat16), vs, vm)]
    plan = pb.compact_plan(mask.to(DEV))
    want = po.sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask, D ** -0.5, out_dtype=torch.bfloat16)
    ptr, cnt = plan.pair_ptr, plan.sched_cnt
    free = ((ptr[1:] - ptr[:-1]) - cnt[:, 0] > 0).nonzero().flatten()
    r = int(free[0]); step = int(cnt[r, 0])
    bad = cnt.clone(); bad[r, 0] += 1
    import dataclasses
    broken = dataclasses.replace(plan, sched_cnt=bad)
    with pytest.raises(ValueError):
        pb.validate_plan(broken)                          # the validator would have caught it
    pb.check_status()
    pb.sparse_attn_quantized(*args, broken, D ** -0.5)    # handed to the kernel all the same
    words = torch.zeros(4, dtype=torch.int32)
    rc = _lib.lib().paro_status_poll(core._status_words(torch.device(DEV, torch.cuda.current_device())).data_ptr(),
                                     words.data_ptr(), _lib.stream_ptr())
    assert rc == _lib.PARO_ETIMEOUT
    assert words[0].item() == _lib.PARO_ETIMEOUT and words[1].item() == 6      # role 6: softmax waiting for scores
    assert words[2].item() == r and words[3].item() == step                   # that pair, that step
    with pytest.raises(_lib.ParoError, match="wait expired"):
        pb.sparse_attn_quantized(*args, plan, D ** -0.5)  # the next call notices, clears the words and raises
    got = pb.sparse_attn_quantized(*args, plan, D ** -0.5)
    pb.check_status()
    assert_close(got, want, "call after the time-out")


@pytest.mark.parametrize("D,N,dtype,layout", [(128, 1024, torch.bfloat16, "HND"), (64, 840, torch.float16, "NHD")])
def test_partial_results_over_split_key_ranges_merge_to_the_full_result(D, N, dtype, layout):
    """What return_lse is for (reference core.py:55-57): attention over the first and over the second half of
    the key blocks, merged, equals attention over all of them.  Some rows keep blocks in one half only."""
    B, H = 2, 3
    q, k, v, orders = po.make_inputs(B, H, N, D, dtype, seed=N)
    nb = (N + 63) // 64
    mask = po.make_mask(H, nb, 0.35, seed=4)
    mask[:, 2, nb // 2:] = False           # q-block 2 keeps nothing in the second half
    mask[:, 5, :nb // 2] = False; mask[:, 5, nb - 1] = True
    ma, mb = mask.clone(), mask.clone()
    ma[:, :, nb // 2:] = False
    mb[:, :, :nb // 2] = False
    grid = (1, 1, N)
    ids = torch.zeros(H, dtype=torch.int32)
    cvt = (lambda t: t.to(DEV)) if layout == "HND" else (lambda t: t.transpose(1, 2).contiguous().to(DEV))
    call = lambda m: pb.paro_attention(cvt(q), cvt(k), cvt(v), ids, m.to(DEV), grid_fhw=grid, return_lse=True,
                                       tensor_layout=layout)
    (oa, la), (ob, lb), (o, l) = call(ma), call(mb), call(mask)
    om, lm = pb.merge_attention_states(oa, la, ob, lb, tensor_layout=layout)
    pb.check_status()
    hnd = (lambda t: t) if layout == "HND" else (lambda t: t.transpose(1, 2))
    assert_close(hnd(om), hnd(o).cpu(), "merged vs unsplit")
    fin = torch.isfinite(l)
    assert torch.equal(torch.isfinite(lm), fin) and (lm[fin] - l[fin]).abs().max().item() < 2e-3
    want, want_lse = po.paro_attention(q, k, v, [0] * H, mask, grid, return_lse=True)
    assert_close(hnd(om), want, "merged vs oracle")
    # the oracle's own merge
    mo, ml = po.merge_attention_states(hnd(oa).cpu(), la.cpu(), hnd(ob).cpu(), lb.cpu())
    assert_close(hnd(om), mo, "kernel merge vs oracle merge")
    assert (ml[fin.cpu()] - lm.cpu()[fin.cpu()]).abs().max().item() < 1e-5
    assert torch.equal(hnd(om)[:, :, 128:192], hnd(oa)[:, :, 128:192])     # q-block 2: only side a has blocks


def test_empty_heads_of_the_permute_plan():
    """permute_plan['empty'] (reference: bench/check.py:116-128): 'zero' drops the video-to-video blocks of the
    flagged heads, 'uniform' (no text tokens) gives them the mean of V."""
    B, H, D, grid, n_text = 2, 4, 64, (2, 6, 10), 70
    N = n_text + grid[0] * grid[1] * grid[2]
    q, k, v, orders = po.make_inputs(B, H, N, D, torch.bfloat16, seed=5)
    nb = (N + 63) // 64
    tb = (n_text + 63) // 64
    mask = po.make_mask(H, nb, 0.5, seed=5, text_blocks=tb)
    empty = torch.tensor([[False, True, False, True]])
    pplan = {"permute": torch.tensor([orders]), "empty": empty}
    got = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), pplan, mask.to(DEV), grid_fhw=grid, n_text=n_text)
    pb.check_status()
    want = po.paro_attention(q, k, v, orders, mask, grid, n_text=n_text, empty=empty[0], empty_mode="zero")
    assert_close(got, want, "empty heads, zero")
    m2 = pb.apply_empty_heads(mask.to(DEV), empty[0], tb).cpu()
    assert torch.equal(m2[[0, 2]], mask[[0, 2]]) and not m2[1, tb:, tb:].any() and torch.equal(m2[1, :tb], mask[1, :tb])
    store = pb.PlanStore(mask.reshape(1, 1, H, nb, nb).to(DEV), empty=empty, n_text_blocks=tb)
    got2 = pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), {"permute": torch.tensor([orders])}, store,
                             grid_fhw=grid, n_text=n_text)
    assert torch.equal(got2, got)
    # uniform: sequences without text
    N2 = grid[0] * grid[1] * grid[2]
    q2, k2, v2, orders2 = po.make_inputs(B, H, N2, D, torch.float16, seed=6)
    mask2 = po.make_mask(H, (N2 + 63) // 64, 0.5, seed=6)
    pplan2 = {"permute": torch.tensor([orders2]), "empty": empty}
    got3, lse3 = pb.paro_attention(q2.to(DEV), k2.to(DEV), v2.to(DEV), pplan2, mask2.to(DEV), grid_fhw=grid,
                                   empty_head_mode="uniform", return_lse=True)
    want3 = po.paro_attention(q2, k2, v2, orders2, mask2, grid, empty=empty[0], empty_mode="uniform")
    assert_close(got3[:, [0, 2]], want3[:, [0, 2]], "kept heads")
    assert (got3[:, [1, 3]].float().cpu() - want3[:, [1, 3]].float()).abs().max().item() < 2e-2
    zero = pb.paro_attention(q2.to(DEV), k2.to(DEV), v2.to(DEV), pplan2, mask2.to(DEV), grid_fhw=grid)
    assert (zero[:, [1, 3]] == 0).all()
    with pytest.raises(NotImplementedError):
        pb.paro_attention(q.to(DEV), k.to(DEV), v.to(DEV), pplan, mask.to(DEV), grid_fhw=grid, n_text=n_text,
                          empty_head_mode="uniform")


def test_processors_apply_the_embedding_they_are_given_and_prefetch_plans():
    """Processor path with a real mask, rotation and a PlanStore: the rotary embedding passed in is what
    gets applied (same output as the composed call with tables for that grid; another theta changes the
    output; an embedding that is no 3-D table over the grid raises), and the next layer's lists are
    prefetched while a layer runs."""
    import torch.nn as nn

    class Attn(nn.Module):
        def __init__(self, dim, heads):
            super().__init__()
            self.heads = heads
            self.to_q, self.to_k, self.to_v = (nn.Linear(dim, dim) for _ in range(3))
            self.to_out = nn.ModuleList([nn.Identity(), nn.Dropout(0.0)])
            self.norm_q = self.norm_k = None

    torch.manual_seed(0)
    heads, D, grid, n_text, L = 4, 64, (3, 6, 10), 50, 2
    n_img = grid[0] * grid[1] * grid[2]
    N = n_text + n_img
    nb, tb = (N + 63) // 64, (n_text + 63) // 64
    attn = Attn(heads * D, heads).to(DEV, torch.bfloat16)
    sparse = torch.stack([po.make_mask(heads, nb, 0.5, seed=l, text_blocks=tb) for l in range(L)]).unsqueeze(0)
    orders = torch.tensor([[4, 2, 0, 5], [1, 1, 3, 2]])
    hs = torch.randn(1, n_img, heads * D, device=DEV, dtype=torch.bfloat16)
    enc = torch.randn(1, n_text, heads * D, device=DEV, dtype=torch.bfloat16)
    cos, sin = po.rope_full_tables(grid, D, "cogvideox")                     # [n_img, D/2]
    emb = tuple(t.repeat_interleave(2, dim=1).to(DEV) for t in (cos, sin))   # diffusers' real layout [n_img, D]
    store = pb.PlanStore(sparse.to(DEV))
    outs = []
    for layer in range(L):
        proc = pb.PARO_CogVideoXAttnProcessor2_0()
        proc.grid_fhw, proc.permute_plan, proc.sparse_mask = grid, {"permute": orders}, store
        proc.i_block, proc.i_timestep = layer, 0
        with torch.no_grad():
            h_out, e_out = proc(attn, hs, enc, image_rotary_emb=emb)
            x = torch.cat([enc, hs], 1)
            q, k, v = (f(x).view(1, N, heads, D) for f in (attn.to_q, attn.to_k, attn.to_v))
        direct = pb.paro_attention(q, k, v, {"permute": orders}, sparse.to(DEV), i_block=layer, i_timestep=0, grid_fhw=grid,
                                   n_text=n_text, rope=pb.rope_tables(grid, D, "cogvideox"), tensor_layout="NHD")
        got = torch.cat([e_out, h_out], 1)
        assert torch.equal(got, direct.reshape(1, N, heads * D)), f"layer {layer}"
        want = po.paro_attention(*(t.transpose(1, 2).cpu() for t in (q, k, v)), orders[layer].tolist(), sparse[0, layer],
                                 grid, n_text=n_text, rope=("real", cos, sin))
        assert_close(got.view(1, N, heads, D).transpose(1, 2), want, f"layer {layer} vs oracle")
        if layer + 1 < L:
            assert (0, layer + 1) in store._slot          # already on its way to the GPU
        outs.append(got)
    pb.check_status()
    # another theta: different angles, different output
    cos2, sin2 = po.rope_full_tables(grid, D, "cogvideox", theta=500.0)
    emb2 = tuple(t.repeat_interleave(2, dim=1).to(DEV) for t in (cos2, sin2))
    with torch.no_grad():
        h2, e2 = proc(attn, hs, enc, image_rotary_emb=emb2)
    assert not torch.equal(torch.cat([e2, h2], 1), outs[-1])
    want2 = po.paro_attention(*(t.transpose(1, 2).cpu() for t in (q, k, v)), orders[L - 1].tolist(), sparse[0, L - 1],
                              grid, n_text=n_text, rope=("real", cos2, sin2))
    assert_close(torch.cat([e2, h2], 1).view(1, N, heads, D).transpose(1, 2), want2, "theta 500")
    # an embedding for another grid is refused
    cos3, sin3 = po.rope_full_tables((3, 10, 6), D, "cogvideox")
    with pytest.raises(ValueError, match="per-axis"):
        proc(attn, hs, enc, image_rotary_emb=tuple(t.repeat_interleave(2, dim=1).to(DEV) for t in (cos3, sin3)))
    # Wan: complex embedding [1, 1, N, D/2]
    wan = pb.PARO_WanAttnProcessor2_0()
    wgrid = (2, 6, 10)
    wn = wgrid[0] * wgrid[1] * wgrid[2]
    wan.grid_fhw, wan.permute_plan = wgrid, {"permute": orders}
    wmask = po.make_mask(heads, (wn + 63) // 64, 0.6, seed=3)
    wan.sparse_mask = wmask.reshape(1, 1, heads, *wmask.shape[1:]).to(DEV)
    wc, ws = po.rope_full_tables(wgrid, D, "wan")
    whs = torch.randn(1, wn, heads * D, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        wout = wan(attn, whs, rotary_emb=torch.complex(wc, ws).reshape(1, 1, wn, D // 2).to(DEV))
        q, k, v = (f(whs).view(1, wn, heads, D) for f in (attn.to_q, attn.to_k, attn.to_v))
    wwant = po.paro_attention(*(t.transpose(1, 2).cpu() for t in (q, k, v)), orders[0].tolist(), wmask, wgrid,
                              rope=("complex", wc, ws))
    assert_close(wout.view(1, wn, heads, D).transpose(1, 2), wwant, "wan processor vs oracle")


@pytest.mark.gpu
@pytest.mark.parametrize("D,N,H,density,n_text", [(128, 64 * 23 + 17, 3, 0.35, 0), (64, 64 * 16, 2, 0.5, 0),
                                                   (64, 226 + 4 * 6 * 10, 2, 0.4, 226)])
def test_pairs_chosen_by_overlap(D, N, H, density, n_text):
    """compact_plan(pairing="overlap"): every q-block is in exactly one pair, the paired plan needs no more
    tiles than the adjacent one, and the kernel's output on it equals the adjacent plan's within rounding
    of the accumulation order (the oracle comparison on such plans: test_kernel_on_oracle_quantised_operands)."""
    g = torch.Generator().manual_seed(11)
    nb = (N + 63) // 64
    mask = po.make_mask(H, nb, density, seed=7, text_blocks=(n_text + 63) // 64)
    adj = pb.compact_plan(mask.to(DEV))
    ovl = pb.compact_plan(mask.to(DEV), pairing="overlap", validate=True)
    assert ovl.pair_tiles <= adj.pair_tiles and ovl.kept_blocks == adj.kept_blocks
    if ovl.pair_q is not None:
        pq = ovl.pair_q.view(H, -1).cpu()
        for h in range(H):
            ids = pq[h][pq[h] >= 0]
            assert sorted(ids.tolist()) == list(range(nb))
    q = torch.randn(1, H, N, D, generator=g).to(torch.bfloat16).to(DEV)
    k = (torch.randn(1, H, N, D, generator=g) + 1.4 * torch.randn(1, H, 1, D, generator=g)).to(torch.bfloat16).to(DEV)
    v = torch.randn(1, H, N, D, generator=g).to(torch.bfloat16).to(DEV)
    q8, qs, k8, ks = pb.per_warp_int8(q, k, pb.channel_mean(k), BLKQ=64, WARPQ=32, BLKK=64)
    _, vs, vm, v16 = pb.per_channel_fp8(v, return_16=True)
    outs = {}
    for name, plan in (("adjacent", adj), ("overlap", ovl)):
        for mode in ("fast", "exact"):
            o, lse = pb.sparse_attn_quantized(q8, qs, k8, ks, v16, vs, vm, plan, D ** -0.5, mode=mode, return_lse=True)
            outs[name, mode] = (o.float().cpu(), lse.cpu())
    pb.check_status()
    for mode in ("fast", "exact"):
        a, b = outs["adjacent", mode], outs["overlap", mode]
        assert po.cosine_per_head(b[0], a[0]).min().item() > 0.99999
        assert torch.allclose(b[1], a[1], atol=2e-3, rtol=0)
