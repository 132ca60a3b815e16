"""The CPU oracle against outputs of the REFERENCE's own CUDA kernels.

tests/golden/refcuda_*.npz were produced on a B200 by the reference's unmodified sources
(csrc/fused/fused.cu, csrc/qattn/qk_int_sv_f16_cuda_sm80.cu) compiled for sm_100a with
oracle/build_ref.py and run by tests/golden/make_golden_refcuda.py on seeded inputs; the inputs are
rebuilt here from the same seeds.  What is pinned:
  * INT8 Q (per 32 rows), INT8 K (per 64 rows, with and without mean subtraction), INT8 Q with the
    softmax scale folded in: the oracle equals the reference kernel BIT FOR BIT (values and fp32 scales)
    when that kernel is built without --use_fast_math; the reference's own build flag (setup.py:26) turns
    127/amax into an approximate divide, which moves a few values in ten thousand by one step.
  * FP8 V: bytes and scales equal bit for bit where the token count is a multiple of 16; otherwise the
    reference divides the channel sum by the count rounded up to 16 (fused.cu:335,381) and also
    quantises its padding -- the oracle, told to use that divisor, agrees up to the fp32 summation order.
  * Dense attention: cosine and relative L1 within the bars the GPU kernel is held to (the reference
    kernel rounds P to fp16 and accumulates P.V in fp16).
"""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import paro_oracle as po

GOLD = os.path.join(os.path.dirname(__file__), "golden")
QUANT_CASES = [("a", 1, 2, 520, 64, torch.bfloat16, 21), ("b", 2, 2, 1024, 128, torch.float16, 22),
               ("c", 1, 3, 1000, 128, torch.bfloat16, 23)]
ATTN_CASES = [("d64", 1, 2, 1024, 64, torch.float16, 31), ("d128", 1, 2, 512, 128, torch.bfloat16, 32)]
# position i of a 16-token group of the reference's V^T holds token SHUFFLE[i] (fused.cu:287-291; quant.py:231)
SHUFFLE = [0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15]


def sha(t) -> str:
    a = t.numpy() if torch.is_tensor(t) else t
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def gq():
    return np.load(os.path.join(GOLD, "refcuda_quant.npz"))


def reference_layout(v8: torch.Tensor) -> torch.Tensor:
    """The oracle's token-contiguous FP8 bytes [B,H,D,Npad] in the reference's 16-token shuffle."""
    B, H, D, npad = v8.shape
    return v8.view(torch.uint8).reshape(B, H, D, npad // 16, 16)[..., SHUFFLE].reshape(B, H, D, npad)


@pytest.mark.parametrize("case", QUANT_CASES, ids=[c[0] for c in QUANT_CASES])
def test_int8_quantisers_equal_the_reference_kernel(gq, case):
    name, B, H, N, D, dt, seed = case
    q, k, v, _ = po.make_inputs(B, H, N, D, dt, seed=seed)
    km = k.float().mean(dim=2).to(dt)
    mine = {}
    mine["q8"], mine["qs"] = po.quant_int8(q, 32)                                     # quant_per_warp_int8_cuda
    mine["k8"], mine["ks"] = po.quant_int8(k, 64)                                     # quant_per_block_int8_cuda
    mine["k8m"], mine["ksm"] = po.quant_int8(k, 64, km=km)                            # ..._fuse_sub_mean_cuda
    mine["q8b"], mine["qsb"] = po.quant_int8(q, 64, fold_scale=float(np.float32(D ** -0.5 * 1.44269504)))  # with sm_scale
    for key in ("q8", "k8", "k8m", "q8b"):
        assert sha(mine[key]) == bytes(gq[f"{name}_sha_{key}"]).decode(), f"{name} {key}: int8 values differ"
    for key in ("qs", "ks", "ksm", "qsb"):
        assert np.array_equal(mine[key].numpy(), gq[f"{name}_ieee_{key}"]), f"{name} {key}: scales differ"
    # the reference's own --use_fast_math build: a handful of values one step away, scales within one ulp
    for key in ("q8", "k8", "k8m", "q8b"):
        pos, val = gq[f"{name}_fastpos_{key}"], gq[f"{name}_fastval_{key}"]
        flat = mine[key].numpy().reshape(-1)
        assert pos.size <= 1e-3 * flat.size
        assert np.all(np.abs(flat[pos].astype(np.int32) - val.astype(np.int32)) == 1)
    for key in ("qs", "ks", "ksm", "qsb"):
        a, b = mine[key].numpy(), gq[f"{name}_fast_{key}"]
        assert np.max(np.abs(a - b) / a) < 2.5e-7


@pytest.mark.parametrize("case", QUANT_CASES, ids=[c[0] for c in QUANT_CASES])
def test_fp8_v_quantiser_against_the_reference_kernel(gq, case):
    name, B, H, N, D, dt, seed = case
    _, _, v, _ = po.make_inputs(B, H, N, D, dt, seed=seed)
    v8, vs, vm = po.quant_v_fp8(v)
    if N % 16 == 0:
        # same divisor as the reference: bytes and scales bit for bit, the mean up to the summation order
        assert sha(reference_layout(v8)) == bytes(gq[f"{name}_sha_v8"]).decode()
        assert np.array_equal(vs.numpy(), gq[f"{name}_ieee_vs"])
        assert np.max(np.abs(vm.numpy() - gq[f"{name}_ieee_vm"])) < 1e-6
    else:
        # the reference's divisor (token count rounded up to 16) handed to the oracle
        n16 = (N + 15) // 16 * 16
        v8r, vsr, vmr = po.quant_v_fp8(v, mean_divisor=n16)
        assert np.max(np.abs(vmr.numpy() - gq[f"{name}_ieee_vm"])) < 1e-6
        assert np.max(np.abs(vsr.numpy() - gq[f"{name}_ieee_vs"]) / vsr.numpy()) < 1e-6
        if f"{name}_ieee_v8" in gq.files:
            ref = torch.from_numpy(gq[f"{name}_ieee_v8"])
            got = reference_layout(v8r)
            npad = got.shape[-1]
            tok = torch.arange(npad).reshape(npad // 16, 16)
            tok = (tok // 16 * 16 + torch.tensor(SHUFFLE)).reshape(-1)       # token held at each position
            valid = tok < N
            differ = (ref[..., valid] != got[..., valid]).float().mean().item()
            assert differ < 2e-3      # mean rounded differently in its last bit moves a few roundings
    assert gq[f"{name}_fastpos_v8"].size <= 1e-3 * v8.numel()


@pytest.mark.parametrize("case", ATTN_CASES, ids=[c[0] for c in ATTN_CASES])
def test_dense_attention_against_the_reference_kernel(case):
    """qk_int8_sv_f16_accum_f16_attn (all-ones block mask) on per_warp_int8 operands and fp16 V: the
    oracle's attention stage with V passed through unquantised (scale 1, no mean)."""
    name, B, H, N, D, dt, seed = case
    g = np.load(os.path.join(GOLD, "refcuda_attn.npz"))
    q, k, v, _ = po.make_inputs(B, H, N, D, dt, seed=seed)
    q8, qs = po.quant_int8(q, 32)
    k8, ks = po.quant_int8(k, 64)
    vt = v.to(torch.float16).float().transpose(2, 3).contiguous()
    nb = N // 64
    want, want_lse = po.sparse_attention(q8, qs, k8, ks, vt, torch.ones(B, H, D), None,
                                         torch.ones(H, nb, nb, dtype=torch.bool), D ** -0.5, out_dtype=dt,
                                         return_lse=True)
    ref = torch.from_numpy(g[f"{name}_o_rows4"]).view(dt)
    assert po.cosine_per_head(ref, want[:, :, ::4]).min().item() >= 0.9995
    assert po.rel_l1_per_head(ref, want[:, :, ::4]).max().item() <= 1e-2
    # (the reference run quantised Q, K with its fast-math build: a few int8 values one step away from the
    # oracle's move single rows' LSE by up to a few 1e-3; the typical row agrees to 1e-4)
    d = (torch.from_numpy(g[f"{name}_lse"]) - want_lse).abs()
    assert d.max().item() < 1e-2 and d.median().item() < 1e-4
