"""Generates tests/golden/refcuda_*.npz: outputs of the REFERENCE's own CUDA kernels (built for
sm_100a by oracle/build_ref.py from the reference's unmodified sources) on seeded inputs.

    python oracle/build_ref.py                         # where the reference checkout is (no GPU needed)
    python tests/golden/make_golden_refcuda.py OUTDIR  # on a machine with a B200; then copy OUTDIR/refcuda_*.npz here

What is called, with the allocation logic of the reference's Python wrappers restated around it
(the wrappers themselves import packages that are not installed):
  quant   paroattention/quant.py:105-180  per_warp_int8  -> _fused.quant_per_warp_int8_cuda (Q, per 32 rows),
                                          _fused.quant_per_block_int8_cuda (K), ..._fuse_sub_mean_cuda (K - km)
          paroattention/quant.py:22-103   per_block_int8 -> _fused.quant_per_block_int8_cuda with sm_scale (Q)
          paroattention/quant.py:224-293  per_channel_fp8 -> transpose_pad_permute_cuda + mean_scale_fuse_quant_cuda
  attn    paroattention/core.py:202-214   per_warp_int8 + qk_int8_sv_f16_accum_f16_attn, all-ones block mask
          and a sequence length that is a multiple of 64 (the only case in which the reference kernel's
          k-block bookkeeping is right, see its skip branches qk_int_sv_f16_cuda_sm80.cu:329-389)
Each quantiser case is produced twice: by the build with the reference's --use_fast_math flag
(setup.py:26) and by the build without it.  The inputs are regenerated from their seeds by the tests.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import paro_oracle as po          # noqa: E402  (input generators only)
from oracle.build_ref import load_built       # noqa: E402

QUANT_CASES = [  # name, B, H, N, D, dtype, seed
    ("a", 1, 2, 520, 64, torch.bfloat16, 21),
    ("b", 2, 2, 1024, 128, torch.float16, 22),
    ("c", 1, 3, 1000, 128, torch.bfloat16, 23),
]
ATTN_CASES = [("d64", 1, 2, 1024, 64, torch.float16, 31), ("d128", 1, 2, 512, 128, torch.bfloat16, 32)]


def ref_per_warp(fused, q, k, km):
    b, h, n, d = q.shape
    q8, k8 = torch.empty_like(q, dtype=torch.int8), torch.empty_like(k, dtype=torch.int8)
    qs = torch.empty(b, h, (n + 63) // 64 * 2, device=q.device, dtype=torch.float32)
    ks = torch.empty(b, h, (n + 63) // 64, device=q.device, dtype=torch.float32)
    fused.quant_per_warp_int8_cuda(q, q8, qs, 64, 32, 1)
    if km is not None:
        fused.quant_per_block_int8_fuse_sub_mean_cuda(k, km, k8, ks, 64, 1)
    else:
        fused.quant_per_block_int8_cuda(k, k8, ks, 64, 1)
    return q8, qs, k8, ks


def ref_per_block_q(fused, q, sm_scale):
    b, h, n, d = q.shape
    q8 = torch.empty_like(q, dtype=torch.int8)
    qs = torch.empty(b, h, (n + 63) // 64, device=q.device, dtype=torch.float32)
    fused.quant_per_block_int8_cuda(q, q8, qs, float(sm_scale * 1.44269504), 64, 1)
    return q8, qs


def ref_per_channel_fp8(fused, v):
    b, h, n, d = v.shape
    npad = (n + 63) // 64 * 64
    vt = torch.empty(b, h, d, npad, dtype=v.dtype, device=v.device)
    fused.transpose_pad_permute_cuda(v, vt, 1)
    v8 = torch.empty(vt.shape, dtype=torch.float8_e4m3fn, device=v.device)
    vs = torch.empty(b, h, d, dtype=torch.float32, device=v.device)
    vm = torch.empty(b, h, d, dtype=torch.float32, device=v.device)
    fused.mean_scale_fuse_quant_cuda(vt, v8, vm, vs, n, 448.0, 1)
    return v8, vs, vm


def main(outdir):
    os.makedirs(outdir, exist_ok=True)
    dev = "cuda"
    builds = {"fast": load_built("_fused"), "ieee": load_built("_fused_ieee")}
    qattn = load_built("_qattn")
    assert all(builds.values()) and qattn is not None, "run oracle/build_ref.py first"
    out = {}
    for name, B, H, N, D, dt, seed in QUANT_CASES:
        q, k, v, _ = po.make_inputs(B, H, N, D, dt, seed=seed)
        km = k.float().mean(dim=2).to(dt)            # [B,H,D] in the input dtype, as quant.py:46-48 expects
        for tag, fused in builds.items():
            qd, kd, vd, kmd = (t.to(dev).contiguous() for t in (q, k, v, km))
            q8, qs, k8, ks = ref_per_warp(fused, qd, kd, None)
            _, _, k8m, ksm = ref_per_warp(fused, qd, kd, kmd)
            q8b, qsb = ref_per_block_q(fused, qd, D ** -0.5)
            v8, vs, vm = ref_per_channel_fp8(fused, vd)
            torch.cuda.synchronize()
            for key, t in (("q8", q8), ("qs", qs), ("k8", k8), ("ks", ks), ("k8m", k8m), ("ksm", ksm), ("q8b", q8b),
                           ("qsb", qsb), ("v8", v8.view(torch.uint8)), ("vs", vs), ("vm", vm)):
                out[f"{name}_{tag}_{key}"] = t.cpu().numpy()
        out[f"{name}_km"] = km.view(torch.int16).numpy()
    np.savez_compressed(os.path.join(outdir, "refcuda_quant.npz"), **out)

    out = {}
    for name, B, H, N, D, dt, seed in ATTN_CASES:
        q, k, v, _ = po.make_inputs(B, H, N, D, dt, seed=seed)
        qd, kd, vd = (t.to(dev).contiguous() for t in (q, k, v))
        q8, qs, k8, ks = ref_per_warp(builds["fast"], qd, kd, None)
        o = torch.empty(B, H, N, D, dtype=dt, device=dev)
        nb = N // 64
        mask = torch.ones(B, H, nb, nb, dtype=torch.bool, device=dev)
        # core.py:207-214: v goes in as fp16, layout HND = 1, per-warp granularity = 2, lse requested
        lse = qattn.qk_int8_sv_f16_accum_f16_attn(q8, k8, vd.to(torch.float16), o, qs, ks, 1, 0, 2, float(D ** -0.5), 1, mask)
        torch.cuda.synchronize()
        for key, t in (("q8", q8), ("qs", qs), ("k8", k8), ("ks", ks), ("o", o.view(torch.int16)),
                       ("lse", lse / 1.44269504)):
            out[f"{name}_{key}"] = t.cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "refcuda_attn.npz"), **out)
    print("wrote", sorted(os.listdir(outdir)))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
