"""Regenerates the fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py --reference /path/to/PAROAtten

Two kinds of fixture are written:

* `perm_*.npz` / `perm_wan_sha256.json` come from the REFERENCE's own Python
  (`paroattention/cogvideox.py` and `paroattention/wan.py`: `permute_qk`,
  `permute_attn_out`) executed on CPU.  The reference modules import packages that
  are not needed for these two functions (diffusers, omegaconf, sageattention and the
  reference's unbuilt CUDA extensions); those imports are satisfied with empty stand-in
  modules, and `torch.tensor(..., device='cuda')` inside `permute_attn_out` is redirected
  to the CPU.  No reference source is copied: the files are loaded from where they lie.
* every other file is produced by the CPU oracle (`oracle/paro_oracle.py`) from seeded
  inputs and pins the oracle against accidental change; the reference has no stored
  expected values for those steps.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import paro_oracle as po  # noqa: E402


class _Anything(types.ModuleType):
    """Module whose every attribute is a throw-away class (enough for `from x import Y`)."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        sub = sys.modules.get(f"{self.__name__}.{name}")
        if sub is not None:
            return sub
        t = type(name, (), {"__init__": lambda self, *a, **k: None})
        setattr(self, name, t)
        return t


class _TorchOnCpu:
    """Forwards to torch, dropping device='cuda' from torch.tensor calls."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def tensor(*a, **k):
        k.pop("device", None)
        return torch.tensor(*a, **k)


def load_reference_module(ref_root: str, name: str):
    for stub in ("omegaconf", "diffusers", "diffusers.models", "diffusers.models.attention",
                 "diffusers.models.embeddings", "diffusers.models.attention_processor",
                 "diffusers.models.modeling_utils", "diffusers.models.modeling_outputs",
                 "diffusers.models.normalization", "diffusers.models.cache_utils",
                 "diffusers.configuration_utils", "diffusers.loaders", "diffusers.utils",
                 "diffusers.callbacks", "sageattention", "sageattention._qattn_sm80",
                 "paroattention._qattn_sm80", "paroattention._fused", "ipdb"):
        sys.modules.setdefault(stub, _Anything(stub))
    pkg = types.ModuleType("paroattention")
    pkg.__path__ = [os.path.join(ref_root, "paroattention")]
    sys.modules["paroattention"] = pkg
    spec = importlib.util.spec_from_file_location(
        f"paroattention.{name}", os.path.join(ref_root, "paroattention", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    mod.torch = _TorchOnCpu()
    return mod


def reference_perm_tables(mod, grid, n_text):
    """Runs the reference's permute_qk / permute_attn_out on tensors whose value is the token
    index, one head per order id 1..5.  Id 0 (identity) is left out: the reference then assigns
    a view onto itself, which torch refuses on CPU; its row is the identity by definition."""
    F, H, W = grid
    n = n_text + F * H * W
    x = torch.arange(n, dtype=torch.float32).reshape(1, 1, n, 1).repeat(1, 5, 1, 2).contiguous()
    plan = {"permute": torch.arange(1, 6).reshape(1, 5)}
    q, k, v = mod.permute_qk(x.clone(), x.clone(), x.clone(), plan, 0)
    assert torch.equal(q, k) and torch.equal(q, v)
    back = mod.permute_attn_out(q.clone(), plan, 0)
    assert torch.equal(back, x), "reference inverse permutation does not undo the forward one"
    assert torch.equal(q[..., 0], q[..., 1])
    ident = torch.arange(n, dtype=torch.float32).reshape(1, n)
    return torch.cat([ident, q[0, :, :, 0]], dim=0).to(torch.int32)  # [6, n]: value at new position = old token


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()

    if os.path.isdir(args.reference):
        cog = load_reference_module(args.reference, "cogvideox")
        t = reference_perm_tables(cog, (13, 30, 45), 226)
        np.savez_compressed(os.path.join(HERE, "perm_cogvideox_ref.npz"), table=t.numpy().astype(np.int32))
        wan = load_reference_module(args.reference, "wan")
        tw = reference_perm_tables(wan, (21, 45, 80), 0)
        with open(os.path.join(HERE, "perm_wan_ref_sha256.json"), "w") as f:
            json.dump({"grid": [21, 45, 80], "n_text": 0,
                       "sha256_int32_table_6xN": po.sha256_of(tw),
                       "first8": tw[:, :8].tolist(), "last8": tw[:, -8:].tolist()}, f, indent=1)
        print("reference permutation fixtures written")
    else:
        print("reference not present: permutation fixtures left as they are")

    # known-answer input of the reference's manual probe (bench/test.py:5-11): rows -256..255
    # repeated over 64 channels, bf16, per_warp_int8(BLKQ=64, WARPQ=32, BLKK=64)
    rows = torch.arange(-256, 256, dtype=torch.bfloat16).unsqueeze(1).repeat(1, 64)
    x = rows.reshape(1, 1, 512, 64)
    q8, qs = po.quant_int8(x, 32)
    k8, ks = po.quant_int8(x, 64)
    np.savez_compressed(os.path.join(HERE, "kat_ramp_int8.npz"), q_col0=q8[0, 0, :, 0].numpy(),
                        q_scale=qs.numpy(), k_col0=k8[0, 0, :, 0].numpy(), k_scale=ks.numpy())

    # the CPU plumbing workload, end to end through the oracle
    cfg = po.CONFIGS["c1_plumbing"]
    F, H_, W = cfg["grid"]
    N = cfg["n_text"] + F * H_ * W
    q, k, v, orders = po.make_inputs(cfg["B"], cfg["H"], N, cfg["D"], cfg["dtype"], seed=0)
    mask = po.make_mask(cfg["H"], (N + 63) // 64, cfg["density"], seed=0)
    qp = po.permute_tokens(q, orders, cfg["grid"], 0)
    kp = po.permute_tokens(k, orders, cfg["grid"], 0)
    vp = po.permute_tokens(v, orders, cfg["grid"], 0)
    km = po.channel_mean(kp, kp.dtype)
    q8, qs = po.quant_int8(qp, 32)
    k8, ks = po.quant_int8(kp, 64, km=km)
    v8, vs, vm = po.quant_v_fp8(vp, smooth=True)
    ptr, cols = po.compact_plan(mask)
    pptr, pent = po.pair_union_plan(mask)
    out, lse = po.paro_attention(q, k, v, orders, mask, cfg["grid"], return_lse=True)
    digests = {n_: po.sha256_of(t_) for n_, t_ in dict(
        q=q, k=k, v=v, mask=mask.to(torch.uint8), q_int8=q8, q_scale=qs, k_int8=k8, k_scale=ks,
        km=km, v_fp8=v8, v_scale=vs, vm=vm, row_ptr=ptr, cols=cols, pair_ptr=pptr, pair_ent=pent,
        out=out).items()}
    with open(os.path.join(HERE, "c1_plumbing_sha256.json"), "w") as f:
        json.dump({"orders": orders, "digests": digests}, f, indent=1)
    np.savez_compressed(os.path.join(HERE, "c1_plumbing_out.npz"),
                        out=out.view(torch.int16).numpy(), lse=lse.numpy())
    print("oracle fixtures written")


if __name__ == "__main__":
    main()
