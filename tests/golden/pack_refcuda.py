"""Packs the raw output of make_golden_refcuda.py (two .npz of several MB) into the small fixtures that
are committed: refcuda_quant.npz / refcuda_attn.npz in this directory.

    python tests/golden/pack_refcuda.py RAW_DIR

Kept per quantiser case: sha256 digests of every tensor the reference build WITHOUT --use_fast_math
produced (the tests rebuild the inputs from their seeds and compare digests), the fp32 scale / mean
tensors of both builds in full (they are small), and for the build WITH the reference's own
--use_fast_math flag the positions and values where its int8 / fp8 output differs from the other build.
FP8 V bytes are kept in full for the one ragged case that is small and as a digest for the others.
Attention: every 4th output row and the full LSE."""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
INT_KEYS = ("q8", "k8", "k8m", "q8b", "v8")
F32_KEYS = ("qs", "ks", "ksm", "qsb", "vs", "vm")


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main(raw_dir):
    g = np.load(os.path.join(raw_dir, "refcuda_quant.npz"))
    cases = sorted({k.split("_")[0] for k in g.files})
    out = {}
    for c in cases:
        for key in INT_KEYS:
            ieee, fast = g[f"{c}_ieee_{key}"], g[f"{c}_fast_{key}"]
            out[f"{c}_sha_{key}"] = np.frombuffer(sha(ieee).encode(), dtype=np.uint8)
            out[f"{c}_shape_{key}"] = np.array(ieee.shape, dtype=np.int64)
            pos = np.flatnonzero(ieee.reshape(-1) != fast.reshape(-1)).astype(np.int64)
            out[f"{c}_fastpos_{key}"] = pos
            out[f"{c}_fastval_{key}"] = fast.reshape(-1)[pos]
        for key in F32_KEYS:
            out[f"{c}_ieee_{key}"] = g[f"{c}_ieee_{key}"]
            out[f"{c}_fast_{key}"] = g[f"{c}_fast_{key}"]
        if g[f"{c}_ieee_v8"].size <= 100_000:
            out[f"{c}_ieee_v8"] = g[f"{c}_ieee_v8"]
    np.savez_compressed(os.path.join(HERE, "refcuda_quant.npz"), **out)

    g = np.load(os.path.join(raw_dir, "refcuda_attn.npz"))
    out = {}
    for c in sorted({k.split("_")[0] for k in g.files}):
        out[f"{c}_o_rows4"] = g[f"{c}_o"][:, :, ::4, :]
        out[f"{c}_lse"] = g[f"{c}_lse"]
    np.savez_compressed(os.path.join(HERE, "refcuda_attn.npz"), **out)
    for f in ("refcuda_quant.npz", "refcuda_attn.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
