"""Developer aid: per-role clock trace of ONE CTA of the attention kernel.

    python -m paroatten_b200.trace_attention --workload wan14b_720p --block 9000 --out trace.npy

Builds a second copy of the library with -DPARO_TRACE=<block> (csrc/sparse_attn.cu: that CTA of the
fixed-reference launch stamps clock64() at the hand-off points of its first 160 steps), runs the
attention call three times on the named bench workload, reads the table back and prints where each
role's clocks of a step go.  The shipped library is untouched and contains none of this.

Table layout [role][step][event] (int64 SM clocks, 0 = not reached):
  role 0 / 1   K / V producer       events 2j: waiting for a free stage, 2j+1: copy issued (j = tile of the step)
  role 2 / 3   Q.K^T / P.V issuer   per tile (offset 0 or 4): 0 polling, 1 barriers complete, 3 MMAs and commit issued
                                    (a side-by-side step issued in one burst: 0, 1, 3 = first tile done, 7 = done)
  role 4 + w   softmax warp w       0 waiting for scores, 1 scores ready, 2 scores in registers (S released),
                                    3 exponentials done, 4 previous P.V seen finished, 5 P written and announced
"""
from __future__ import annotations

import argparse
import ctypes
import os
import subprocess
import sys

import numpy as np

ROLES, STEPS, EVENTS = 16, 160, 8


def build_trace_library(block: int) -> str:
    from . import _lib
    out = os.path.join(_lib.HERE, f"libparo_b200_trace{block}.so")
    nvcc = _lib._nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found")
    cmd = [nvcc, *_lib.NVCC_FLAGS, f"-DPARO_TRACE={block}", *[os.path.join(_lib.CSRC, s) for s in _lib.SOURCES], "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return out


def run(workload: str, block: int, library: str) -> np.ndarray:
    from . import _lib
    _lib.LIB_PATH = library          # before the first call into the library
    _lib._stale = lambda: False
    import torch
    import paroatten_b200 as pb
    sys.path.insert(0, os.path.dirname(_lib.HERE))
    from bench import WORKLOADS, make_mask
    wl = WORKLOADS[workload]
    B, H, D = wl["B"], wl["H"], wl["D"]
    F, Hh, W = wl["grid"]
    n_text = wl["n_text"]
    N = n_text + F * Hh * W
    nb = (N + 63) // 64
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    q, k, v = (torch.randn(B, H, N, D, generator=g, device=dev).to(torch.bfloat16) for _ in range(3))
    plan = pb.compact_plan(make_mask(H, nb, wl["density"], 0, (n_text + 63) // 64, wl["window"]).to(dev))
    q8, qs, k8, ks = pb.per_warp_int8(q, k, pb.channel_mean(k), BLKQ=64, WARPQ=32, BLKK=64)
    _, vs, vm, v16 = pb.per_channel_fp8(v, return_16=True)
    table = np.zeros((ROLES, STEPS, EVENTS), dtype=np.int64)
    fn = _lib.lib().paro_debug_trace
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_void_p]
    for rep in range(3):             # two warm-up calls; reading the table clears it, the third call is the one kept
        pb.sparse_attn_quantized(q8, qs, k8, ks, v16, vs, vm, plan, D ** -0.5)
        torch.cuda.synchronize()
        if fn(table.ctypes.data) != 0:
            raise RuntimeError("paro_debug_trace failed")
    pb.check_status()
    return table


def summarise(t: np.ndarray, lo: int = 60, hi: int = 150) -> str:
    """Mean clocks per segment over steps [lo, hi) (pick a range of side-by-side or of shared steps)."""
    hi = min(hi, int((t[2, :, 0] > 0).sum()) - 1)
    lines = [f"steps {lo}..{hi}: Q.K^T issuer period {np.diff(t[2, lo:hi + 1, 0]).mean():.0f} clocks per step"]
    for r, name in ((2, "Q.K^T issuer"), (3, "P.V issuer")):
        x = t[r, lo:hi]
        two = x[:, 5] > 0          # both tiles went through the per-tile path
        if two.any():
            y = x[two]
            lines.append(f"{name}: tile 0 polls {np.mean(y[:, 1] - y[:, 0]):.0f}, issue+commit {np.mean(y[:, 3] - y[:, 1]):.0f}; "
                         f"tile 1 polls {np.mean(y[:, 5] - y[:, 4]):.0f}, issue+commit {np.mean(y[:, 7] - y[:, 5]):.0f}; "
                         f"loop {np.mean((t[r, lo + 1:hi + 1, 0] - x[:, 7])[two]):.0f}")
        burst = (x[:, 5] == 0) & (x[:, 7] > 0)          # side-by-side step issued in one burst
        if burst.any():
            y = x[burst]
            lines.append(f"{name} (burst, {100 * burst.mean():.0f} % of the steps): polls {np.mean(y[:, 1] - y[:, 0]):.0f}, "
                         f"tile 0 {np.mean(y[:, 3] - y[:, 1]):.0f}, tile 1 {np.mean(y[:, 7] - y[:, 3]):.0f}, "
                         f"loop {np.mean((t[r, lo + 1:hi + 1, 0] - x[:, 7])[burst]):.0f}")
        one = (x[:, 5] == 0) & (x[:, 7] == 0) & (x[:, 3] > 0)
        if one.any():
            y = x[one]
            lines.append(f"{name} (one tile): polls {np.mean(y[:, 1] - y[:, 0]):.0f}, issue+commit {np.mean(y[:, 3] - y[:, 1]):.0f}, "
                         f"loop {np.mean((t[r, lo + 1:hi + 1, 0] - x[:, 3])[one]):.0f}")
    for w in range(8):
        steps = np.arange(lo + ((lo & 1) != (w >> 2)), hi, 2)
        x = t[4 + w][steps]
        if not (x[:, 5] > 0).all():
            continue
        lines.append(f"softmax warp {w}: waits for scores {np.mean(x[:, 1] - x[:, 0]):.0f}, TMEM load {np.mean(x[:, 2] - x[:, 1]):.0f}, "
                     f"exponentials {np.mean(x[:, 3] - x[:, 2]):.0f}, waits for previous P.V {np.mean(x[:, 4] - x[:, 3]):.0f}, "
                     f"P store + arrival {np.mean(x[:, 5] - x[:, 4]):.0f}")
    return "\n".join(lines)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--workload", default="wan14b_720p")
    ap.add_argument("--block", type=int, default=9000, help="index of the traced CTA (work item)")
    ap.add_argument("--out", default=None, help="write the raw table here (.npy)")
    ap.add_argument("--steps", default="60:150", help="step range lo:hi of the printed summary")
    a = ap.parse_args()
    table = run(a.workload, a.block, build_trace_library(a.block))
    if a.out:
        np.save(a.out, table)
    lo, hi = (int(x) for x in a.steps.split(":"))
    print(summarise(table, lo, hi))


if __name__ == "__main__":
    main()
