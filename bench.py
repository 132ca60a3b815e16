#!/usr/bin/env python
"""Benchmark of the PAROAttention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one sparse-attention call of the named workload (default: Wan2.1-14B 720p shape,
B=1 H=40 D=128 N=75600, block density 0.2): fused RoPE+reorder of Q/K/V, INT8 Q / smoothed K,
FP8 V, block-sparse attention, inverse reorder fused in the store.  With N>1 (launched by
torch.distributed.run) the heads are split across the ranks; no data-path collective is used.
Prints ONE JSON line (rank 0).
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # the reference's three model-shaped workloads
    "wan14b_720p": dict(B=1, H=40, D=128, grid=(21, 45, 80), n_text=0, density=0.2, family="wan", window=0),
    "wan1p3b_480p": dict(B=2, H=12, D=128, grid=(21, 30, 52), n_text=0, density=0.3, family="wan", window=1),
    "cogvideox_5b": dict(B=2, H=48, D=64, grid=(13, 30, 45), n_text=226, density=0.3, family="cogvideox", window=0),
}
METRIC = "effective TOPS per sparse-attn call (kept-block FLOPs only)"
DTYPE = "int8 QK^T (s32 acc), bf16 PV (f32 acc), fp32 softmax"
# DRAM bytes of one attention launch per (batch entry, head, token) at D = 128, from one ncu capture of a
# B=2 H=12 N=32760 launch (read + written = int8 Q, K + 16-bit V + 16-bit O, i.e. the compulsory bytes);
# the traffic of other D = 128 shapes is this figure times B*H*N, to which those bytes are proportional.
ATTN_DRAM_BYTES_PER_BHN_D128 = 588.5e6 / (2 * 12 * 32760)


def config_of(name, wl, world):
    """The `config` object of the JSON line; the same for both arms."""
    F, Hh, W = wl["grid"]
    return {"workload": name, "B": wl["B"], "H": wl["H"], "D": wl["D"], "N": wl["n_text"] + F * Hh * W,
            "grid_fhw": list(wl["grid"]), "n_text": wl["n_text"], "block": 64, "nominal_density": wl["density"],
            "window": wl["window"], "partition": f"{world} x heads", "in_dtype": "bf16",
            "l2": "inputs larger than L2 (no flush needed)"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], src="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, src="fallback")


def make_mask(H, nb, density, seed, text_blocks=0, window=0):
    """Bernoulli(density) block mask shared by the batch; diagonal, text rows/columns and an
    optional local band forced on (stand-in for the calibrated plans, which are not public)."""
    g = torch.Generator().manual_seed(seed)
    m = torch.rand(H, nb, nb, generator=g) < density
    i = torch.arange(nb)
    m[:, i, i] = True
    if text_blocks:
        m[:, :text_blocks, :] = True
        m[:, :, :text_blocks] = True
    if window:
        m |= ((i.reshape(-1, 1) - i.reshape(1, -1)).abs() <= window).unsqueeze(0)
    return m


class ClockSampler:
    """nvidia-smi in the background while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(index)], stdout=subprocess.PIPE, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
def cpu_sample(wl, n_qblocks=512, seed=0):
    """Bounded CPU sample of the same workload through the oracle: ONE head, the first
    `n_qblocks` q-blocks.  Operands are prepared (RoPE, reorder, quantisers) outside the timed
    callable; the callable is the block-sparse attention stage.  Returns (callable, kept_flops,
    description)."""
    from oracle import paro_oracle as po
    F, Hh, W = wl["grid"]
    N = wl["n_text"] + F * Hh * W
    D = wl["D"]
    nb = (N + 63) // 64
    q, k, v, orders = po.make_inputs(1, 1, N, D, torch.bfloat16, seed=seed)
    mask = make_mask(1, nb, wl["density"], seed, (wl["n_text"] + 63) // 64, wl["window"])
    cos, sin = po.rope_full_tables(wl["grid"], D, wl["family"])
    fn = po.apply_rope_real if wl["family"] == "cogvideox" else po.apply_rope_complex
    q, k = fn(q, cos, sin, wl["n_text"]), fn(k, cos, sin, wl["n_text"])
    qp, kp, vp = (po.permute_tokens(t, orders, wl["grid"], wl["n_text"]) for t in (q, k, v))
    km = po.channel_mean(kp, kp.dtype)
    q8, qs = po.quant_int8(qp, 32)
    k8, ks = po.quant_int8(kp, 64, km=km)
    v8, vs, vm = po.quant_v_fp8(vp)
    blocks = list(range(min(n_qblocks, nb)))
    kept = int(mask[0, blocks].sum())
    flops = kept * 4 * 64 * 64 * D

    def run():
        return po.sparse_attention(q8, qs, k8, ks, v8, vs, vm, mask, D ** -0.5, out_dtype=torch.bfloat16,
                                   heads=[0], q_blocks=blocks)
    desc = (f"oracle port, 1 head x {len(blocks)} of {nb} q-blocks ({kept} kept 64x64 blocks), attention stage only, "
            f"fp32 torch CPU")
    return run, flops, desc


def time_cpu(run, steps, warmup):
    for _ in range(warmup):
        run()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        run()
        ts.append(time.perf_counter() - t0)
    return sum(ts) / len(ts)


def run_reference(args, wl_name, wl, rank):
    """The reference has no CPU implementation and its CUDA extensions are sm80-only, so the
    reference arm times the CPU restatement of its algorithm (the oracle) on the host cores."""
    if rank != 0:
        return
    # all host cores this process may use (torchrun sets OMP_NUM_THREADS=1 for multi-rank launches)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    run, flops, desc = cpu_sample(wl)
    sec = time_cpu(run, args.steps, max(1, min(args.warmup, 3)))
    tops = flops / sec / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 QK^T, fp32 softmax and PV (CPU emulation)",
        "data": "synthetic", "config": config_of(wl_name, wl, args.gpus),
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port", "sample": desc},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "each step is the bounded sample, not the whole call",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
class Workload:
    """Device-resident inputs, plans and tables of one workload for this rank's heads."""

    def __init__(self, name, wl, rank, world, dev, permute=True):
        import paroatten_b200 as pb
        from paroatten_b200.dist import head_range
        self.name, self.wl, self.dev = name, wl, dev
        B, H, D = wl["B"], wl["H"], wl["D"]
        F, Hh, W = wl["grid"]
        self.B, self.H, self.D, self.n_text = B, H, D, wl["n_text"]
        self.N = N = self.n_text + F * Hh * W
        self.nb = nb = (N + 63) // 64
        # heads of every batch entry are split contiguously across ranks
        self.h0, self.h1 = head_range(H, rank, world)
        Hl = self.Hl = self.h1 - self.h0
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        self.q = torch.randn(B, Hl, N, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.k = (torch.randn(B, Hl, N, D, generator=gen, device=dev, dtype=torch.float32)
                  + math.sqrt(2.0) * torch.randn(1, Hl, 1, D, generator=gen, device=dev)).to(torch.bfloat16)
        self.v = torch.randn(B, Hl, N, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.orders_all = torch.randint(0, 6, (H,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
        if not permute:
            self.orders_all.zero_()
        self.mask_all = make_mask(H, nb, wl["density"], 0, (self.n_text + 63) // 64, wl["window"])
        self.plan = pb.compact_plan(self.mask_all[self.h0:self.h1].to(dev), pairing="overlap")
        self.pplan = pb.PermutePlan({"permute": self.orders_all[self.h0:self.h1].to(dev).reshape(1, -1)}, wl["grid"], dev)
        self.rope = pb.rope_tables(wl["grid"], D, wl["family"], device=dev)
        self.kept_local = self.plan.kept_blocks * B
        self.kept_total = int(self.mask_all.sum()) * B
        self.flops_block = 4 * 64 * 64 * D
        torch.cuda.synchronize()

    def step(self, q=None, k=None, v=None):
        import paroatten_b200 as pb
        return pb.paro_attention(self.q if q is None else q, self.k if k is None else k, self.v if v is None else v,
                                 self.pplan, self.plan, i_block=0, grid_fhw=self.wl["grid"], n_text=self.n_text,
                                 rope=self.rope)


class Timer:
    """Device time of repeated calls: CUDA events on the launching stream, barrier and synchronise on both
    sides, max over ranks."""

    def __init__(self, dev, world):
        self.dev, self.world = dev, world

    def barrier(self):
        import torch.distributed as dist
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        import torch.distributed as dist
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def timed(self, fn, steps):
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1))


def measure_device_arm(w, timer, steps, warmup):
    """(ms per step of the whole path, ms of the attention launches inside it, kernels launched)."""
    import paroatten_b200 as pb
    from paroatten_b200 import _lib, core
    for _ in range(max(3, warmup)):
        out = w.step()
    pb.check_status(w.dev)
    attn_events = []
    core.set_attention_timing(attn_events)
    launches0 = _lib.lib().paro_launch_count()
    total_ms = timer.timed(w.step, steps)
    launches = _lib.lib().paro_launch_count() - launches0
    core.set_attention_timing(None)
    pb.check_status(w.dev)
    attn_ms = timer.max_over_ranks(statistics.mean(s.elapsed_time(e) for s, e in attn_events))
    return total_ms / steps, attn_ms, int(launches), out


def other_workloads(rank, world, dev, timer, pk, steps=5):
    """The configurations besides the headline one, a few steps each: CogVideoX-5b, Wan-1.3B-480p at three
    densities (kernel TFLOP/s against the same peak as the headline), and the pre-attention passes alone on
    the CogVideoX shape with and without the token permutation (GB/s of algorithmic bytes: three 16-bit
    tensors read, int8 Q, K and 8-bit V written, against the measured copy bandwidth)."""
    import paroatten_b200 as pb
    from paroatten_b200.quant import _quant_int8
    peak = 2.0 * pk["bf16_sustained"]
    res = {}
    cases = [("cogvideox_5b", None), ("wan1p3b_480p", 0.5), ("wan1p3b_480p", 0.3), ("wan1p3b_480p", 0.2)]
    for name, dens in cases:
        wl = dict(WORKLOADS[name])
        if dens is not None:
            wl["density"] = dens
        w = Workload(name, wl, rank, world, dev)
        ms, attn_ms, _, _ = measure_device_arm(w, timer, steps, 3)
        key = name if dens is None else f"{name}@{dens}"
        res[key] = {"ms_per_step": ms, "attention_kernel_ms": attn_ms, "pre_attention_ms": ms - attn_ms,
                    "value_tops": w.kept_total * w.flops_block / (ms * 1e-3) / 1e12,
                    "kernel_tflops": w.kept_local * w.flops_block / (attn_ms * 1e-3) / 1e12,
                    "kernel_frac": w.kept_local * w.flops_block / (attn_ms * 1e-3) / 1e12 / peak,
                    "kept_blocks": w.kept_total, "density": w.kept_total / (w.B * w.H * w.nb * w.nb)}
        del w
        torch.cuda.empty_cache()
    # pre-attention pipeline alone (RoPE + reorder + INT8 Q / smoothed K + FP8 V)
    wl = dict(WORKLOADS["cogvideox_5b"])
    for label, permute in (("pre_attention_permuted", True), ("pre_attention_unpermuted", False)):
        w = Workload("cogvideox_5b", wl, rank, world, dev, permute=permute)
        orders = w.pplan.orders(0) if permute else None

        def prep():
            q8, qs, _ = pb.prep_qk_int8(w.q, orders, wl["grid"], w.n_text, w.rope, group=32)
            kp = pb.rope_permute(w.k, orders, wl["grid"], w.n_text, w.rope)
            k8, ks = _quant_int8(kp, "HND", 64, km=pb.channel_mean(kp))
            v16, vs, vm, _ = pb.prep_v_fp8(w.v, orders, wl["grid"], w.n_text)
            return q8, k8, v16
        for _ in range(3):
            prep()
        ms = timer.timed(prep, steps) / steps
        elems = w.B * w.Hl * w.N * w.D
        algo = 3 * elems * 2 + 3 * elems            # bytes: 16-bit Q, K, V in; int8 Q, K and 8-bit V out
        res[label] = {"ms": ms, "algorithmic_bytes": algo, "gbs": algo / (ms * 1e-3) / 1e9,
                      "frac_of_hbm_peak": algo / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                      "note": "K goes through its reordered 16-bit copy (mean smoothing) and V is written as 16-bit: "
                              "bytes actually moved are higher than the algorithmic figure"}
        del w
        torch.cuda.empty_cache()
    return res


def ulysses_arm(w, out_heads, rank, world, dev, timer, steps):
    """Sequence-sharded activations: every rank starts from ITS token slice of ALL heads, one all-to-all per
    tensor brings it its heads' full sequences, the path runs, one all-to-all returns O to token slices.
    Checked against the head-partition result (which was computed from the same values)."""
    import torch.distributed as dist
    from paroatten_b200 import dist as pdist
    B, H, N, D = w.B, w.H, w.N, w.D
    if H % world or N % world:
        return {"ok": None, "skipped": f"H={H} or N={N} not divisible by {world} ranks"}
    n_loc = N // world

    def to_seq_shards(x_heads):        # [B, H/P, N, D] head shard -> this rank's [B, H, N/P, D] token shard
        return pdist.ulysses_heads_to_seq(x_heads)
    qs, ks, vs = (to_seq_shards(t).contiguous() for t in (w.q, w.k, w.v))   # set-up, not timed

    def run():
        qh, kh, vh = (pdist.ulysses_seq_to_heads(t) for t in (qs, ks, vs))
        o = w.step(qh, kh, vh)
        return pdist.ulysses_heads_to_seq(o)
    for _ in range(2):
        o_seq = run()
    want = pdist.ulysses_heads_to_seq(out_heads)
    ok = bool(torch.equal(o_seq, want))
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ms = timer.timed(run, steps) / steps
    per_tensor = B * H * n_loc * D * 2
    return {"ok": bool(flag.item()), "ms_per_step": ms,
            "value_tops": w.kept_total * w.flops_block / (ms * 1e-3) / 1e12,
            "a2a_bytes_per_rank": 4 * per_tensor * (world - 1) // world, "steps": steps,
            "what": "3 all-to-alls in (q, k, v), path, 1 all-to-all out; compared torch.equal with the head-partition output"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wan14b_720p", choices=sorted(WORKLOADS))
    ap.add_argument("--density", type=float, default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other workloads and the Ulysses arm")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.density is not None:
        wl["density"] = args.density

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, args.workload, wl, rank)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")

    import torch.distributed as dist
    import paroatten_b200 as pb

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    timer = Timer(dev, world)
    pk = peaks()

    w = Workload(args.workload, wl, rank, world, dev)
    B, H, D, N, nb, Hl, n_text = w.B, w.H, w.D, w.N, w.nb, w.Hl, w.n_text

    # ---- device-resident arm ------------------------------------------------------------------
    sampler = ClockSampler(local) if rank == 0 else None
    ms_per_step, attn_ms_max, launches, out = measure_device_arm(w, timer, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    redone = pb.last_redo_count(dev)
    value = w.kept_total * w.flops_block / (ms_per_step * 1e-3) / 1e12

    # ---- end-to-end arm: host buffers, copies inside the timed region ------------------------
    e2e = None
    if not args.no_e2e:
        # the public host-memory entry point: head groups pipelined over three streams, so the copy of
        # group c+1 and the read-back of group c-1 overlap the kernels of group c
        hq, hk, hv = (pb.pinned_like(t_.shape, t_.dtype, dev) for t_ in (w.q, w.k, w.v))   # pages next to the GPU
        for h_, d_ in zip((hq, hk, hv), (w.q, w.k, w.v)):
            h_.copy_(d_)
        ho = pb.pinned_like(out.shape, out.dtype, dev)
        pipe = pb.HostPipelinedAttention(w.orders_all[w.h0:w.h1], w.mask_all[w.h0:w.h1], (B, Hl, N, D), torch.bfloat16,
                                         grid_fhw=wl["grid"], n_text=n_text, rope=w.rope, device=dev)

        def e2e_step():
            pipe(hq, hk, hv, ho)
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(3):
            e2e_step()
        e2e_ms = timer.timed(e2e_step, e2e_steps) / e2e_steps
        pb.check_status(dev)
        same = bool(torch.equal(ho.to(dev), out))
        e2e = {"value": w.kept_total * w.flops_block / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": pipe.h2d_bytes * world, "d2h_bytes_per_step": pipe.d2h_bytes * world,
               "h2d_gbs_per_rank": pipe.h2d_bytes / (e2e_ms * 1e-3) / 1e9,
               "steps": e2e_steps, "api": "paroatten_b200.HostPipelinedAttention (pinned host in, pinned host out)",
               "matches_device_arm": same}
        del hq, hk, hv, ho, pipe

    # ---- sequence-sharded (Ulysses) variant, multi-GPU runs only ------------------------------
    ulysses = None
    if world > 1 and not args.no_extra:
        ulysses = ulysses_arm(w, out, rank, world, dev, timer, max(3, min(args.steps, 5)))

    kept_local, kept_total, flops_block = w.kept_local, w.kept_total, w.flops_block
    plan_info = {"measured_density": kept_total / (B * H * nb * nb), "kept_blocks": kept_total,
                 "walk_steps_rank0": w.plan.steps * B, "tiles_rank0": w.plan.tiles * B,
                 "shared_tiles_rank0": w.plan.shared_tiles * B, "given_back_to_exact_walk_rank0": redone}
    del w, out
    torch.cuda.empty_cache()

    # ---- the other configurations (a few steps each) -----------------------------------------
    extra = None
    if not args.no_extra:
        extra = other_workloads(rank, world, dev, timer, pk)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak_i8 = 2.0 * pk["bf16_sustained"]  # dense INT8/FP8 tensor rate taken as twice the measured bf16 rate
    achieved = kept_local * flops_block / (attn_ms_max * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": config_of(args.workload, wl, world),
        "plan": plan_info,
        "attention_kernel_ms": attn_ms_max,
        "pre_attention_ms": ms_per_step - attn_ms_max,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_i8, "unit": "TFLOP/s",
                     "frac": achieved / peak_i8,
                     "peak_note": f"2 x bf16_tflops_sustained of {pk['src']} peaks (dense INT8/FP8 rate); "
                                  f"the kernel's PV half runs at the 16-bit rate, so its own ceiling is 4/3 x bf16",
                     "traffic": ATTN_DRAM_BYTES_PER_BHN_D128 * B * Hl * N if D == 128 else None},
        "e2e": e2e,
    }
    if ulysses is not None:
        line["ulysses"] = ulysses
    if extra is not None:
        line["workloads"] = extra
    if not args.no_cpu and world == 1:
        run, flops, desc = cpu_sample(wl)
        sec = time_cpu(run, 3, 1)
        line["cpu_baseline"] = {"value": flops / sec / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(),
                                "kind": "port", "sample": desc, "sample_seconds": sec}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
