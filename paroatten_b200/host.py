"""The path for activations that live in HOST memory.

Every (batch, head) is independent, so a call whose q, k, v sit in pinned host memory can be cut
into groups of heads and pipelined: while group c is computed, group c+1 is copied to the device
and the result of group c-1 is copied back (PCIe carries both directions at once).  The per-group
work is the ordinary device path (`core.paro_attention`), so results are bit-identical to a single
device-resident call.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from .core import paro_attention
from .plan import CompactPlan, PermutePlan, compact_plan
from .rope import RopeTables


def _gpu_local_cpus(device) -> Optional[set]:
    """CPUs on the NUMA node the GPU's PCIe slot hangs off (from sysfs), or None when unknown."""
    try:
        pr = torch.cuda.get_device_properties(device)
        path = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0/local_cpulist"
        with open(path) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        return cpus or None
    except Exception:
        return None


def pinned_like(shape, dtype, device=None) -> torch.Tensor:
    """A pinned host tensor whose pages sit on the NUMA node next to the GPU: the calling thread is
    bound to that node's CPUs while the buffer is allocated and first touched, then released again.
    Copies from a far node cross the inter-socket link and lose PCIe bandwidth.  Falls back to a plain
    pinned allocation when the topology cannot be read."""
    import os
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    old = None
    try:
        cpus = _gpu_local_cpus(device)
        if cpus:
            old = os.sched_getaffinity(0)
            usable = cpus & old
            if usable:
                os.sched_setaffinity(0, usable)
            else:
                old = None
    except Exception:
        old = None
    try:
        t = torch.empty(shape, dtype=dtype).pin_memory()
        t.zero_()          # first touch
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)
    return t


def head_groups(H: int, heads_per_group: Optional[int] = None) -> List[Tuple[int, int]]:
    """Cuts H heads into the [h0, h1) groups the pipeline works on.  The host-to-device copies are
    the slowest stage, so what is left after the last copy -- the last group's kernels and its
    copy back -- is pure tail: the groups shrink towards the end (g, ..., g, g-1, ..., 2, 1; a remainder
    goes first, where a short group also shortens the start-up), and the default g gives at least
    four groups so that a rank with few heads still overlaps its stages."""
    H = int(H)
    g = max(1, min(5, (H + 3) // 4)) if heads_per_group is None else max(1, min(int(heads_per_group), H))
    tail = list(range(g - 1, 0, -1))            # g-1, ..., 2, 1
    while tail and sum(tail) > H - min(g, H):   # keep at least one full-size group
        tail.pop(0)
    body = H - sum(tail)
    sizes = ([body % g] if body % g else []) + [g] * (body // g) + tail
    out, h0 = [], 0
    for n in sizes:
        out.append((h0, h0 + n))
        h0 += n
    return out


class HostPipelinedAttention:
    """Set up once per (layer, timestep bin) -- the sparse plan is compacted per head group and
    the staging buffers are allocated here -- then call it with pinned host tensors.

    orders: int order ids [H]; mask: bool [H, nb, nb] (shared by the batch);
    shape = (B, H, N, D) of the host tensors; heads_per_group: heads copied/computed at a time
    (default: see `head_groups`)."""

    def __init__(self, orders, mask: torch.Tensor, shape: Tuple[int, int, int, int], dtype, *, grid_fhw,
                 n_text: int = 0, rope: Optional[RopeTables] = None, heads_per_group: Optional[int] = None, device=None,
                 sm_scale: Optional[float] = None, smooth_k: bool = True, smooth_v: bool = True):
        B, H, N, D = (int(x) for x in shape)
        self.shape, self.dtype = (B, H, N, D), dtype
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.kw = dict(grid_fhw=tuple(int(g) for g in grid_fhw), n_text=int(n_text), rope=rope, sm_scale=sm_scale,
                       smooth_k=smooth_k, smooth_v=smooth_v)
        if mask.dim() != 3 or mask.shape[0] != H:
            raise ValueError("mask must be [H, nb, nb]")
        orders = torch.as_tensor(orders).to(torch.int32)
        if orders.numel() != H:
            raise ValueError("orders must hold one id per head")
        self.groups: List[Tuple[int, int]] = head_groups(H, heads_per_group)
        g = max(h1 - h0 for h0, h1 in self.groups)
        with torch.cuda.device(self.device):
            self.plans: List[CompactPlan] = [compact_plan(mask[h0:h1].to(self.device), pairing="overlap") for h0, h1 in self.groups]
            self.pplans = [PermutePlan({"permute": orders[h0:h1].reshape(1, -1)}, self.kw["grid_fhw"], self.device)
                           for h0, h1 in self.groups]
            # two sets of staging buffers: one being filled while the other is consumed
            self.stage = [[torch.empty(B, g, N, D, dtype=dtype, device=self.device) for _ in range(3)] for _ in range(2)]
            self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.h2d_bytes = 3 * B * H * N * D * torch.empty((), dtype=dtype).element_size()
        self.d2h_bytes = self.h2d_bytes // 3

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None):
        B, H, N, D = self.shape
        for t in (q, k, v):
            if t.is_cuda or tuple(t.shape) != self.shape or t.dtype != self.dtype:
                raise ValueError("q, k, v must be host tensors of the shape and dtype given at set-up")
            if not t.is_pinned():
                raise ValueError("q, k, v must be in pinned host memory (torch.Tensor.pin_memory())")
        if out is None:
            out = pinned_like(self.shape, self.dtype, self.device)
        elif out.is_cuda or tuple(out.shape) != self.shape or not out.is_pinned():
            raise ValueError("out must be a pinned host tensor of the same shape")
        with torch.cuda.device(self.device):
            main = torch.cuda.current_stream()
            start = torch.cuda.Event()
            start.record(main)
            for s in (self.s_in, self.s_comp, self.s_out):
                s.wait_event(start)
            comp_done: List[torch.cuda.Event] = []
            last_out = None
            for c, (h0, h1) in enumerate(self.groups):
                n = h1 - h0
                bufs = [b[:, :n] for b in self.stage[c % 2]]
                with torch.cuda.stream(self.s_in):
                    if c >= 2:
                        self.s_in.wait_event(comp_done[c - 2])       # the staging set is free again
                    for dst, src in zip(bufs, (q, k, v)):
                        for b in range(B):   # each (batch entry, head range) slab is contiguous on both sides
                            dst[b].copy_(src[b, h0:h1], non_blocking=True)
                    in_done = torch.cuda.Event()
                    in_done.record(self.s_in)
                with torch.cuda.stream(self.s_comp):
                    self.s_comp.wait_event(in_done)
                    o = paro_attention(bufs[0], bufs[1], bufs[2], self.pplans[c], self.plans[c], i_block=0, **self.kw)
                    ev = torch.cuda.Event()
                    ev.record(self.s_comp)
                    comp_done.append(ev)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev)
                    o.record_stream(self.s_out)
                    for b in range(B):
                        out[b, h0:h1].copy_(o[b], non_blocking=True)
                    last_out = torch.cuda.Event()
                    last_out.record(self.s_out)
            main.wait_event(last_out)
            main.wait_event(comp_done[-1])
        return out
