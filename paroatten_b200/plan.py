"""Permutation tables and compacted sparse plans (device resident, built once per plan slice).

The reference keeps a boolean mask `[timestep_bin, layer, head, nb, nb]` and lets the kernel
test one byte per k-block (example/pipeline_cogvideox.py:75-102,
csrc/qattn/qk_int_sv_f16_cuda_sm80.cu:222,268).  Here each mask slice is compacted once into
ascending walk lists that the attention kernel follows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib


def perm_index(order_ids, grid: Tuple[int, int, int], device=None) -> torch.Tensor:
    """[H, F*H*W] int32 table, idx[h][new] = old, for per-head axis-order ids 0..5
    (FHW, FWH, HWF, HFW, WHF, WFH; paroattention/cogvideox.py:38-45)."""
    if not torch.is_tensor(order_ids):
        order_ids = torch.tensor(list(order_ids), dtype=torch.int32)
    if device is None:
        device = order_ids.device if order_ids.is_cuda else torch.device("cuda")
    ids = order_ids.to(device=device, dtype=torch.int32).contiguous()
    _lib.require_cuda(ids)
    F, H, W = (int(g) for g in grid)
    with torch.cuda.device(ids.device):
        out = torch.empty(ids.numel(), F * H * W, dtype=torch.int32, device=ids.device)
        _lib.check(_lib.lib().paro_build_perm_index(ids.data_ptr(), ids.numel(), F, H, W, out.data_ptr(),
                                                    _lib.stream_ptr()))
    return out


@dataclass
class CompactPlan:
    """Walk lists of one mask slice set [slices, nbq, nbk]."""
    slices: int
    nbq: int
    nbk: int
    row_ptr: Optional[torch.Tensor]    # int32 [slices*nbq + 1]                      (CSR form of the mask;
    cols: Optional[torch.Tensor]       # int32 [kept]: ascending k-block ids per q-block   not read by the kernel)
    pair_ptr: torch.Tensor             # int32 [slices*ceil(nbq/2) + 1]: offsets of a pair's merged list and schedule
    pair_ent: Optional[torch.Tensor]   # int32: kb*4 + flags per pair of adjacent q-blocks (merged list; auxiliary)
    kept_blocks: int         # number of true entries of the mask
    pair_tiles: int          # size of the merged (union) lists over all q-block pairs
    sched: Optional[torch.Tensor] = None       # int32 [pair_tiles]: kbA | kbB << 16 per step (what the kernel walks)
    sched_cnt: Optional[torch.Tensor] = None   # int32 [slices*ceil(nbq/2), 2]: steps of the pair's two q-blocks
    # pairing="overlap": the q-blocks each pair is made of, int32 [slices*ceil(nbq/2), 2] (-1: none); row_ptr/cols,
    # pair_ent and sched are then those of the mask with its rows in that order.  None: pair p = q-blocks 2p, 2p+1.
    pair_q: Optional[torch.Tensor] = None
    sched_cnt_kernel: Optional[torch.Tensor] = None   # what the kernel reads: sched_cnt | (pair_q + 1) << 16

    @property
    def steps(self) -> int:
        """Steps of the kernel's walk over all pairs (a step is one or two MMA groups)."""
        return int((self.sched_cnt & 0xFFFF).max(dim=1).values.sum().item())

    @property
    def tiles(self) -> int:
        """K/V tiles the kernel loads = MMA groups of each kind it issues: a tile shared by both
        q-blocks of a pair counts once."""
        c = (self.sched_cnt & 0xFFFF).long()
        n = int(c.sum().item())
        return n - self.shared_tiles

    @property
    def shared_tiles(self) -> int:
        """Tiles that serve both q-blocks of their pair."""
        return int((self.pair_ent & 3).eq(3).sum().item()) if self.pair_ent is not None else -1


def apply_empty_heads(mask: torch.Tensor, empty: Optional[torch.Tensor], n_text_blocks: int = 0) -> torch.Tensor:
    """mask [..., H, nbq, nbk] with the video-to-video blocks of the heads flagged in `empty` (bool [H])
    switched off; the first n_text_blocks rows and columns (text tokens) stay as they are.  This is the mask
    multiply of the reference's pipeline set-up (example/pipeline_cogvideox.py:76-77) applied before the text
    padding.  Returns `mask` itself when no head is flagged."""
    if empty is None:
        return mask
    empty = torch.as_tensor(empty).to(mask.device).bool()
    if empty.numel() != mask.shape[-3]:
        raise ValueError(f"empty-head flags must hold one entry per head ({mask.shape[-3]})")
    if not bool(empty.any()):
        return mask
    out = mask.clone()
    t = int(n_text_blocks)
    region = out[..., t:, t:]
    region[..., empty, :, :] = False if out.dtype == torch.bool else 0
    return out


def validate_plan(plan: "CompactPlan") -> None:
    """Checks the walk lists of a plan on the GPU (paro_plan_validate) and raises ValueError naming the first
    fault.  Lists produced by compact_plan in this process are correct by construction; this is for lists
    that come from a file or from other code.  Synchronises the current stream."""
    _lib.require_cuda(plan.pair_ptr, plan.sched, plan.sched_cnt)
    dev = plan.pair_ptr.device
    with torch.cuda.device(dev):
        report = torch.zeros(4, dtype=torch.int32, device=dev)
        _lib.check(_lib.lib().paro_plan_validate(
            plan.pair_ptr.data_ptr(), plan.sched.data_ptr(), plan.sched_cnt.data_ptr(), plan.slices, plan.nbq, plan.nbk,
            plan.sched.numel(), report.data_ptr(), _lib.stream_ptr()))


def pair_rows_by_overlap(m: torch.Tensor) -> torch.Tensor:
    """m: uint8/bool [slices, nbq, nbk] on the GPU.  Returns int64 [slices, nbq]: an order of the q-blocks
    in which rows 2p and 2p+1 are good partners -- the kernel walks the UNION of a pair's two lists, a
    k-block both keep costs one tile instead of two.  Greedy: the first q-block not yet paired takes the
    free q-block it shares most k-blocks with (ties: the lowest index).  Deterministic; nbq/2 rounds of a
    few small kernels, vectorised over the slices."""
    S, nbq, _ = m.shape
    mf = m.to(torch.float32)
    ov = torch.bmm(mf, mf.transpose(1, 2))                    # shared k-blocks of every two q-blocks
    idx = torch.arange(S, device=m.device)
    free = torch.ones(S, nbq, dtype=torch.bool, device=m.device)
    order = torch.empty(S, nbq, dtype=torch.int64, device=m.device)
    for pidx in range(nbq // 2):
        i = free.to(torch.uint8).argmax(dim=1)                # first free row of each slice
        free[idx, i] = False
        cand = torch.where(free, ov[idx, i], torch.full_like(ov[idx, i], -1.0))
        j = cand.argmax(dim=1)
        free[idx, j] = False
        order[:, 2 * pidx] = i
        order[:, 2 * pidx + 1] = j
    if nbq % 2:
        order[:, nbq - 1] = free.to(torch.uint8).argmax(dim=1)
    return order


def compact_plan(mask: torch.Tensor, validate: Optional[bool] = None, pairing: str = "adjacent") -> CompactPlan:
    """mask: bool/uint8 [..., nbq, nbk] on the GPU (leading dims are flattened to slices).
    validate: run validate_plan on the result (default: only when the environment variable
    PARO_DEBUG_PLANS is set to a non-empty value other than 0).
    pairing: "adjacent" -- work item p is q-blocks 2p and 2p+1; "overlap" -- q-blocks are paired by the
    k-blocks they share (pair_rows_by_overlap), kept for the slices (heads) where that needs fewer tiles than adjacency."""
    if pairing not in ("adjacent", "overlap"):
        raise ValueError(f"unknown pairing {pairing!r}")
    if pairing == "overlap":
        _lib.require_cuda(mask)
        nbq0, nbk0 = int(mask.shape[-2]), int(mask.shape[-1])
        m0 = mask.reshape(-1, nbq0, nbk0)
        m0 = (m0 if m0.dtype in (torch.uint8, torch.bool) else (m0 != 0)).contiguous().view(torch.uint8)
        base = compact_plan(m0, validate=validate)
        if nbq0 < 4 or nbq0 >= 0xFFFF:
            return base
        npairs0 = (nbq0 + 1) // 2
        order = pair_rows_by_overlap(m0)
        plan = compact_plan(torch.gather(m0, 1, order.unsqueeze(-1).expand(-1, -1, nbk0)), validate=validate)
        # The choice is made slice by slice (head by head), so that a head's plan -- and with it the order
        # in which its rows accumulate -- does not depend on which other heads are compacted with it.
        ends = torch.arange(0, m0.shape[0] + 1, device=m0.device) * npairs0
        per_slice = lambda pl: (pl.pair_ptr[ends[1:]] - pl.pair_ptr[ends[:-1]])
        better = per_slice(plan) < per_slice(base)
        if not bool(better.any()):
            return base
        if not bool(better.all()):
            ident = torch.arange(nbq0, device=m0.device).expand_as(order)
            order = torch.where(better.unsqueeze(1), order, ident)
            plan = compact_plan(torch.gather(m0, 1, order.unsqueeze(-1).expand(-1, -1, nbk0)), validate=validate)
        pq = torch.full((m0.shape[0], 2 * npairs0), -1, dtype=torch.int32, device=m0.device)
        pq[:, :nbq0] = order.to(torch.int32)
        plan.pair_q = pq.view(-1, 2).contiguous()
        plan.sched_cnt_kernel = (plan.sched_cnt | ((plan.pair_q + 1) << 16)).contiguous()
        return plan
    _lib.require_cuda(mask)
    if validate is None:
        import os
        validate = os.environ.get("PARO_DEBUG_PLANS", "0") not in ("", "0")
    if mask.dim() < 2:
        raise ValueError("mask must have at least 2 dimensions")
    nbq, nbk = int(mask.shape[-2]), int(mask.shape[-1])
    m = mask.reshape(-1, nbq, nbk)
    m = (m if m.dtype in (torch.uint8, torch.bool) else (m != 0)).contiguous().view(torch.uint8)
    slices = m.shape[0]
    npairs = (nbq + 1) // 2
    L = _lib.lib()
    with torch.cuda.device(m.device):
        row_ptr = torch.empty(slices * nbq + 1, dtype=torch.int32, device=m.device)
        pair_ptr = torch.empty(slices * npairs + 1, dtype=torch.int32, device=m.device)
        s = _lib.stream_ptr()
        _lib.check(L.paro_plan_count(m.data_ptr(), slices, nbq, nbk, row_ptr.data_ptr(), pair_ptr.data_ptr(), s))
        kept, tiles = int(row_ptr[-1].item()), int(pair_ptr[-1].item())
        cols = torch.empty(max(kept, 1), dtype=torch.int32, device=m.device)
        pair_ent = torch.empty(max(tiles, 1), dtype=torch.int32, device=m.device)
        _lib.check(L.paro_plan_fill(m.data_ptr(), slices, nbq, nbk, row_ptr.data_ptr(), cols.data_ptr(), kept,
                                    pair_ptr.data_ptr(), pair_ent.data_ptr(), tiles, s))
        sched = torch.empty(max(tiles, 1), dtype=torch.int32, device=m.device)
        sched_cnt = torch.empty(slices * npairs, 2, dtype=torch.int32, device=m.device)
        _lib.check(L.paro_plan_schedule(pair_ptr.data_ptr(), pair_ent.data_ptr(), slices, nbq, nbk, sched.data_ptr(),
                                        sched_cnt.data_ptr(), s))
    plan = CompactPlan(slices, nbq, nbk, row_ptr, cols[:kept], pair_ptr, pair_ent[:tiles], kept, tiles,
                       sched[:tiles], sched_cnt)
    if validate:
        validate_plan(plan)
    return plan


class SparsePlan:
    """The reference's `sparse_plan['sparse']` tensor `[T, L, H, nb, nb]` with lazily compacted
    and cached slices; `get(i_timestep, i_block)` replaces `sparse_mask[i_timestep, i_block]`
    (paroattention/cogvideox.py:193)."""

    def __init__(self, sparse: torch.Tensor, device=None):
        if sparse.dim() != 5:
            raise ValueError("sparse plan must be [timestep_bins, layers, heads, nb, nb]")
        self.sparse = sparse
        self.device = torch.device(device) if device is not None else (
            sparse.device if sparse.is_cuda else torch.device("cuda"))
        self._cache: Dict[Tuple[int, int], CompactPlan] = {}

    def get(self, i_timestep: int, i_block: int) -> CompactPlan:
        key = (int(i_timestep), int(i_block))
        if key not in self._cache:
            self._cache[key] = compact_plan(self.sparse[key[0], key[1]].to(self.device, non_blocking=True),
                                            pairing="overlap")
        return self._cache[key]


class PermutePlan:
    """The reference's `permute_plan` dict (`'permute'`: `[L, H]` order ids) with cached
    per-layer index tables."""

    def __init__(self, permute_plan, grid: Tuple[int, int, int], device=None):
        self.permute = permute_plan["permute"] if isinstance(permute_plan, dict) else permute_plan
        self._empty = permute_plan.get("empty") if isinstance(permute_plan, dict) else None
        self.grid = tuple(int(g) for g in grid)
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        self._orders: Dict[int, torch.Tensor] = {}
        self._index: Dict[int, torch.Tensor] = {}

    def orders(self, i_block: int) -> torch.Tensor:
        if i_block not in self._orders:
            self._orders[i_block] = torch.as_tensor(self.permute[i_block]).to(self.device, torch.int32).contiguous()
        return self._orders[i_block]

    def empty(self, i_block: int) -> Optional[torch.Tensor]:
        """bool [H] flags of the layer's empty heads (the plan's 'empty' entry), or None."""
        if self._empty is None:
            return None
        return torch.as_tensor(self._empty[i_block]).to(self.device).bool()

    def index(self, i_block: int) -> torch.Tensor:
        if i_block not in self._index:
            self._index[i_block] = perm_index(self.orders(i_block), self.grid, self.device)
        return self._index[i_block]


class PlanStore:
    """Every (timestep bin, layer) slice of a sparse plan `[T, L, H, nb, nb]`, compacted ONCE and kept
    as walk lists in pinned host memory; the lists of the layer that runs next are streamed to the
    GPU on a side stream while the current layer computes.

    Replaces the reference's `SparseMaskPrefetchStream` (paroattention/prefetch_utils.py:34-59), which
    double-buffers the boolean mask itself (nb*nb bytes per head and layer: 55.9 MB at Wan-14B-720p);
    the compacted lists are 4 bytes per KEPT block (9 MB at density 0.2).  `get` has the call shape of
    `SparsePlan.get`, so a processor can use either."""

    def __init__(self, sparse: Optional[torch.Tensor] = None, device=None, _lists=None, empty: Optional[torch.Tensor] = None,
                 n_text_blocks: int = 0):
        """empty: the permute plan's 'empty' flags, bool [L, H]; flagged heads lose their video-to-video
        blocks (apply_empty_heads) before compaction."""
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.kept = {}
        if _lists is not None:
            self.meta, self.lists, self.kept = _lists
        else:
            if sparse.dim() != 5:
                raise ValueError("sparse plan must be [timestep_bins, layers, heads, nb, nb]")
            T, L, H, nbq, nbk = (int(x) for x in sparse.shape)
            self.meta = dict(T=T, L=L, H=H, nbq=nbq, nbk=nbk)
            self.lists = {}
            for t in range(T):
                for l in range(L):
                    p = compact_plan(apply_empty_heads(sparse[t, l].to(self.device),
                                                       None if empty is None else empty[l], n_text_blocks),
                                     pairing="overlap")
                    # (the step counts are stored in the form the kernel reads: with the pairs' q-block ids
                    # in their high halves when the q-blocks were paired by overlap)
                    cnt = p.sched_cnt_kernel if p.sched_cnt_kernel is not None else p.sched_cnt
                    self.lists[(t, l)] = tuple(x.cpu().pin_memory() for x in (p.pair_ptr, p.sched, cnt))
                    self.kept[(t, l)] = p.kept_blocks
        cap = max(c.numel() for _, c, _ in self.lists.values())
        prows = self.meta["H"] * ((self.meta["nbq"] + 1) // 2)
        with torch.cuda.device(self.device):
            self._buf = [(torch.empty(prows + 1, dtype=torch.int32, device=self.device),
                          torch.empty(max(cap, 1), dtype=torch.int32, device=self.device),
                          torch.empty(prows, 2, dtype=torch.int32, device=self.device)) for _ in range(2)]
            self._stream = torch.cuda.Stream(self.device)
        self._slot = {}          # key -> (buffer index, event of its copy)
        self._next = 0

    def keys(self):
        return sorted(self.lists)

    def prefetch(self, i_timestep: int, i_block: int) -> None:
        """Starts the host-to-device copy of one slice's lists into the buffer that `get` did not
        hand out last.  The copy waits for everything enqueued so far on the current stream (the
        kernels that may still read that buffer) and overlaps with whatever is enqueued afterwards."""
        key = (int(i_timestep), int(i_block))
        if key in self._slot or key not in self.lists:
            return
        b = self._next
        self._next ^= 1
        self._slot = {k: v for k, v in self._slot.items() if v[0] != b}
        pair_ptr, sched, sched_cnt = self.lists[key]
        with torch.cuda.device(self.device):
            fence = torch.cuda.Event()
            fence.record(torch.cuda.current_stream())
            self._stream.wait_event(fence)
            with torch.cuda.stream(self._stream):
                self._buf[b][0].copy_(pair_ptr, non_blocking=True)
                self._buf[b][1][:sched.numel()].copy_(sched, non_blocking=True)
                self._buf[b][2].copy_(sched_cnt, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._stream)
        self._slot[key] = (b, ev)

    def get(self, i_timestep: int, i_block: int) -> CompactPlan:
        """The slice's plan, usable on the current stream (waits for its copy if one is in flight).
        It stays valid until the second `prefetch` after this call."""
        key = (int(i_timestep), int(i_block))
        if key not in self.lists:
            raise KeyError(f"the plan store holds no slice for (timestep bin {key[0]}, layer {key[1]}); "
                           f"it has {self.meta['T']} bins x {self.meta['L']} layers")
        if key not in self._slot:
            self.prefetch(*key)
        b, ev = self._slot[key]
        self._next = b ^ 1       # the next prefetch goes to the other buffer
        n = self.lists[key][1].numel()
        with torch.cuda.device(self.device):
            torch.cuda.current_stream().wait_event(ev)
        m = self.meta
        return CompactPlan(m["H"], m["nbq"], m["nbk"], None, None, self._buf[b][0], None, int(self.kept.get(key, 0)),
                           int(n), self._buf[b][1][:n], self._buf[b][2])

    def save(self, path: str) -> None:
        torch.save({"meta": self.meta, "kept": {f"{t},{l}": n for (t, l), n in self.kept.items()},
                    "lists": {f"{t},{l}": tuple(x.clone() for x in v) for (t, l), v in self.lists.items()}}, path)

    @classmethod
    def load(cls, path: str, device=None) -> "PlanStore":
        blob = torch.load(path, map_location="cpu")
        key = lambda k: tuple(int(x) for x in k.split(","))
        lists = {key(k): tuple(x.pin_memory() for x in v) for k, v in blob["lists"].items()}
        kept = {key(k): int(n) for k, n in blob.get("kept", {}).items()}
        store = cls(device=device, _lists=(blob["meta"], lists, kept))
        store.validate()          # lists from a file go to the kernel only after the device-side check
        return store

    def validate(self) -> None:
        """Runs validate_plan on every stored slice (uploads each once); raises ValueError on the first fault."""
        m = self.meta
        prows = m["H"] * ((m["nbq"] + 1) // 2)
        for key_, (pair_ptr, sched, sched_cnt) in sorted(self.lists.items()):
            if pair_ptr.numel() != prows + 1 or sched_cnt.numel() != 2 * prows or pair_ptr.dtype != torch.int32:
                raise ValueError(f"sparse plan slice {key_}: list sizes do not match H={m['H']}, nbq={m['nbq']}")
            dev_lists = [x.to(self.device) for x in (pair_ptr, sched, sched_cnt)]
            try:
                validate_plan(CompactPlan(m["H"], m["nbq"], m["nbk"], None, None, dev_lists[0], None, 0, sched.numel(),
                                          dev_lists[1], dev_lists[2]))
            except ValueError as e:
                raise ValueError(f"sparse plan slice {key_}: {e}") from None
