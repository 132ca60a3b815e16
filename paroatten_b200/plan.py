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
    row_ptr: torch.Tensor    # int32 [slices*nbq + 1]
    cols: torch.Tensor       # int32 [kept]: ascending k-block ids per q-block
    pair_ptr: torch.Tensor   # int32 [slices*ceil(nbq/2) + 1]
    pair_ent: torch.Tensor   # int32: kb*4 + flags per pair of adjacent q-blocks (merged walk; auxiliary)
    kept_blocks: int         # number of true entries of the mask
    pair_tiles: int          # size of the merged (union) walk over all q-block pairs


def compact_plan(mask: torch.Tensor) -> CompactPlan:
    """mask: bool/uint8 [..., nbq, nbk] on the GPU (leading dims are flattened to slices)."""
    _lib.require_cuda(mask)
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
    return CompactPlan(slices, nbq, nbk, row_ptr, cols[:kept], pair_ptr, pair_ent[:tiles], kept, tiles)


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
            self._cache[key] = compact_plan(self.sparse[key[0], key[1]].to(self.device, non_blocking=True))
        return self._cache[key]


class PermutePlan:
    """The reference's `permute_plan` dict (`'permute'`: `[L, H]` order ids) with cached
    per-layer index tables."""

    def __init__(self, permute_plan, grid: Tuple[int, int, int], device=None):
        self.permute = permute_plan["permute"] if isinstance(permute_plan, dict) else permute_plan
        self.grid = tuple(int(g) for g in grid)
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        self._orders: Dict[int, torch.Tensor] = {}
        self._index: Dict[int, torch.Tensor] = {}

    def orders(self, i_block: int) -> torch.Tensor:
        if i_block not in self._orders:
            self._orders[i_block] = torch.as_tensor(self.permute[i_block]).to(self.device, torch.int32).contiguous()
        return self._orders[i_block]

    def index(self, i_block: int) -> torch.Tensor:
        if i_block not in self._index:
            self._index[i_block] = perm_index(self.orders(i_block), self.grid, self.device)
        return self._index[i_block]
