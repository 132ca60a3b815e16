"""Sparse-attention entry points (reference: paroattention/core.py)."""
from __future__ import annotations

from typing import Any, Optional, Sequence, Tuple, Union

import torch
import torch.nn.functional as F

from . import _lib
from .plan import (CompactPlan, PermutePlan, PlanStore, SparsePlan, apply_empty_heads, compact_plan, perm_index)
from .quant import (_hnd, _quant_int8, channel_mean, per_channel_fp8, per_warp_int8, per_block_int8, prep_qk_int8,
                    prep_v_fp8)
from .rope import RopeTables, rope_permute

_status = {}
_status_mirror = {}   # device index -> pinned host copy of the status words, refreshed after every launch
_redo = {}       # (device index, stream handle) -> work space of the fast walk
_timing_sink = None  # optional list receiving (start, end) CUDA events around each attention launch


def set_attention_timing(sink) -> None:
    """Pass a list to have every attention launch bracketed by CUDA events on the launching
    stream (appended as (start, end) pairs); pass None to switch it off."""
    global _timing_sink
    _timing_sink = sink


def _status_words(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[key]


def _redo_space(device: torch.device, B: int, H: int, N: int) -> torch.Tensor:
    """Work space of the attention call's fast walk (the list of work items it hands to the exact
    walk), one per device and stream: calls on different streams must not share it."""
    need = (_lib.lib().paro_sparse_attn_redo_bytes(B, H, N) + 3) // 4
    key = (device.index if device.index is not None else torch.cuda.current_device(), _lib.stream_ptr())
    buf = _redo.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(need, dtype=torch.int32, device=device)
        _redo[key] = buf
    return buf


def last_redo_count(device=None) -> int:
    """How many work items (pairs of q-blocks) of the latest attention call on the current stream the
    fast walk handed to the exact walk (synchronises)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _lib.stream_ptr())
    buf = _redo.get(key)
    return 0 if buf is None else int(buf[0].item())


def check_status(device=None) -> None:
    """Synchronises the current stream and raises if an attention launch on `device` gave up a
    bounded wait (the launch's output is then invalid).  The status words are cleared when it raises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    words = _status_words(device)
    with torch.cuda.device(device):
        rc = _lib.lib().paro_status_poll(words.data_ptr(), None, _lib.stream_ptr())
        if rc != _lib.PARO_OK:
            words.zero_()
            key = device.index if device.index is not None else torch.cuda.current_device()
            if key in _status_mirror:
                _status_mirror[key].zero_()
        _lib.check(rc)


def _mirror(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status_mirror:
        _status_mirror[key] = torch.zeros(4, dtype=torch.int32).pin_memory()
    return _status_mirror[key]


def _raise_if_earlier_launch_failed(device: torch.device) -> None:
    """Every attention launch is followed by an asynchronous copy of the status words into pinned host
    memory; each new call looks at that copy first (no synchronisation).  A launch that gave up a wait
    therefore stops the caller at the next attention call at the latest, instead of every later launch
    returning at once and leaving its output unwritten."""
    m = _mirror(device)
    if int(m[0]) != 0:
        check_status(device)      # synchronises, clears the words and raises with the waiter's position


def sparse_attn_quantized(q_int8, q_scale, k_int8, k_scale, v16, v_scale, vm, plan: CompactPlan, sm_scale: float,
                          out_dtype=torch.bfloat16, q_group: int = 32, inv_index: Optional[torch.Tensor] = None,
                          n_text: int = 0, return_lse: bool = False, out: Optional[torch.Tensor] = None,
                          out_layout: str = "HND", mode: str = "fast"):
    """The attention kernel on already quantised operands (HND, contiguous).
    q_int8/k_int8 int8 [B,H,N,D]; q_scale [B,H,nb*(64/q_group)]; k_scale [B,H,nb];
    v16 bf16 [B,H,D,ceil64(N)] holding e4m3 values; v_scale / vm fp32 [B,H,D] (vm may be None).
    mode: "fast" (fixed reference exponent per row, exact walk only for the work items that need
    it) or "exact" (running row maximum everywhere).
    inv_index: int32 [H, N-n_text] table from plan.perm_index -- when given, the inverse token
    permutation is applied as rows are stored.  Returns O [B,H,N,D] (or [B,N,H,D] when
    out_layout="NHD") and, if asked, LSE [B,H,N] (natural log, in output token order)."""
    _lib.require_cuda(q_int8, k_int8, v16, q_scale, k_scale, v_scale, vm, inv_index)
    if mode not in ("fast", "exact"):
        raise ValueError(f"unknown mode {mode!r}")
    B, H, N, D = q_int8.shape
    nb = (N + 63) // 64
    if plan.nbq != nb or plan.nbk != nb:
        raise ValueError(f"sparse plan is {plan.nbq}x{plan.nbk} blocks but the sequence has {nb}")
    if plan.slices not in (H, B * H):
        raise ValueError(f"sparse plan has {plan.slices} slices; expected H={H} or B*H={B * H}")
    for t, name in ((q_int8, "q_int8"), (k_int8, "k_int8"), (v16, "v16")):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    if q_int8.dtype != torch.int8 or k_int8.dtype != torch.int8 or tuple(k_int8.shape) != (B, H, N, D):
        raise ValueError("q_int8 and k_int8 must be int8 [B,H,N,D]")
    if tuple(v16.shape) != (B, H, D, nb * 64) or v16.dtype != torch.bfloat16:
        raise ValueError("v16 must be bf16 [B,H,D,ceil64(N)]")
    if q_group not in (32, 64):
        raise ValueError("q_group must be 32 or 64")
    for t, name, shape in ((q_scale, "q_scale", (B, H, nb * (64 // q_group))), (k_scale, "k_scale", (B, H, nb)),
                           (v_scale, "v_scale", (B, H, D)), (vm, "vm", (B, H, D))):
        if t is None and name == "vm":
            continue
        if t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous fp32 {list(shape)}")
    if inv_index is not None and (inv_index.dtype != torch.int32 or tuple(inv_index.shape) != (H, N - n_text)
                                  or not inv_index.is_contiguous()):
        raise ValueError(f"inv_index must be contiguous int32 [H, N - n_text] = [{H}, {N - n_text}]")
    dev = q_int8.device
    _raise_if_earlier_launch_failed(dev)
    with torch.cuda.device(dev):
        if out is None:
            shape = (B, H, N, D) if out_layout == "HND" else (B, N, H, D)
            out = torch.empty(shape, dtype=out_dtype, device=dev)
        ov = out if out_layout == "HND" else out.transpose(1, 2)
        if tuple(ov.shape) != (B, H, N, D) or ov.stride(-1) != 1:
            raise ValueError("out has the wrong shape or a strided last dimension")
        lse = torch.empty(B, H, N, dtype=torch.float32, device=dev) if return_lse else None
        sink = _timing_sink
        if sink is not None:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        redo = _redo_space(dev, B, H, N) if mode != "exact" else None
        _lib.check(_lib.lib().paro_sparse_attn(
            q_int8.data_ptr(), k_int8.data_ptr(), v16.data_ptr(), q_scale.data_ptr(), int(q_group),
            k_scale.data_ptr(), v_scale.data_ptr(), _lib.ptr(vm), plan.pair_ptr.data_ptr(), plan.sched.data_ptr(),
            (plan.sched_cnt_kernel if plan.sched_cnt_kernel is not None else plan.sched_cnt).data_ptr(),
            plan.slices, _lib.ptr(inv_index), int(n_text), out.data_ptr(), _lib.dtype_code(out.dtype),
            ov.stride(0), ov.stride(1), ov.stride(2), _lib.ptr(lse), B, H, N, D, float(sm_scale),
            _lib.ATTN_FAST if mode == "fast" else _lib.ATTN_EXACT, _lib.ptr(redo),
            redo.numel() * 4 if redo is not None else 0, _status_words(dev).data_ptr(), _lib.stream_ptr()))
        if sink is not None:
            ev[1].record()
            sink.append(ev)
        _mirror(dev).copy_(_status_words(dev), non_blocking=True)
    return (out, lse) if return_lse else out


def merge_attention_states(o_a: torch.Tensor, lse_a: torch.Tensor, o_b: torch.Tensor, lse_b: torch.Tensor,
                           tensor_layout: str = "HND", out: Optional[torch.Tensor] = None):
    """Combines two partial attention results over DISJOINT sets of key blocks -- (o_a, lse_a) and
    (o_b, lse_b) from calls with return_lse=True -- into the result over their union: the consumer of the
    LSE that the reference returns "for cases like Ring Attention" (paroattention/core.py:55-57).
    o_*: [B,H,N,D] ("HND") or [B,N,H,D] ("NHD"), fp16/bf16; lse_*: fp32 [B,H,N], natural log, -inf for rows
    without a kept block.  Returns (o, lse)."""
    _lib.require_cuda(o_a, o_b, lse_a, lse_b)
    if o_a.shape != o_b.shape or o_a.dtype != o_b.dtype or o_a.stride() != o_b.stride():
        raise ValueError("o_a and o_b must have the same shape, dtype and strides")
    va = o_a if tensor_layout == "HND" else o_a.transpose(1, 2)
    vb = o_b if tensor_layout == "HND" else o_b.transpose(1, 2)
    B, H, N, D = va.shape
    if va.stride(-1) != 1:
        raise ValueError("last dimension must be contiguous")
    for t in (lse_a, lse_b):
        if t.dtype != torch.float32 or tuple(t.shape) != (B, H, N) or not t.is_contiguous():
            raise ValueError("lse_a / lse_b must be contiguous fp32 [B,H,N]")
    with torch.cuda.device(o_a.device):
        if out is None:
            out = torch.empty_like(o_a)
        elif out.shape != o_a.shape or out.dtype != o_a.dtype or out.stride() != o_a.stride():
            raise ValueError("out must match o_a")
        lse = torch.empty(B, H, N, dtype=torch.float32, device=o_a.device)
        _lib.check(_lib.lib().paro_merge_attn_states(
            o_a.data_ptr(), lse_a.data_ptr(), o_b.data_ptr(), lse_b.data_ptr(), out.data_ptr(), lse.data_ptr(),
            _lib.dtype_code(o_a.dtype), B, H, N, D, va.stride(0), va.stride(1), va.stride(2), _lib.stream_ptr()))
    return out, lse


def _pad_head_dim(*ts):
    """Pads head_dim up to 64 or 128 like the reference (core.py:181-192)."""
    d = ts[0].size(-1)
    if d > 128:
        raise ValueError(f"Unsupported head_dim: {d}")
    target = 64 if d <= 64 else 128
    if d == target:
        return ts, d
    return tuple(F.pad(t, (0, target - d)) for t in ts), d


def _as_plan(sparse: Union[torch.Tensor, CompactPlan]) -> CompactPlan:
    return sparse if isinstance(sparse, CompactPlan) else compact_plan(sparse)


@torch.compiler.disable
def paroattn_qk_int8_pv_fp16_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                  sparse: Union[torch.Tensor, CompactPlan], tensor_layout: str = "HND",
                                  is_causal: bool = False, qk_quant_gran: str = "per_warp",
                                  sm_scale: Optional[float] = None, return_lse: bool = False,
                                  smooth_k: bool = False, smooth_v: bool = True, attn_mode: str = "fast",
                                  **kwargs: Any):
    """Same call as the reference operator (core.py:88-216): q, k, v are ALREADY in the
    reordered token order, `sparse` is the boolean block mask `[B,H,nb,nb]` (or `[H,nb,nb]`,
    shared by the batch; or an already compacted plan).  INT8 Q.K^T, fp16 P.V with fp32
    accumulation.  Unlike the reference, V is first quantised per channel to FP8-e4m3 values
    (carried as bf16), as the fake-quant emulation this library is checked against does.
    smooth_k defaults to False as in the reference processors (cogvideox.py:186 passes no km).
    `is_causal` is not supported (the video models never use it).  The returned LSE is that of
    the scores the kernel saw (shifted by q.mean(k) per row when smooth_k is on)."""
    dtype = q.dtype
    assert q.is_cuda, "Input tensors must be on cuda."
    assert dtype in [torch.float16, torch.bfloat16], "Input tensors must be in dtype of torch.float16 or torch.bfloat16"
    assert qk_quant_gran in ["per_warp", "per_thread"], "qk_quant_gran must be either 'per_warp' or 'per_thread'."
    assert q.device == k.device == v.device, "All tensors must be on the same device."
    assert q.dtype == k.dtype == v.dtype, "All tensors must have the same dtype."
    if is_causal:
        raise ValueError("is_causal=True is not supported by paroatten_b200")
    if tensor_layout not in ("HND", "NHD"):
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    (q, k, v), head_dim_og = _pad_head_dim(q, k, v)
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1, "Last dim of qkv must be contiguous."
    if sm_scale is None:
        sm_scale = head_dim_og ** -0.5
    with torch.cuda.device(q.device):
        km = channel_mean(k, tensor_layout) if smooth_k else None
        if qk_quant_gran == "per_warp":
            q8, qs, k8, ks = per_warp_int8(q, k, km, BLKQ=64, WARPQ=32, BLKK=64, tensor_layout=tensor_layout)
            group, scale = 32, sm_scale
        else:
            # the reference's "per_thread" branch quantises per 64-token block with the softmax scale
            # folded into Q (core.py:204-205, quant.py:91-96)
            q8, qs, k8, ks = per_block_int8(q, k, km, BLKQ=64, BLKK=64, sm_scale=sm_scale, tensor_layout=tensor_layout)
            group, scale = 64, 1.0 / 1.44269504
        _, vs, vm, v16 = per_channel_fp8(v, tensor_layout, smooth_v=smooth_v, return_16=True)
        if tensor_layout == "NHD":
            q8, k8 = q8.transpose(1, 2), k8.transpose(1, 2)  # back to the HND buffers
        res = sparse_attn_quantized(q8, qs, k8, ks, v16, vs, vm, _as_plan(sparse), scale, out_dtype=dtype,
                                    q_group=group, return_lse=return_lse, out_layout=tensor_layout, mode=attn_mode)
    o, lse = res if return_lse else (res, None)
    o = o[..., :head_dim_og]
    return (o, lse) if return_lse else o


def paroattn(q, k, v, tensor_layout: str = "HND", is_causal: bool = False, sm_scale: Optional[float] = None,
             return_lse: bool = False, sparse=None, **kwargs: Any):
    """Reference dispatcher signature (core.py:13-85).  There is one implementation here
    (sm_100a); `sparse` is required."""
    if sparse is None:
        raise ValueError("paroattn needs the block mask `sparse`")
    major, minor = torch.cuda.get_device_capability(q.device)
    if major != 10:
        raise ValueError(f"Unsupported CUDA architecture: sm{major}{minor}")
    return paroattn_qk_int8_pv_fp16_cuda(q, k, v, sparse, tensor_layout=tensor_layout, is_causal=is_causal,
                                         sm_scale=sm_scale, return_lse=return_lse, **kwargs)


def paro_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, permute_plan, sparse_plan, *,
                   i_block: int = 0, i_timestep: int = 0, grid_fhw: Tuple[int, int, int], n_text: int = 0,
                   rope: Optional[RopeTables] = None, tensor_layout: str = "HND", sm_scale: Optional[float] = None,
                   smooth_k: bool = True, smooth_v: bool = True, return_lse: bool = False,
                   q_norm=None, k_norm=None, attn_mode: str = "fast", empty_head_mode: str = "zero"):
    """The whole path of one self-attention layer, as the reference processors compose it
    (cogvideox.py:161-227): q, k, v in NATURAL token order ->
    [q_norm / k_norm (rope.QKNorm): the processors' norm_q / norm_k, applied to every token as it is read]
    RoPE on the video tokens of q, k + per-head F/H/W reordering of q, k, v (one fused pass each)
    -> INT8 q (per 32 rows) / INT8 k (per 64 rows, mean-smoothed) / FP8 v
    -> block-sparse attention over the kept blocks of sparse_plan[i_timestep, i_block]
    -> output rows stored back in natural token order.

    permute_plan: PermutePlan, or the reference's dict {'permute': [L,H], 'empty': [L,H]}, or int order ids [H].
    sparse_plan: SparsePlan, the reference's [T,L,H,nb,nb] tensor, a mask [H,nb,nb] / [B,H,nb,nb],
    or a CompactPlan.
    Heads flagged in permute_plan['empty'][i_block] (the reference computes the flags and acts on them in
    bench/check.py:116-128; its pipeline's mask multiply is commented out, example/pipeline_cogvideox.py:76-77):
    empty_head_mode "zero" drops every video-to-video block of such a head from the walk (text rows and
    columns stay; a head without text keeps nothing and yields zeros); "uniform" -- sequences without text
    only -- makes the head attend uniformly, i.e. its output is the mean of V over the tokens.  Masks handed
    over already compacted (CompactPlan, SparsePlan, PlanStore) must have had plan.apply_empty_heads applied
    by the caller."""
    _lib.require_cuda(q, k, v)
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("q, k, v must share dtype fp16 or bf16")
    grid = tuple(int(g) for g in grid_fhw)
    (q, k, v), head_dim_og = _pad_head_dim(q, k, v)
    if (q_norm is not None or k_norm is not None) and q.shape[-1] != head_dim_og:
        raise ValueError("q_norm / k_norm need a head dimension of 64 or 128 (no padding)")
    if sm_scale is None:
        sm_scale = head_dim_og ** -0.5
    dev = q.device
    with torch.cuda.device(dev):
        empty = None
        if isinstance(permute_plan, PermutePlan):
            orders, index = permute_plan.orders(i_block), permute_plan.index(i_block)
            empty = permute_plan.empty(i_block)
        else:
            ids = permute_plan["permute"][i_block] if isinstance(permute_plan, dict) else permute_plan
            orders = torch.as_tensor(ids).to(dev, torch.int32).contiguous()
            index = perm_index(orders, grid, dev)
            if isinstance(permute_plan, dict) and permute_plan.get("empty") is not None:
                empty = torch.as_tensor(permute_plan["empty"][i_block]).to(dev).bool()
        if empty is not None and not bool(empty.any()):
            empty = None
        if empty_head_mode not in ("zero", "uniform"):
            raise ValueError(f"unknown empty_head_mode {empty_head_mode!r}")
        if empty is not None and empty_head_mode == "uniform" and n_text > 0:
            raise NotImplementedError("empty_head_mode='uniform' is defined for sequences without text tokens")
        n_text_blocks = (n_text + 63) // 64
        if isinstance(sparse_plan, (SparsePlan, PlanStore)):
            plan = sparse_plan.get(i_timestep, i_block)
        elif isinstance(sparse_plan, CompactPlan):
            plan = sparse_plan
        elif sparse_plan.dim() == 5:
            plan = compact_plan(apply_empty_heads(sparse_plan[i_timestep, i_block].to(dev), empty, n_text_blocks),
                                pairing="overlap")
        else:
            plan = compact_plan(apply_empty_heads(sparse_plan.to(dev), empty, n_text_blocks), pairing="overlap")
        # Q and V: the quantisers read the natural-order tensors through the RoPE + reordering front end
        # (no reordered 16-bit copy).  Smoothed K needs the mean of the rotated values first; rotating
        # twice costs more than writing the rotated copy once, so K keeps the two-step form.
        q8, qs, _ = prep_qk_int8(q, orders, grid, n_text, rope, group=32, tensor_layout=tensor_layout, norm=q_norm)
        if smooth_k:
            kp = rope_permute(k, orders, grid, n_text, rope, tensor_layout=tensor_layout, norm=k_norm)
            k8, ks = _quant_int8(kp, "HND", 64, km=channel_mean(kp))
        else:
            k8, ks, _ = prep_qk_int8(k, orders, grid, n_text, rope, group=64, tensor_layout=tensor_layout,
                                     norm=k_norm)
        v16, vs, vm, _ = prep_v_fp8(v, orders, grid, n_text, smooth_v=smooth_v, tensor_layout=tensor_layout)
        res = sparse_attn_quantized(q8, qs, k8, ks, v16, vs, vm, plan, sm_scale, out_dtype=q.dtype, q_group=32,
                                    inv_index=index, n_text=n_text, return_lse=return_lse, out_layout=tensor_layout,
                                    mode=attn_mode)
        if empty is not None and empty_head_mode == "uniform":
            # uniform attention over all N tokens: O = mean of V (the channel mean the V quantiser produced,
            # or one reduction when smoothing is off); LSE of N equal scores of value 0
            o_, _ = res if return_lse else (res, None)
            mean_v = vm if vm is not None else channel_mean(v, tensor_layout, out_dtype=torch.float32)
            hsel = empty.nonzero().flatten()
            fill = mean_v[:, hsel].to(o_.dtype)                       # [B, n_empty, D]
            if tensor_layout == "HND":
                o_[:, hsel] = fill.unsqueeze(2).expand(-1, -1, o_.shape[2], -1)
            else:
                o_[:, :, hsel] = fill.unsqueeze(1).expand(-1, o_.shape[1], -1, -1)
            if return_lse:
                res[1][:, hsel] = float(torch.log(torch.tensor(float(q.shape[2 if tensor_layout == "HND" else 1]))))
    o, lse = res if return_lse else (res, None)
    o = o[..., :head_dim_og]
    return (o, lse) if return_lse else o
