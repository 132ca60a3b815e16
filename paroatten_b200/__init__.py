"""paroatten_b200: PAROAttention's reordered, quantized, block-sparse attention path for
NVIDIA B200 (sm_100a), behind the reference's `paroattention` Python names."""
from .core import (check_status, last_redo_count, merge_attention_states, paro_attention, paroattn, paroattn_qk_int8_pv_fp16_cuda,
                   sparse_attn_quantized)
from .host import HostPipelinedAttention, pinned_like
from .plan import (CompactPlan, PermutePlan, PlanStore, SparsePlan, apply_empty_heads, compact_plan, perm_index,
                   validate_plan)
from .processors import PARO_CogVideoXAttnProcessor2_0, PARO_WanAttnProcessor2_0, TimestepCallback
from .quant import (channel_mean, per_block_int8, per_channel_fp8, per_warp_int8, prep_qk_int8, prep_v_fp8,
                    sub_mean)
from .rope import QKNorm, RopeTables, rope_permutation, rope_permute, rope_tables

__all__ = [
    "paroattn", "paroattn_qk_int8_pv_fp16_cuda", "paro_attention", "sparse_attn_quantized", "check_status", "last_redo_count", "merge_attention_states",
    "apply_empty_heads", "validate_plan",
    "PARO_CogVideoXAttnProcessor2_0", "PARO_WanAttnProcessor2_0", "TimestepCallback",
    "per_block_int8", "per_warp_int8", "sub_mean", "per_channel_fp8", "channel_mean", "prep_qk_int8", "prep_v_fp8",
    "rope_permutation", "rope_permute", "rope_tables", "RopeTables", "QKNorm",
    "HostPipelinedAttention", "pinned_like", "CompactPlan", "SparsePlan", "PlanStore", "PermutePlan", "compact_plan", "perm_index",
]
