"""diffusers attention processors with the reference's names, call signatures and attribute
contract (paroattention/cogvideox.py:112-250, paroattention/wan.py:113-327).

State injected by the pipeline set-up, exactly as the reference's `paroattn_convert` does
(example/pipeline_cogvideox.py:120-136):
    permute_plan  dict {'permute': [L,H] order ids, ...} (or a plan.PermutePlan)
    sparse_mask   bool [T, L, H, nb, nb] (or a plan.SparsePlan / plan.PlanStore shared by all layers)
    i_block       layer index, i_timestep  timestep bin (set by TimestepCallback)
    grid_fhw      latent grid (F, H, W); defaults to the reference's hard-coded 13x30x45 / 21x45x80
The processors only need `attn` to expose to_q/to_k/to_v/to_out, norm_q/norm_k and heads, so
they also work with any module of that shape.  Shapes are taken from the inputs (the reference
hard-codes them at cogvideox.py:184 and wan.py:204).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .core import check_status, paro_attention
from .plan import PermutePlan, PlanStore, SparsePlan
from .rope import QKNorm, RopeTables, rope_tables, tables_from_embedding


class _ProcessorBase:
    default_grid = None
    rope_family = None

    def __init__(self):
        self.time_accum = {"total": 0.0}
        self.call_count = 0
        self._pending = []
        self.grid_fhw = self.default_grid
        self.i_block = 0
        self.i_timestep = 0
        self.smooth_k = True
        self.empty_head_mode = "zero"  # what to do with heads flagged in permute_plan['empty'] (see paro_attention)
        self.fuse_qk_norm = True      # fold norm_q / norm_k into the RoPE + reorder + quantise passes
        self._rope_cache = {}
        self._pplan = None
        self._splan = None

    # -- plan handling ------------------------------------------------------------------------
    def _plans(self, device):
        if self._pplan is None or self._pplan_src is not self.permute_plan:
            self._pplan_src = self.permute_plan
            self._pplan = (self.permute_plan if isinstance(self.permute_plan, PermutePlan)
                           else PermutePlan(self.permute_plan, self.grid_fhw, device))
        src = getattr(self, "sparse_mask", None)
        if src is None and hasattr(self, "prefetch_stream"):
            src = self.prefetch_stream.sparse_mask  # the reference's CPU-resident mask holder
        if src is None:
            raise RuntimeError("processor has no sparse_mask")
        if self._splan is None or self._splan_src is not src:
            self._splan_src = src
            self._splan = src if isinstance(src, (SparsePlan, PlanStore)) else SparsePlan(src, device)
        return self._pplan, self._splan

    def _rope(self, head_dim, device, emb=None) -> RopeTables:
        """Tables for the fused rotation.  `emb` is the rotary embedding the pipeline passed in: the angles
        are taken from it (rope.tables_from_embedding; cached per tensor), as the reference applies the
        embedding it is given (cogvideox.py:167-172, wan.py:161-167).  With emb=True the tables are built
        for grid_fhw with theta 10000."""
        if emb is None or emb is True:
            key = (head_dim, tuple(self.grid_fhw), str(device))
            if key not in self._rope_cache:
                self._rope_cache[key] = rope_tables(self.grid_fhw, head_dim, self.rope_family, device=device)
            return self._rope_cache[key]
        first = emb[0] if isinstance(emb, (tuple, list)) else emb
        key = ("emb", first.data_ptr(), tuple(first.shape), first._version, head_dim, tuple(self.grid_fhw), str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = tables_from_embedding(emb, self.grid_fhw, head_dim, self.rope_family, device=device)
        return self._rope_cache[key]

    def _norms(self, attn, query, key, D, per_head):
        """Folds attn.norm_q / attn.norm_k into the pre-attention passes when they are of a known
        form (rope.QKNorm.from_module); any other module is simply called, as the reference does
        (cogvideox.py:161-164, wan.py:150-153).  Returns (query, key, q_norm, k_norm)."""
        out = []
        for t, name in ((query, "norm_q"), (key, "norm_k")):
            mod = getattr(attn, name, None)
            spec = None
            if mod is not None:
                spec = QKNorm.from_module(mod, attn.heads, D) if self.fuse_qk_norm and D in (64, 128) else None
                if spec is None:
                    B, N, inner = t.shape
                    t = mod(t.view(B, N, attn.heads, D)).reshape(B, N, inner) if per_head else mod(t)
            out.append((t, spec))
        return out[0][0], out[1][0], out[0][1], out[1][1]

    def _attend(self, query, key, value, n_text, rotary, q_norm=None, k_norm=None):
        """query/key/value: [B, N, H*D] projections; rotary: the embedding passed to the processor (None =
        no rotation).  Returns [B, N, H*D]."""
        B, N, inner = query.shape
        H = self._heads
        D = inner // H
        q, k, v = (t.view(B, N, H, D) for t in (query, key, value))
        pplan, splan = self._plans(query.device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = paro_attention(q, k, v, pplan, splan, i_block=self.i_block, i_timestep=self.i_timestep,
                             grid_fhw=self.grid_fhw, n_text=n_text,
                             rope=self._rope(D, query.device, rotary) if rotary is not None else None,
                             tensor_layout="NHD", smooth_k=self.smooth_k, q_norm=q_norm, k_norm=k_norm,
                             empty_head_mode=self.empty_head_mode)
        if isinstance(splan, PlanStore):     # stream the next layer's lists in while this layer computes
            splan.prefetch(self.i_timestep, self.i_block + 1)
        end.record()
        self._pending.append((start, end))   # read lazily: no device sync per layer
        self.call_count += 1
        return out.reshape(B, N, inner)

    def get_time_stats(self):
        """Accumulated attention milliseconds (reference: cogvideox.py:247-250).  Events are
        resolved here instead of synchronising the device after every layer (cogvideox.py:224)."""
        if self._pending:
            torch.cuda.synchronize()
            check_status()            # a launch that gave up a wait must not pass as a timing
            for s, e in self._pending:
                self.time_accum["total"] += s.elapsed_time(e)
            self._pending.clear()
        return {"total_ms": self.time_accum["total"]}


class PARO_CogVideoXAttnProcessor2_0(_ProcessorBase):
    """CogVideoX joint text+video self-attention (reference: cogvideox.py:112-250).  When
    `image_rotary_emb` = (cos, sin) is given, the rotation is applied inside the fused RoPE+permute pass
    with the angles of that embedding (reduced once to per-axis tables; an embedding that is not a 3-D
    table over `grid_fhw` raises)."""
    default_grid = (13, 30, 45)
    rope_family = "cogvideox"

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: torch.Tensor,
                 attention_mask: Optional[torch.Tensor] = None,
                 image_rotary_emb: Optional[torch.Tensor] = None) -> torch.Tensor:
        text_seq_length = encoder_hidden_states.size(1)
        hidden_states = torch.cat([encoder_hidden_states, hidden_states], dim=1)
        self._heads = attn.heads
        query, key, value = attn.to_q(hidden_states), attn.to_k(hidden_states), attn.to_v(hidden_states)
        B, N, inner = key.shape
        D = inner // attn.heads
        query, key, q_norm, k_norm = self._norms(attn, query, key, D, per_head=True)
        hidden_states = self._attend(query, key, value, text_seq_length, image_rotary_emb, q_norm, k_norm)
        hidden_states = attn.to_out[0](hidden_states)
        hidden_states = attn.to_out[1](hidden_states)
        encoder_hidden_states, hidden_states = hidden_states.split(
            [text_seq_length, hidden_states.size(1) - text_seq_length], dim=1)
        return hidden_states, encoder_hidden_states


class PARO_WanAttnProcessor2_0(_ProcessorBase):
    """Wan2.1 self-attention (reference: wan.py:113-327, without its debugging detours at
    :209-297).  Cross-attention layers keep the stock processor in the reference (wan.py:566) and
    are not handled here."""
    default_grid = (21, 45, 80)
    rope_family = "wan"

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None,
                 attention_mask: Optional[torch.Tensor] = None,
                 rotary_emb: Optional[torch.Tensor] = None) -> torch.Tensor:
        if encoder_hidden_states is not None and encoder_hidden_states is not hidden_states:
            raise ValueError("PARO_WanAttnProcessor2_0 handles self-attention only")
        self._heads = attn.heads
        query, key, value = attn.to_q(hidden_states), attn.to_k(hidden_states), attn.to_v(hidden_states)
        D = query.shape[-1] // attn.heads
        query, key, q_norm, k_norm = self._norms(attn, query, key, D, per_head=False)
        hidden_states = self._attend(query, key, value, 0, rotary_emb, q_norm, k_norm)
        hidden_states = attn.to_out[0](hidden_states)
        hidden_states = attn.to_out[1](hidden_states)
        return hidden_states


class TimestepCallback:
    """Maps the denoising step to the sparse plan's timestep bin and pushes it into every
    processor (reference: paroattention/prefetch_utils.py:4-32).  Duck-typed: no diffusers import."""
    tensor_inputs = []

    def __init__(self, num_timestep_for_sparse_mask: int = 10):
        self.num_timestep_for_sparse_mask = num_timestep_for_sparse_mask
        self.sparse_mask_timestep = 0

    def on_step_end(self, pipeline, step, timestep, callback_kwargs):
        total_steps = len(pipeline.scheduler.timesteps)
        step = step % total_steps
        normalized = (step + 1) / total_steps
        self.sparse_mask_timestep = int(normalized * self.num_timestep_for_sparse_mask)
        pipeline.transformer.i_timestep = self.sparse_mask_timestep
        for block in pipeline.transformer.transformer_blocks:
            block.attn1.processor.i_timestep = self.sparse_mask_timestep
        if torch.cuda.is_available():
            check_status()     # once per denoising step: stop the run if an attention launch gave up a wait
        return callback_kwargs

    __call__ = on_step_end
