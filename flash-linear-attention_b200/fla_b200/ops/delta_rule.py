# -*- coding: utf-8 -*-
"""DeltaNet: S_t = S_{t-1} + k_t^T beta_t (v_t - k_t S_{t-1}), chunked through the WY representation.
Public signatures follow fla/ops/delta_rule/chunk.py:243 and fla/ops/delta_rule/fused_recurrent.py:478."""

from typing import Optional, Tuple

import torch

from ..utils import SAVE_STATES, Geometry, autocast_custom_bwd, autocast_custom_fwd, contiguous, resolve_offsets
from . import common as C
from .recurrent import FusedRecurrentDeltaRuleFunction
from .simple_gla import check_varlen_args


def chunk_delta_rule_fwd(geo, q, k, v, beta, scale, initial_state, output_final_state):
    aw, _, w, u = C.fwd_prepare_wy_repr(geo, k, v, beta)
    plan, M = C.slab_plan(geo, k), None
    if plan is not None:  # a few long sequences: the scan runs over slabs of T side by side
        h, v_new, ht, M = C.slab_delta_fwd_h(plan, geo, k, w, u, h0=initial_state, output_final_state=output_final_state)
    else:
        h, v_new, ht = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, h0=initial_state, output_final_state=output_final_state)
    o = C.chunk_fwd_o(geo, q, k, v_new, h, scale=scale)
    return o, aw, ht, (w, h, v_new, M)


def chunk_delta_rule_bwd(geo, q, k, v, beta, aw, scale, initial_state, do, dht, saved=None):
    """Same stage order as fla/ops/delta_rule/chunk.py:70-163. `saved` = (w, h, v_new, M) kept from
    forward (M: slab transitions of a split scan, else None); None recomputes them like the reference."""
    if saved is not None:
        w, h, v_new, M = saved
        plan = C.slab_plan(geo, k) if M is not None else None  # split the reverse scan iff the forward one was
    else:
        plan = C.slab_plan(geo, k)
        w, u = C.fwd_recompute_w_u(geo, k, v, beta, aw)
        if plan is not None:
            h, v_new, _, M = C.slab_delta_fwd_h(plan, geo, k, w, u, h0=initial_state, output_final_state=False)
        else:
            h, v_new, _ = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, h0=initial_state, output_final_state=False)
    dv = C.chunk_bwd_dv_local(geo, q, k, None, do, scale)
    if plan is not None:
        dh, dh0, dv = C.slab_delta_bwd_dhu(plan, geo, M, q, k, w, do, dv, scale, dht=dht, want_dh0=initial_state is not None)
    else:
        dh, dh0, dv = C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, dht=dht,
                                                       want_dh0=initial_state is not None)
    dq, dk, dw, _ = C.chunk_bwd_dqkwg(geo, q, k, v_new, h, dh, do, scale, w=w, dv=dv)
    dk, dv, db, _ = C.bwd_prepare_wy_repr(geo, k, v, beta, aw, dw, dv, dk_in=dk)
    return dq, dk, dv, db, dh0


class ChunkDeltaRuleFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, beta, scale, initial_state, output_final_state, offsets, head_first):
        geo = Geometry(k, v, offsets, head_first)
        beta_k = beta.to(k.dtype)
        o, aw, ht, states = chunk_delta_rule_fwd(geo, q, k, v, beta_k, scale, initial_state, output_final_state)
        ctx.save_for_backward(q, k, v, beta_k, aw, initial_state, *(states if SAVE_STATES else ()))
        ctx.geo, ctx.scale, ctx.beta_dtype = geo, scale, beta.dtype
        return o.to(q.dtype), ht

    @staticmethod
    @contiguous
    @autocast_custom_bwd
    def backward(ctx, do, dht):
        q, k, v, beta, aw, initial_state, *states = ctx.saved_tensors
        dq, dk, dv, db, dh0 = chunk_delta_rule_bwd(ctx.geo, q, k, v, beta, aw, ctx.scale, initial_state, do, dht,
                                                   saved=states or None)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), db.to(ctx.beta_dtype), None, dh0, None, None, None


def chunk_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    beta: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q, k: [B,H,T,K] (or [B,T,H,K]); v: [...,V]; beta: [B,H,T] (or [B,T,H]). bf16/fp16 only."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype != torch.float32, "ChunkDeltaRuleFunction does not support float32. Please use bfloat16."
    assert len(beta.shape) == 3, "beta must be of shape (batch size, num of head, seq len)."
    check_varlen_args(q, initial_state, offsets, head_first)
    scale = k.shape[-1] ** -0.5 if scale is None else scale
    return ChunkDeltaRuleFunction.apply(q, k, v, beta, scale, initial_state, output_final_state, offsets, head_first)


def fused_recurrent_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    beta: torch.Tensor = None,
    scale: float = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Token-by-token delta rule; beta may be per head ([B,H,T]) or per value channel ([B,H,T,V])."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    else:
        assert scale > 0, "scale must be positive"
    if beta is None:
        beta = torch.ones_like(q[..., 0])
    return FusedRecurrentDeltaRuleFunction.apply(q, k, v, beta, scale, initial_state, output_final_state, offsets,
                                                 head_first)


def fused_chunk_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    beta: torch.Tensor,
    scale: float = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    head_first: bool = True,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """The reference's fused execution mode of the delta rule (fla/ops/delta_rule/fused_chunk.py:359): fixed-length
    batches, chunks of 16 tokens walked by one kernel. The recurrence, the arguments and the gradients (including the
    one of the initial state) are those of `chunk_delta_rule`, whose kernels compute it here."""
    if scale is None:
        scale = k.shape[-1] ** -0.5
    else:
        assert scale > 0, "scale must be positive."
    return chunk_delta_rule(q, k, v, beta, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                            head_first=head_first)
