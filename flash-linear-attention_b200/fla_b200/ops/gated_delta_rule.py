# -*- coding: utf-8 -*-
"""Gated DeltaNet: S_t = e^{g_t} S_{t-1} + k_t^T beta_t (v_t - k_t e^{g_t} S_{t-1}).
Public signatures follow fla/ops/gated_delta_rule/chunk.py:258 and
fla/ops/gated_delta_rule/fused_recurrent.py:210."""

from typing import Optional, Tuple

import torch

from ..utils import SAVE_STATES, Geometry, autocast_custom_bwd, autocast_custom_fwd, contiguous, resolve_offsets
from . import common as C
from .recurrent import FusedRecurrentGatedDeltaRuleFunction
from .simple_gla import check_varlen_args


def chunk_gated_delta_rule_fwd(geo, q, k, v, g, beta, scale, initial_state, output_final_state, g_cum=None):
    """Stage order of fla/ops/gated_delta_rule/chunk.py:20-73. `g_cum`: the chunk-local cumsum of g when the caller
    already has it (the gate prologue computes it in the pass that makes g)."""
    g = g_cum if g_cum is not None else C.chunk_local_cumsum(g, offsets=geo.offsets_tensor, head_first=geo.head_first)
    aw, au, w, u = C.fwd_prepare_wy_repr(geo, k, v, beta, g=g)
    plan, M = C.slab_plan(geo, k), None
    if plan is not None:  # a few long sequences: the scan runs over slabs of T side by side
        h, v_new, ht, M = C.slab_delta_fwd_h(plan, geo, k, w, u, g=g, h0=initial_state, output_final_state=output_final_state)
    else:
        h, v_new, ht = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=g, h0=initial_state,
                                                      output_final_state=output_final_state)
    o = C.chunk_fwd_o(geo, q, k, v_new, h, g=g, scale=scale)
    return g, o, aw, au, ht, (w, h, v_new, M)


def chunk_gated_delta_rule_fwd_fused(geo, q, k, v, g, beta, scale, initial_state, output_final_state):
    """Forward only, as ONE call into the library (flab_gated_delta_rule_fwd): the four stages are
    enqueued back to back with their intermediates in a workspace tensor. Used when no gradient is
    needed (prefill / evaluation); same results as the staged forward."""
    from .. import _lib
    o = torch.empty_like(v)
    ht = torch.empty(geo.N, geo.H, geo.K, geo.V, dtype=torch.float32, device=q.device) if output_final_state else None
    probe = _lib.fill_args(q, **geo.kw())
    need = _lib.load().flab_gated_delta_rule_fwd_workspace(probe)
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    _lib.call("flab_gated_delta_rule_fwd", q, **geo.kw(), scale=scale, q=q, k=k, v=v, g=g.float().contiguous(), beta=beta,
              h0=None if initial_state is None else initial_state.float().contiguous(), o=o, ht=ht, ws=ws, ws_bytes=need)
    return o, ht


def chunk_gated_delta_rule_bwd(geo, q, k, v, g, beta, aw, au, scale, initial_state, do, dht, saved=None, dv_local=None, slab_c=None):
    """Stage order of fla/ops/gated_delta_rule/chunk.py:76-177; `g` is the chunk-local cumsum.
    `saved` = (w, h, v_new, M) kept from forward (M: slab transitions of a split scan, else None); None recomputes them like the
    reference. `dv_local` / `slab_c`: the local dv and the first pass of a split reverse scan when the caller (the
    sequence-parallel backward) has computed them already."""
    if saved is not None:
        w, h, v_new, M = saved
        plan = C.slab_plan(geo, k) if M is not None else None  # split the reverse scan iff the forward one was
    else:
        plan = C.slab_plan(geo, k)
        w, u = C.fwd_recompute_w_u(geo, k, v, beta, aw, au)
        if plan is not None:
            h, v_new, _, M = C.slab_delta_fwd_h(plan, geo, k, w, u, g=g, h0=initial_state, output_final_state=False)
        else:
            h, v_new, _ = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=g, h0=initial_state, output_final_state=False)
    dv = dv_local if dv_local is not None else C.chunk_bwd_dv_local(geo, q, k, g, do, scale)
    if plan is not None:
        dh, dh0, dv = C.slab_delta_bwd_dhu(plan, geo, M, q, k, w, do, dv, scale, g=g, dht=dht, want_dh0=initial_state is not None,
                                           c_=slab_c)
    else:
        dh, dh0, dv = C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, g=g, dht=dht,
                                                       want_dh0=initial_state is not None)
    dq, dk, dw, dg = C.chunk_bwd_dqkwg(geo, q, k, v_new, h, dh, do, scale, g=g, w=w, dv=dv)
    # the last stage also finishes the gate gradient: dg(dqkwg) + its own share, reverse chunk-local cumsum
    dk, dv, db, dg = C.bwd_prepare_wy_repr(geo, k, v, beta, aw, dw, dv, g=g, au=au, dk_in=dk, dg_in=dg)
    return dq, dk, dv, db, dg, dh0


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, offsets, head_first, g_cum=None):
        geo = Geometry(k, v, offsets, head_first)
        beta_k = beta.to(k.dtype)
        g_cum, o, aw, au, ht, states = chunk_gated_delta_rule_fwd(geo, q, k, v, g, beta_k, scale, initial_state,
                                                                  output_final_state, g_cum=g_cum)
        ctx.n_saved_states = len(states) if SAVE_STATES else 0
        ctx.save_for_backward(q, k, v, g_cum, beta_k, aw, au, initial_state, *(states if SAVE_STATES else ()))
        ctx.geo, ctx.scale, ctx.g_dtype, ctx.beta_dtype = geo, scale, g.dtype, beta.dtype
        return o.to(q.dtype), ht

    @staticmethod
    @contiguous
    @autocast_custom_bwd
    def backward(ctx, do, dht):
        q, k, v, g_cum, beta, aw, au, initial_state, *states = ctx.saved_tensors
        dq, dk, dv, db, dg, dh0 = chunk_gated_delta_rule_bwd(ctx.geo, q, k, v, g_cum, beta, aw, au, ctx.scale,
                                                            initial_state, do, dht, saved=states or None)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg.to(ctx.g_dtype), db.to(ctx.beta_dtype),
                None, dh0, None, None, None, None)


def chunk_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: float = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q, k: [B,H,T,K] (or [B,T,H,K]); v: [...,V]; g (log decay), beta: [B,H,T] (or [B,T,H]). bf16/fp16 only."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype != torch.float32, "ChunkGatedDeltaRuleFunction does not support float32. Please use bfloat16."
    assert len(beta.shape) == 3, "beta must be of shape [B, H, T] if head_first=True, or [B, T, H] if head_first=False."
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    else:
        assert scale > 0, "Scale must be positive."
    needs_grad = torch.is_grad_enabled() and any(
        x is not None and x.requires_grad for x in (q, k, v, g, beta, initial_state))
    if not needs_grad and not torch.is_autocast_enabled():
        q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
        geo = Geometry(k, v, offsets, head_first)
        if C.slab_plan(geo, k) is not None:  # a few long sequences: staged forward, scan split into slabs of T
            _, o, _, _, ht, _ = chunk_gated_delta_rule_fwd(geo, q, k, v, g, beta.to(k.dtype), scale, initial_state,
                                                           output_final_state)
            return o.to(q.dtype), ht
        return chunk_gated_delta_rule_fwd_fused(geo, q, k, v, g, beta.to(k.dtype), scale, initial_state,
                                                output_final_state)
    from ..modules.gate_prologue import attached_cumsum
    g_cum = attached_cumsum(g, offsets, head_first)  # made together with g by the gate prologue, if g is its output
    return ChunkGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state, offsets,
                                             head_first, g_cum)


def fused_recurrent_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor = None,
    scale: float = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Decode / token-recurrent form (forward only, like the reference)."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    else:
        assert scale > 0, "scale must be positive"
    if beta is None:
        beta = torch.ones_like(q[..., 0])
    return FusedRecurrentGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state,
                                                      offsets, head_first)
