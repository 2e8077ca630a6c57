# -*- coding: utf-8 -*-
"""Simple GLA (one log-decay per token and head): chunked forward/backward and the token-recurrent
form.  Public signatures follow fla/ops/simple_gla/chunk.py:213 and
fla/ops/simple_gla/fused_recurrent.py:11."""

from typing import Optional, Tuple

import torch

from ..utils import SAVE_STATES, Geometry, autocast_custom_bwd, autocast_custom_fwd, contiguous, resolve_offsets
from . import common as C
from .recurrent import fused_recurrent


def chunk_simple_gla_fwd(geo, q, k, v, g, scale, initial_state, output_final_state, g_cum=None):
    if g_cum is None:
        g_cum = C.chunk_local_cumsum(g, offsets=_off(geo), head_first=geo.head_first) if g is not None else None
    h, ht = C.chunk_fwd_h(geo, k, v, g=g_cum, h0=initial_state, output_final_state=output_final_state)
    o = C.chunk_fwd_o(geo, q, k, v, h, g=g_cum, scale=scale)
    return g_cum, o, ht, h


def chunk_simple_gla_bwd(geo, q, k, v, g_cum, initial_state, do, dht, scale, h=None):
    if h is None:  # recompute the chunk states like the reference (fla/ops/simple_gla/chunk.py:73-86)
        h, _ = C.chunk_fwd_h(geo, k, v, g=g_cum, h0=initial_state, output_final_state=False)
    dh, dh0 = C.chunk_bwd_dh(geo, q, do, scale, g=g_cum, dht=dht, want_dh0=initial_state is not None)
    dq, dk, _, dg = C.chunk_bwd_dqkwg(geo, q, k, v, h, dh, do, scale, g=g_cum)
    dv = C.chunk_bwd_dv(geo, q, k, g_cum, do, dh, scale)
    return dq, dk, dv, dg, dh0


def _off(geo):
    return geo.offsets_tensor


class ChunkSimpleGLAFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, g, scale, initial_state, output_final_state, offsets, head_first, g_cum=None):
        geo = Geometry(k, v, offsets, head_first)
        geo.offsets_tensor = offsets
        g_cum, o, ht, h = chunk_simple_gla_fwd(geo, q, k, v, g, scale, initial_state, output_final_state, g_cum=g_cum)
        ctx.save_for_backward(q, k, v, g_cum, initial_state, *((h,) if SAVE_STATES else ()))
        ctx.geo, ctx.scale = geo, scale
        ctx.g_dtype = g.dtype if g is not None else None
        return o.to(q.dtype), ht

    @staticmethod
    @contiguous
    @autocast_custom_bwd
    def backward(ctx, do, dht):
        q, k, v, g_cum, initial_state, *states = ctx.saved_tensors
        geo = ctx.geo
        dq, dk, dv, dg, dh0 = chunk_simple_gla_bwd(geo, q, k, v, g_cum, initial_state, do, dht, ctx.scale,
                                                   h=states[0] if states else None)
        if g_cum is not None and ctx.needs_input_grad[3]:
            dg = C.chunk_local_cumsum(dg, reverse=True, offsets=geo.offsets_tensor,
                                      head_first=geo.head_first).to(ctx.g_dtype)
        else:  # no gate, or a constant one (retention's fixed decay)
            dg = None
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg, None, dh0, None, None, None, None


def check_varlen_args(q, initial_state, offsets, head_first):
    """Argument checks shared by every chunk op (same conditions and exception types as
    fla/ops/simple_gla/chunk.py:286-295)."""
    if offsets is not None:
        if q.shape[0] != 1:
            raise ValueError(f"The batch size is expected to be 1 rather than {q.shape[0]} when using `offsets`."
                             f"Please flatten variable-length inputs before processing.")
        if head_first:
            raise RuntimeError("Sequences with variable lengths are not supported for head-first mode")
        if initial_state is not None and initial_state.shape[0] != len(offsets) - 1:
            raise ValueError(f"The number of initial states is expected to be equal to the number of input sequences, "
                             f"i.e., {len(offsets) - 1} rather than {initial_state.shape[0]}.")


def chunk_simple_gla(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
    _g_cumsum: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """o_t = scale * q_t S_t with S_t = exp(g_t) S_{t-1} + k_t^T v_t, computed chunk-wise.

    q, k: [B,H,T,K] (or [B,T,H,K] when head_first=False); v: [..., V]; g: [B,H,T] / [B,T,H] log decays.
    Returns (o, final_state) with final_state [N,H,K,V] fp32 or None.
    (`_g_cumsum`: the chunk-local cumsum of g when the caller already holds it; used by `chunk_retention`, whose decay
    is a constant per head.)
    """
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    return ChunkSimpleGLAFunction.apply(q, k, v, g, scale, initial_state, output_final_state, offsets, head_first, _g_cumsum)


def fused_recurrent_simple_gla(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    reverse: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Token-by-token form of `chunk_simple_gla` (fla/ops/simple_gla/fused_recurrent.py:11)."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    return fused_recurrent(q, k, v, g=g, scale=scale, initial_state=initial_state,
                           output_final_state=output_final_state, reverse=reverse, offsets=offsets,
                           head_first=head_first)


def parallel_simple_gla(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    output_attentions: bool = False,
    head_first: bool = True,
    offsets: Optional[torch.LongTensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """The reference's attention-like ("parallel") form of simple GLA (fla/ops/simple_gla/parallel.py:666):
    o_i = scale * sum_{j <= i} <q_i, k_j> exp(G_i - G_j) v_j with G the cumulative log decay, no initial or final state.
    Returns (o, attn); attn `[B, H, T, T]` only with `output_attentions=True` (fixed length only, not differentiable,
    as in the reference, whose backward ignores its gradient). o and the gradients of q, k, v, g are computed by the
    chunk kernels: the same sums, regrouped so that no T x T intermediate exists."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if offsets is not None:
        assert q.shape[0] == 1, "batch size must be 1 when offsets are provided"
        assert not head_first, "head_first must be False when offsets are provided"
    if g is not None:
        g = g.float()
    if output_attentions:
        assert offsets is None, "output_attentions=True is not supported with variable-length sequences"
    o, _ = ChunkSimpleGLAFunction.apply(q, k, v, g, scale, None, False, offsets, head_first, None)
    attn = None
    if output_attentions:
        from .. import _lib
        with torch.no_grad():
            qc, kc = q.contiguous(), k.contiguous()
            geo = Geometry(kc, v, None, head_first)
            G = C.chunk_global_cumsum(g.contiguous(), dtype=torch.float32, head_first=head_first) if g is not None else None
            attn = torch.empty(geo.B, geo.H, geo.T, geo.T, dtype=q.dtype, device=q.device)
            _lib.call("flab_simple_gla_attn", qc, **geo.kw(), scale=scale, q=qc, k=kc, g=G, a=attn)
    return o, attn
