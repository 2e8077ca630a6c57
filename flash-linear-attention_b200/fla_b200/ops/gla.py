# -*- coding: utf-8 -*-
"""GLA: S_t = diag(exp(g_t)) S_{t-1} + k_t^T v_t with one log gate per key channel.
Public signatures follow fla/ops/gla/chunk.py:1409 and fla/ops/gla/fused_recurrent.py:11."""

from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils import SAVE_STATES, Geometry, contiguous, resolve_offsets
from . import common as C
from .recurrent import fused_recurrent
from .simple_gla import check_varlen_args


def chunk_gla_fwd_intra_gk(geo, q, k, g_cum, scale):
    """Intra-chunk score matrix A [.., 64] fp32 (fla/ops/gla/chunk.py:840)."""
    a = torch.empty(*q.shape[:-1], _lib.CHUNK, dtype=torch.float32, device=q.device)
    _lib.call("flab_gla_fwd_intra", q, **geo.kw(), scale=scale, q=q, k=k, gk=g_cum, a=a)
    return a


def chunk_gla_fwd_o_gk(geo, q, v, g_cum, a, h, scale):
    """o = (q * scale * e^g) h + tril(A) v (fla/ops/gla/chunk.py:941)."""
    o = torch.empty_like(v)
    _lib.call("flab_gla_fwd_o", q, **geo.kw(), scale=scale, q=q, v=v, gk=g_cum, h=h, a=a, o=o)
    return o


def chunk_gla_fwd(geo, q, k, v, g, scale, initial_state, output_final_state):
    g_cum = C.chunk_local_cumsum(g, offsets=geo.offsets_tensor, head_first=geo.head_first)
    h, ht = C.chunk_fwd_h(geo, k, v, gk=g_cum, h0=initial_state, output_final_state=output_final_state)
    a = chunk_gla_fwd_intra_gk(geo, q, k, g_cum, scale)
    o = chunk_gla_fwd_o_gk(geo, q, v, g_cum, a, h, scale)
    return g_cum, a, h, ht, o


def chunk_gla_bwd(geo, q, k, v, g_cum, scale, initial_state, a, do, dht, h=None):
    """Stage order of fla/ops/gla/chunk.py:1217-1320; the returned dg is w.r.t. the raw gate."""
    if h is None:
        h, _ = C.chunk_fwd_h(geo, k, v, gk=g_cum, h0=initial_state, output_final_state=False)
    dh, dh0 = C.chunk_bwd_dh(geo, q, do, scale, gk=g_cum, dht=dht, want_dh0=initial_state is not None)
    da = torch.empty_like(a)
    dv = torch.empty_like(v)
    _lib.call("flab_gla_bwd_dav", q, **geo.kw(), scale=scale, k=k, v=v, gk=g_cum, a=a, d_o=do, dh=dh, da=da, dv=dv)
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dg = torch.empty(g_cum.shape, dtype=torch.float32, device=q.device)
    _lib.call("flab_gla_bwd_dqkg", q, **geo.kw(), scale=scale, q=q, k=k, v=v, gk=g_cum, h=h, dh=dh, d_o=do, da=da,
              dq=dq, dk=dk, dgk=dg)
    return dq, dk, dv, dg, dh0


class ChunkGLAFunction(torch.autograd.Function):
    # like the reference (fla/ops/gla/chunk.py:1333) this Function has no autocast decorator

    @staticmethod
    @contiguous
    def forward(ctx, q, k, v, g, scale, initial_state, output_final_state, offsets, head_first):
        geo = Geometry(k, v, offsets, head_first)
        g_cum, a, h, ht, o = chunk_gla_fwd(geo, q, k, v, g, scale, initial_state, output_final_state)
        ctx.save_for_backward(q, k, v, g_cum, initial_state, a, *((h,) if SAVE_STATES else ()))
        ctx.geo, ctx.scale, ctx.g_dtype = geo, scale, g.dtype
        return o, ht

    @staticmethod
    @contiguous
    def backward(ctx, do, dht):
        q, k, v, g_cum, initial_state, a, *states = ctx.saved_tensors
        dq, dk, dv, dg, dh0 = chunk_gla_bwd(ctx.geo, q, k, v, g_cum, ctx.scale, initial_state, a, do, dht,
                                            h=states[0] if states else None)
        return dq.to(q), dk.to(k), dv.to(v), dg.to(ctx.g_dtype), None, dh0, None, None, None


def chunk_gla(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    scale: Optional[int] = None,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q, k, g: [B,H,T,K] (or [B,T,H,K]); v: [...,V]; g holds log forget gates per key channel."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return ChunkGLAFunction.apply(q, k, v, g, scale, initial_state, output_final_state, offsets, head_first)


def fused_recurrent_gla(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    gk: Optional[torch.Tensor] = None,
    gv: Optional[torch.Tensor] = None,
    scale: Optional[int] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    reverse: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Token-by-token GLA with optional per-key (gk) and per-value (gv) log gates."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    return fused_recurrent(q=q, k=k, v=v, gk=gk, gv=gv, scale=scale, initial_state=initial_state,
                           output_final_state=output_final_state, reverse=reverse, offsets=offsets,
                           head_first=head_first)


def fused_chunk_gla(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    scale: int = -1,
    initial_state: torch.Tensor = None,
    output_final_state: bool = False,
    head_first: bool = True,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """The reference's fused execution mode of GLA (fla/ops/gla/fused_chunk.py:622): same recurrence and arguments
    as `chunk_gla` with two differences in the contract, both kept: `scale=-1` means K^-0.5, and the initial state is
    a constant (no gradient flows into it). The reference fuses the state walk and the output into one kernel per
    (value tile, key tile); here the same result comes from the chunk kernels, which never hold more than one chunk of
    the sequence per CTA either."""
    if scale == -1:
        scale = q.shape[-1] ** -0.5
    if initial_state is not None:
        initial_state = initial_state.detach()
    return chunk_gla(q, k, v, g, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                     head_first=head_first)
