# -*- coding: utf-8 -*-
"""RetNet retention: fixed per-head decay log(1 - 2^(-5-h)) fed to the simple-GLA kernels
(fla/ops/retention/chunk.py:8, fla/ops/retention/fused_recurrent.py:9)."""

from typing import Optional, Tuple

import torch

from .simple_gla import chunk_simple_gla, fused_recurrent_simple_gla


def retention_decay(q: torch.Tensor, head_first: bool) -> torch.Tensor:
    """Per-token log decay [B,H,T] / [B,T,H] (fp32), constant along T (fla/ops/retention/chunk.py:56-60)."""
    n_heads = q.shape[1] if head_first else q.shape[2]
    s = (1 - q.new_tensor(2., dtype=torch.float).pow(-5. - q.new_tensor(range(n_heads), dtype=torch.float))).log()
    if head_first:
        return s[None, :, None].expand(q.shape[0], q.shape[1], q.shape[2]).contiguous()
    return s[None, None, :].expand(q.shape[0], q.shape[1], q.shape[2]).contiguous()


_DECAY_CACHE = {}  # (B, T, H, head_first, device, offsets id) -> (g, its chunk-local cumsum): constants of the shape


def _cached_decay(q, head_first, offsets):
    """The decay is a constant per head, so g and its chunk-local cumsum depend on the shape (and offsets) only: they are
    built once per shape instead of by four elementwise launches and a cumsum per call."""
    from . import common as C
    key = (tuple(q.shape[:3]), bool(head_first), str(q.device), None if offsets is None else (id(offsets), offsets._version))
    hit = _DECAY_CACHE.get(key)
    if hit is None:
        if len(_DECAY_CACHE) >= 8:
            _DECAY_CACHE.clear()
        g = retention_decay(q, head_first)
        hit = (g, C.chunk_local_cumsum(g, offsets=offsets, head_first=head_first), offsets)
        _DECAY_CACHE[key] = hit
    return hit[0], hit[1]


def chunk_retention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    from ..utils import resolve_offsets
    from .simple_gla import check_varlen_args
    offsets = resolve_offsets(offsets, cu_seqlens)
    check_varlen_args(q, initial_state, offsets, head_first)
    g, g_cum = _cached_decay(q, head_first, offsets)
    return chunk_simple_gla(q=q, k=k, v=v, scale=scale, g=g, initial_state=initial_state,
                            output_final_state=output_final_state, head_first=head_first, offsets=offsets,
                            _g_cumsum=g_cum)


def fused_recurrent_retention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    reverse: bool = False,
    offsets: Optional[torch.LongTensor] = None,
    head_first: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    g = retention_decay(q, head_first)
    return fused_recurrent_simple_gla(q, k, v, g, scale=scale, initial_state=initial_state,
                                      output_final_state=output_final_state, reverse=reverse, offsets=offsets,
                                      head_first=head_first, cu_seqlens=cu_seqlens)


def fused_chunk_retention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    head_first: bool = True,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """The reference's fused execution mode of retention (fla/ops/retention/fused_chunk.py:296): fixed-length batches
    only, the initial state is a constant (its backward returns no gradient for it). Same decay and result as
    `chunk_retention`."""
    if initial_state is not None:
        initial_state = initial_state.detach()
    return chunk_retention(q, k, v, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                           head_first=head_first)
