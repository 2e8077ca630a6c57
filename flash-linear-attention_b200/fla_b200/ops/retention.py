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
    g = retention_decay(q, head_first)
    return chunk_simple_gla(q=q, k=k, v=v, scale=scale, g=g, initial_state=initial_state,
                            output_final_state=output_final_state, head_first=head_first, offsets=offsets,
                            cu_seqlens=cu_seqlens)


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
