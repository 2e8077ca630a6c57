# -*- coding: utf-8 -*-
"""Drop-in counterparts of the functions exported by fla.ops.{gla,simple_gla,retention,delta_rule,
gated_delta_rule} (fla/ops/__init__.py)."""

from .delta_rule import chunk_delta_rule, fused_chunk_delta_rule, fused_recurrent_delta_rule
from .gated_delta_rule import chunk_gated_delta_rule, fused_recurrent_gated_delta_rule
from .gla import chunk_gla, fused_chunk_gla, fused_recurrent_gla
from .retention import chunk_retention, fused_chunk_retention, fused_recurrent_retention
from .simple_gla import chunk_simple_gla, fused_recurrent_simple_gla, parallel_simple_gla

__all__ = [
    "chunk_gla", "fused_recurrent_gla",
    "chunk_simple_gla", "fused_recurrent_simple_gla",
    "chunk_retention", "fused_recurrent_retention",
    "chunk_delta_rule", "fused_recurrent_delta_rule",
    "chunk_gated_delta_rule", "fused_recurrent_gated_delta_rule",
    "fused_chunk_gla", "fused_chunk_retention", "fused_chunk_delta_rule", "parallel_simple_gla",
]
