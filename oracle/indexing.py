"""Integer chunk tables for variable-length batches, restated with the same torch expressions the
reference uses, so the host-side tables of the CUDA path can be compared bit for bit."""

import torch


def _cdiv(a, b):
    return -(a // -b)


def chunk_indices_ref(offsets: torch.Tensor, chunk_size: int = 64) -> torch.Tensor:
    """[NT, 2] rows (sequence id, chunk id in sequence); fla/ops/gated_delta_rule/chunk.py:204-207."""
    counts = _cdiv(offsets[1:] - offsets[:-1], chunk_size).tolist()
    indices = torch.cat([torch.arange(n) for n in counts])
    return torch.stack([indices.eq(0).cumsum(0) - 1, indices], 1).to(offsets)


def chunk_offsets_ref(offsets: torch.Tensor, chunk_size: int = 64) -> torch.Tensor:
    """[N+1] exclusive prefix sum of per-sequence chunk counts; fla/ops/common/chunk_h.py:274-279."""
    counts = _cdiv(offsets[1:] - offsets[:-1], chunk_size)
    return torch.cat([offsets.new_tensor([0]), counts]).cumsum(-1)
