# -*- coding: utf-8 -*-
"""Host-side helpers shared by the op wrappers: argument normalisation, variable-length chunk
tables (the integer index data of this path) and the autograd decorators the reference applies
(fla/utils.py:10-21 `contiguous`, :88-93 autocast wrappers)."""

import functools
import os
import weakref
from collections import namedtuple
from typing import Optional

import torch

from ._lib import CHUNK

# Keep the chunk states (and the WY factors) computed in forward for backward instead of recomputing
# them as the reference does: costs ~4 extra [B,T,H,D] activations, saves two kernel launches and a
# full serial state scan in backward.  FLA_B200_SAVE_STATES=0 restores the recomputing behaviour.
SAVE_STATES = os.environ.get("FLA_B200_SAVE_STATES", "1") != "0"

Varlen = namedtuple("Varlen", ["cu_seqlens", "chunk_indices", "chunk_offsets", "N", "NT", "lengths"])


def contiguous(fn):
    """Make every tensor argument contiguous before the autograd Function body runs."""
    @functools.wraps(fn)
    def wrapper(ctx, *args, **kwargs):
        return fn(ctx,
                  *(i if not isinstance(i, torch.Tensor) else i.contiguous() for i in args),
                  **{k: (v if not isinstance(v, torch.Tensor) else v.contiguous()) for k, v in kwargs.items()})
    return wrapper


autocast_custom_fwd = functools.partial(torch.amp.custom_fwd, device_type="cuda")
autocast_custom_bwd = functools.partial(torch.amp.custom_bwd, device_type="cuda")


def chunk_tables(lengths, chunk_size: int = CHUNK):
    """Integer chunk tables for a list of sequence lengths.

    Returns (indices, chunk_offsets): `indices[c] = (sequence id, chunk id inside that sequence)` for
    every chunk in sequence order, and `chunk_offsets[n]` = number of chunks before sequence n
    (length N+1).  Same values as the reference builds in
    fla/ops/gated_delta_rule/chunk.py:204-207 and fla/ops/common/chunk_h.py:274-279.
    """
    indices, chunk_offsets, total = [], [0], 0
    for n, length in enumerate(lengths):
        nt = -(-int(length) // chunk_size)
        indices.extend((n, i) for i in range(nt))
        total += nt
        chunk_offsets.append(total)
    return indices, chunk_offsets


_VARLEN_CACHE = {}  # id(offsets tensor) -> (weakref to it, its version counter, Varlen)


def prepare_varlen(offsets: Optional[torch.Tensor], device) -> Optional[Varlen]:
    """Device-resident int32 tables for `offsets` (int32 or int64, [N+1]).

    Reading `offsets` on the host costs one device-to-host copy, like the reference's `.tolist()`.
    The result is cached per tensor OBJECT (validated through a weak reference and the tensor's
    version counter), never per address: the allocator reuses addresses, and a table built for
    another batch would silently index the wrong tokens.
    """
    if offsets is None:
        return None
    key = id(offsets)
    hit = _VARLEN_CACHE.get(key)
    if hit is not None and hit[0]() is offsets and hit[1] == offsets._version and hit[2].cu_seqlens.device == torch.device(device):
        return hit[2]
    host = [int(x) for x in offsets.tolist()]
    if len(host) < 2 or host[0] != 0 or any(b < a for a, b in zip(host, host[1:])):
        raise ValueError(f"`offsets` must start at 0 and be non-decreasing, got {host[:8]}...")
    lengths = [b - a for a, b in zip(host, host[1:])]
    indices, chunk_offsets = chunk_tables(lengths)
    cu = torch.tensor(host, dtype=torch.int32, device=device)
    idx = torch.tensor(indices if indices else [(0, 0)], dtype=torch.int32, device=device).reshape(-1, 2)
    co = torch.tensor(chunk_offsets, dtype=torch.int32, device=device)
    out = Varlen(cu, idx, co, len(lengths), len(indices), lengths)
    if len(_VARLEN_CACHE) > 64:
        _VARLEN_CACHE.clear()
    _VARLEN_CACHE[key] = (weakref.ref(offsets), offsets._version, out)
    return out


def varlen_from_lengths(lengths, device) -> Varlen:
    """The same tables as `prepare_varlen`, from sequence lengths already known on the host (no device read)."""
    host = [0]
    for L in lengths:
        host.append(host[-1] + int(L))
    indices, chunk_offsets = chunk_tables(lengths)
    cu = torch.tensor(host, dtype=torch.int32, device=device)
    idx = torch.tensor(indices if indices else [(0, 0)], dtype=torch.int32, device=device).reshape(-1, 2)
    co = torch.tensor(chunk_offsets, dtype=torch.int32, device=device)
    return Varlen(cu, idx, co, len(lengths), len(indices), list(lengths))


def resolve_offsets(offsets, cu_seqlens):
    """`cu_seqlens=` is accepted as an alias of the reference's `offsets=` keyword."""
    if offsets is not None and cu_seqlens is not None:
        raise ValueError("pass either `offsets` or `cu_seqlens`, not both")
    return offsets if offsets is not None else cu_seqlens


class Geometry:
    """Shape bookkeeping for one op call (seq-first or head-first, fixed or variable length)."""

    def __init__(self, k: torch.Tensor, v: Optional[torch.Tensor], offsets, head_first: bool):
        if head_first:
            self.B, self.H, self.T, self.K = k.shape
        else:
            self.B, self.T, self.H, self.K = k.shape
        self.V = v.shape[-1] if v is not None else 0
        self.head_first = bool(head_first)
        self.offsets_tensor = offsets
        self.varlen = prepare_varlen(offsets, k.device)
        if self.varlen is not None:
            self.N, self.NT = self.varlen.N, self.varlen.NT
        else:
            self.N, self.NT = self.B, self.B * (-(-self.T // CHUNK))

    @classmethod
    def packed(cls, k: torch.Tensor, v: Optional[torch.Tensor], varlen: Varlen) -> "Geometry":
        """Geometry of sequences packed seq-first into B = 1 (`k` is `[1, T, H, K]`), from ready-made tables."""
        geo = cls.__new__(cls)
        geo.B, geo.T, geo.H, geo.K = k.shape
        geo.V = v.shape[-1] if v is not None else 0
        geo.head_first = False
        geo.offsets_tensor = varlen.cu_seqlens
        geo.varlen = varlen
        geo.N, geo.NT = varlen.N, varlen.NT
        return geo

    def kw(self):
        return dict(B=self.B, T=self.T, H=self.H, K=self.K, V=self.V, N=self.N, NT=self.NT,
                    head_first=self.head_first, varlen=self.varlen)
