# -*- coding: utf-8 -*-
"""Gate and beta of the gated delta rule layer, as ONE fused elementwise step with the gate's chunk-local cumulative
sum (fla/layers/gated_deltanet.py:236-237 followed by fla/ops/gated_delta_rule/chunk.py:33):

    beta = b.sigmoid();   g = -A_log.float().exp() * softplus(a.float() + dt_bias)

`gdn_gate_beta(a, b, A_log, dt_bias)` returns `(g, beta)` like those two lines (g fp32, beta in b's dtype) and is
differentiable in a, b, A_log and dt_bias. The cumulative sum computed by the same kernel travels with `g`: when that
very tensor is passed to `chunk_gated_delta_rule` (same layout, same offsets, unmodified) the op skips its own cumsum
launch."""
import ctypes
import weakref
from typing import Optional, Tuple

import torch

from .. import _lib
from ..utils import Geometry, resolve_offsets

_CUMSUMS = {}  # id(g) -> (weakref to g, version, head_first, id of the offsets tensor, g_cumsum)


def attached_cumsum(g: torch.Tensor, offsets, head_first: bool) -> Optional[torch.Tensor]:
    """The chunk-local cumsum computed together with `g` by `gdn_gate_beta`, if `g` is that tensor, unmodified, and the
    layout and offsets agree; else None."""
    hit = _CUMSUMS.get(id(g))
    if hit is None or hit[0]() is not g or hit[1] != g._version or hit[2] != bool(head_first) or hit[3] != (None if offsets is None else id(offsets)):
        return None
    return hit[4]


def _attach(g, g_cum, offsets, head_first):
    if len(_CUMSUMS) > 64:
        for key in [k_ for k_, v_ in _CUMSUMS.items() if v_[0]() is None]:
            del _CUMSUMS[key]
        if len(_CUMSUMS) > 64:
            _CUMSUMS.clear()
    _CUMSUMS[id(g)] = (weakref.ref(g), g._version, bool(head_first), None if offsets is None else id(offsets), g_cum)


def _geo_args(x: torch.Tensor, offsets, head_first):
    geo = Geometry(x.unsqueeze(-1), None, offsets, head_first)
    return geo, _lib.fill_args(x, **geo.kw())


class GdnGateBetaFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, a, b, A_log, dt_bias, offsets, head_first):
        if not a.is_cuda:
            raise RuntimeError("flab200 kernels run on CUDA tensors only (no CPU fallback)")
        a, b = a.contiguous(), b.contiguous()
        assert a.shape == b.shape and a.dim() == 3 and a.dtype == b.dtype, "a and b must both be [B,T,H] (or [B,H,T]) of one dtype"
        A32 = A_log.detach().float().contiguous()
        bias32 = None if dt_bias is None else dt_bias.detach().float().contiguous()
        _, args = _geo_args(a, offsets, head_first)
        g = torch.empty(a.shape, dtype=torch.float32, device=a.device)
        g_cum = torch.empty_like(g)
        beta = torch.empty_like(b)
        lib = _lib.load()
        with torch.cuda.device(a.device):
            rc = lib.flab_gdn_gate_fwd(ctypes.byref(args), a.data_ptr(), b.data_ptr(), A32.data_ptr(),
                                       None if bias32 is None else bias32.data_ptr(), g.data_ptr(), g_cum.data_ptr(), beta.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"flab_gdn_gate_fwd failed ({rc}): {lib.flab_last_error().decode()}")
        _lib.LAUNCHES += 1
        ctx.save_for_backward(a, b, A32, bias32)
        ctx.offsets, ctx.head_first = offsets, head_first
        ctx.A_dtype, ctx.bias_dtype = A_log.dtype, (None if dt_bias is None else dt_bias.dtype)
        ctx.mark_non_differentiable(g_cum)
        return g, beta, g_cum

    @staticmethod
    def backward(ctx, dg, dbeta, _):
        a, b, A32, bias32 = ctx.saved_tensors
        _, args = _geo_args(a, ctx.offsets, ctx.head_first)
        dg = torch.zeros_like(a, dtype=torch.float32) if dg is None else dg.float().contiguous()
        dbeta = torch.zeros_like(b) if dbeta is None else dbeta.to(b.dtype).contiguous()
        da, db = torch.empty_like(a), torch.empty_like(b)
        dA = torch.zeros_like(A32)
        dbias = None if bias32 is None else torch.zeros_like(bias32)
        lib = _lib.load()
        with torch.cuda.device(a.device):
            rc = lib.flab_gdn_gate_bwd(ctypes.byref(args), a.data_ptr(), b.data_ptr(), A32.data_ptr(),
                                       None if bias32 is None else bias32.data_ptr(), dg.data_ptr(), dbeta.data_ptr(), da.data_ptr(),
                                       db.data_ptr(), dA.data_ptr(), None if dbias is None else dbias.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"flab_gdn_gate_bwd failed ({rc}): {lib.flab_last_error().decode()}")
        _lib.LAUNCHES += 1
        return da, db, dA.to(ctx.A_dtype), (None if dbias is None else dbias.to(ctx.bias_dtype)), None, None


def gdn_gate_beta(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: Optional[torch.Tensor] = None,
                  offsets: Optional[torch.Tensor] = None, head_first: bool = False,
                  cu_seqlens: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """a, b: `[B, T, H]` outputs of the layer's `a_proj` / `b_proj` (`[B, H, T]` with head_first); A_log, dt_bias: `[H]`.
    Returns (g `[B, T, H]` fp32 log decay, beta in b's dtype)."""
    offsets = resolve_offsets(offsets, cu_seqlens)
    g, beta, g_cum = GdnGateBetaFunction.apply(a, b, A_log, dt_bias, offsets, head_first)
    _attach(g, g_cum, offsets, head_first)
    return g, beta
