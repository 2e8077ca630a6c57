# -*- coding: utf-8 -*-
"""RMS norm with a weight, times a swish gate, with the names of fla/modules/fused_norm_gate.py
(`rms_norm_swish_gate_fn` :610, `FusedRMSNormSwishGate` :728): the delta-rule layers apply it to the op's output and
the gate projection (fla/layers/gated_deltanet.py:278-280). Covers what those layers use: weight, no bias, no
residual; the other arguments of the reference are accepted and rejected with a message when set."""
from typing import Optional

import torch
import torch.nn as nn

from .. import _lib
from .._lib import _DTYPES


def _rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.is_contiguous() else x2.contiguous()


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_lib.load().flab_last_error().decode()}")
    _lib.LAUNCHES += 1


class RMSNormSwishGateFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, o, weight, eps=1e-6):
        if not x.is_cuda:
            raise RuntimeError("flab200 kernels run on CUDA tensors only (no CPU fallback)")
        lib = _lib.load()
        x2, g2 = _rows(x), _rows(o.to(x.dtype))
        assert g2.shape == x2.shape and weight.shape == (x2.shape[1],)
        w32 = weight.detach().float().contiguous()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _check(lib.flab_rms_norm_swish_gate_fwd(x2.data_ptr(), g2.data_ptr(), w32.data_ptr(), y.data_ptr(), rstd.data_ptr(), x2.shape[0],
                                                    x2.shape[1], _DTYPES[x2.dtype], float(eps),
                                                    torch.cuda.current_stream(x.device).cuda_stream), "flab_rms_norm_swish_gate_fwd")
        ctx.save_for_backward(x2, g2, w32, rstd)
        ctx.shapes, ctx.w_dtype, ctx.o_dtype = (x.shape, o.shape), weight.dtype, o.dtype
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, g2, w32, rstd = ctx.saved_tensors
        lib = _lib.load()
        dy2 = _rows(dy.to(x2.dtype))
        dx, dg = torch.empty_like(x2), torch.empty_like(x2)
        rows, n = x2.shape
        parts = lib.flab_rms_norm_swish_gate_partials(rows, n, _DTYPES[x2.dtype])
        dwp = torch.empty(parts, n, dtype=torch.float32, device=x2.device)
        if rows == 0:
            dwp.zero_()
        with torch.cuda.device(x2.device):
            _check(lib.flab_rms_norm_swish_gate_bwd(x2.data_ptr(), g2.data_ptr(), w32.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                                    dg.data_ptr(), dwp.data_ptr(), rows, n, _DTYPES[x2.dtype],
                                                    torch.cuda.current_stream(x2.device).cuda_stream), "flab_rms_norm_swish_gate_bwd")
        dw = dwp.sum(0).to(ctx.w_dtype)
        return dx.reshape(ctx.shapes[0]), dg.reshape(ctx.shapes[1]).to(ctx.o_dtype), dw, None


def rms_norm_swish_gate_fn(x, o, weight, bias=None, residual=None, prenorm=False, residual_in_fp32=False, eps=1e-6):
    if bias is not None or residual is not None or prenorm or residual_in_fp32:
        raise NotImplementedError("rms_norm_swish_gate_fn: bias, residual, prenorm and residual_in_fp32 are not built "
                                  "(the delta-rule layers use none of them)")
    return RMSNormSwishGateFn.apply(x, o, weight, eps)


class FusedRMSNormSwishGate(nn.Module):

    def __init__(self, hidden_size, elementwise_affine: bool = True, eps=1e-5) -> "FusedRMSNormSwishGate":
        super().__init__()
        if not elementwise_affine:
            raise NotImplementedError("FusedRMSNormSwishGate without a weight is not built")
        self.hidden_size = hidden_size
        self.elementwise_affine = elementwise_affine
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.register_parameter("bias", None)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}({self.hidden_size}, eps={self.eps})"

    def forward(self, x, o, residual=None, prenorm=False, residual_in_fp32=False):
        return rms_norm_swish_gate_fn(x, o, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm,
                                      residual_in_fp32=residual_in_fp32)
