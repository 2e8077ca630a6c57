# -*- coding: utf-8 -*-
"""Row-wise L2 normalisation with the names and signatures of fla/modules/l2norm.py
(`l2norm_fwd` :89, `l2norm_bwd` :131, `L2NormFunction` :170, `l2_norm` :195): q and k of the delta-rule layers
pass through it right before the chunk op (fla/layers/gated_deltanet.py:234-235)."""
from typing import Optional

import torch

from .. import _lib
from .._lib import _DTYPES


def _rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.is_contiguous() else x2.contiguous()


def _stream(x: torch.Tensor):
    return torch.cuda.current_stream(x.device).cuda_stream


def l2norm_fwd(x: torch.Tensor, eps: float = 1e-6, output_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("flab200 kernels run on CUDA tensors only (no CPU fallback)")
    x2 = _rows(x)
    if x2.shape[-1] * x2.element_size() > 65536:
        raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")
    y = torch.empty_like(x2, dtype=output_dtype or x.dtype)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.flab_l2norm_fwd(x2.data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1], _DTYPES[x2.dtype], _DTYPES[y.dtype],
                                 float(eps), _stream(x))
    if rc != 0:
        raise RuntimeError(f"flab_l2norm_fwd failed ({rc}): {lib.flab_last_error().decode()}")
    _lib.LAUNCHES += 1
    return y.reshape(x.shape)


def l2norm_bwd(x: torch.Tensor, dy: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("flab200 kernels run on CUDA tensors only (no CPU fallback)")
    x2 = _rows(x)
    dy2 = _rows(dy.to(x.dtype))
    assert dy2.shape == x2.shape
    dx = torch.empty_like(x2)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.flab_l2norm_bwd(x2.data_ptr(), dy2.data_ptr(), dx.data_ptr(), x2.shape[0], x2.shape[1], _DTYPES[x2.dtype],
                                 float(eps), _stream(x))
    if rc != 0:
        raise RuntimeError(f"flab_l2norm_bwd failed ({rc}): {lib.flab_last_error().decode()}")
    _lib.LAUNCHES += 1
    return dx.reshape(x.shape)


class L2NormFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, eps=1e-6, output_dtype=None):
        y = l2norm_fwd(x, eps, output_dtype)
        ctx.eps = eps
        ctx.x_dtype = x.dtype
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy, *args):
        x, = ctx.saved_tensors
        dx = l2norm_bwd(x, dy, ctx.eps)
        return dx, None, None


def l2_norm(x: torch.Tensor, eps: float = 1e-6, output_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    return L2NormFunction.apply(x, eps, output_dtype)
