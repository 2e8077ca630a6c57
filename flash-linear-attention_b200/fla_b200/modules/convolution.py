# -*- coding: utf-8 -*-
"""Causal depthwise short convolution with the interface of fla/modules/convolution.py (`ShortConvolution` :79):
`forward(x, mask=None, cache=None, output_final_state=False) -> (y, cache)` on `[B, T, D]`, the cache `[B, D, W]`
updated in place, and the one-token `step`. The reference computes it with the `causal_conv1d` package or with
`nn.Conv1d`; here it is one CUDA kernel per direction (csrc/short_conv.cu)."""
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib
from .._lib import _DTYPES


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_lib.load().flab_last_error().decode()}")
    _lib.LAUNCHES += 1


def _f32(t):
    return None if t is None else t.detach().float().contiguous()


def _p(t):
    return None if t is None else t.data_ptr()


class ShortConvFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, bias, silu):
        if not x.is_cuda:
            raise RuntimeError("flab200 kernels run on CUDA tensors only (no CPU fallback)")
        lib = _lib.load()
        x = x.contiguous()
        B, T, D = x.shape
        w32, b32 = _f32(weight.reshape(D, -1)), _f32(bias)
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _ok(lib.flab_short_conv_fwd(x.data_ptr(), w32.data_ptr(), _p(b32), y.data_ptr(), B, T, D, w32.shape[1], int(silu),
                                        _DTYPES[x.dtype], torch.cuda.current_stream(x.device).cuda_stream), "flab_short_conv_fwd")
        ctx.save_for_backward(x, w32, b32)
        ctx.silu, ctx.w_shape, ctx.w_dtype, ctx.b_dtype = silu, weight.shape, weight.dtype, None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w32, b32 = ctx.saved_tensors
        lib = _lib.load()
        B, T, D = x.shape
        dy = dy.to(x.dtype).contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w32)
        db = None if b32 is None else torch.zeros_like(b32)
        with torch.cuda.device(x.device):
            _ok(lib.flab_short_conv_bwd(x.data_ptr(), w32.data_ptr(), _p(b32), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(), _p(db), B, T, D,
                                        w32.shape[1], int(ctx.silu), _DTYPES[x.dtype], torch.cuda.current_stream(x.device).cuda_stream),
                "flab_short_conv_bwd")
        return dx, dw.reshape(ctx.w_shape).to(ctx.w_dtype), None if db is None else db.to(ctx.b_dtype), None


class ShortConvolution(nn.Conv1d):
    """`nn.Conv1d` (depthwise, causal) that takes the channel dimension last."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = "silu",
                 use_fast_conv1d: Optional[bool] = True):
        super().__init__(in_channels=hidden_size, out_channels=hidden_size, kernel_size=kernel_size, groups=hidden_size, bias=bias,
                         padding=kernel_size - 1)
        self.hidden_size = hidden_size
        self.activation = None
        if activation is not None:
            assert activation in ["silu", "swish"], f"Activation `{activation}` not supported yet."
            self.activation = activation
        self.use_fast_conv1d = use_fast_conv1d  # kept for signature compatibility: there is one implementation here

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None, cache: Optional[torch.Tensor] = None,
                output_final_state: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        batch_size, _, hidden_size = x.shape
        if mask is not None:
            x = x.mul_(mask.unsqueeze(-1))
        if output_final_state and cache is None:
            cache = x.new_zeros(batch_size, hidden_size, self.kernel_size[0])
        if cache is not None and x.shape[1] == 1:
            return self.step(x, cache)
        if cache is not None:  # the last W inputs, [B, D, W] (fla/modules/convolution.py:176-177)
            cache.copy_(F.pad(x.transpose(1, 2), (self.kernel_size[0] - x.shape[1], 0)))
        y = ShortConvFn.apply(x, self.weight, self.bias, self.activation is not None)
        return y, cache

    def step(self, x: torch.Tensor, cache: torch.Tensor):
        assert x.shape[1] == 1, "Only support decoding with 1 token at a time for now"
        lib = _lib.load()
        B, _, D = x.shape
        W = self.kernel_size[0]
        assert cache.is_contiguous() and cache.shape == (B, D, W) and cache.dtype == x.dtype
        xs = x.squeeze(1).contiguous()
        y = torch.empty_like(xs)
        w32, b32 = _f32(self.weight.reshape(D, W)), _f32(self.bias)
        with torch.cuda.device(x.device):
            _ok(lib.flab_short_conv_update(xs.data_ptr(), cache.data_ptr(), w32.data_ptr(), _p(b32), y.data_ptr(), B, D, W,
                                           int(self.activation is not None), _DTYPES[x.dtype],
                                           torch.cuda.current_stream(x.device).cuda_stream), "flab_short_conv_update")
        return y.unsqueeze(1), cache

    @property
    def state_size(self) -> int:
        return self.hidden_size * self.kernel_size[0]
