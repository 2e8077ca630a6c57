"""CPU restatement of the reference's causal depthwise short convolution.  TEST INFRASTRUCTURE ONLY.

Follows fla/modules/convolution.py: forward :171-187 (`nn.Conv1d` with left padding W-1, first T outputs, then the
activation x * sigmoid(x)), cache :176-177 (the last W inputs, `[B, D, W]`, left-padded with zeros), decode step
:204-213 (shift the cache by one, append x, dot with the filter). Gradients by autograd. Pinned in
tests/test_oracle_golden.py against tests/golden/short_conv_vectors.npz (outputs of the reference's module on CPU,
tests/golden/make_golden_short_conv.py).
"""
import torch
import torch.nn.functional as F


def short_conv(x, weight, bias=None, silu=True):
    """x [B, T, D], weight [D, 1, W] or [D, W]. Returns (y [B, T, D], cache [B, D, W])."""
    B, T, D = x.shape
    w = weight.reshape(D, 1, -1).float()
    W = w.shape[-1]
    xt = x.float().transpose(1, 2)
    pre = F.conv1d(xt, w, None if bias is None else bias.float(), padding=W - 1, groups=D)[..., :T]
    y = pre * torch.sigmoid(pre) if silu else pre
    cache = F.pad(xt, (W - T, 0)) if T < W else xt[..., T - W:]
    return y.transpose(1, 2).to(x.dtype), cache.to(x.dtype)


def short_conv_step(x, cache, weight, bias=None, silu=True):
    """x [B, 1, D], cache [B, D, W]. Returns (y [B, 1, D], new cache)."""
    D = x.shape[-1]
    w = weight.reshape(D, -1).float()
    c = torch.cat([cache[..., 1:], x.transpose(1, 2)], dim=-1)
    pre = (c.float() * w).sum(-1)
    if bias is not None:
        pre = pre + bias.float()
    y = pre * torch.sigmoid(pre) if silu else pre
    return y.unsqueeze(1).to(x.dtype), c
