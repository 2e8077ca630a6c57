"""Generate tests/golden/short_conv_vectors.npz from the reference's own ShortConvolution module
(fla/modules/convolution.py:79), run on CPU through its `use_fast_conv1d=False` path (nn.Conv1d; the other path needs
the third-party causal_conv1d package): forward with cache, all gradients by autograd, and decode steps. The module is
built with activation=None and the activation is applied here with torch (x * sigmoid(x)): the reference's own "silu"
entry is a CUDA-only jiterator function (fla/modules/activations.py) of the same formula.

    FLA_REFERENCE=<path to flash-linear-attention> python tests/golden/make_golden_short_conv.py
"""
import os
import sys
import types
import warnings

import numpy as np
import torch

REF = os.environ.get("FLA_REFERENCE")
if not REF or not os.path.isfile(os.path.join(REF, "fla/modules/convolution.py")):
    sys.exit("set FLA_REFERENCE to the path of a flash-linear-attention checkout")
stub = types.ModuleType("fla")
stub.__path__ = [os.path.join(REF, "fla")]
sys.modules["fla"] = stub
mods = types.ModuleType("fla.modules")
mods.__path__ = [os.path.join(REF, "fla/modules")]
sys.modules["fla.modules"] = mods
warnings.simplefilter("ignore")
from fla.modules.convolution import ShortConvolution  # noqa: E402

out = {}
g = torch.Generator().manual_seed(21)
for name, (B, T, D, W, bias, act) in {"w4_silu": (2, 37, 64, 4, False, "silu"), "w3_bias": (1, 70, 32, 3, True, None),
                                      "w2_silu_bias": (3, 9, 16, 2, True, "silu")}.items():
    conv = ShortConvolution(D, W, bias=bias, activation=None, use_fast_conv1d=False)
    act_fn = (lambda v: v * torch.sigmoid(v)) if act else (lambda v: v)
    with torch.no_grad():
        conv.weight.copy_(torch.randn(D, 1, W, generator=g) * 0.5)
        if bias:
            conv.bias.copy_(torch.randn(D, generator=g) * 0.1)
    x = torch.randn(B, T, D, generator=g, requires_grad=True)
    dy = torch.randn(B, T, D, generator=g)
    y, cache = conv(x, output_final_state=True)
    y = act_fn(y)
    gx, gw, *gb = torch.autograd.grad((y * dy).sum(), [x, conv.weight] + ([conv.bias] if bias else []))
    rec = {"silu": torch.tensor(1 if act else 0), "x": x, "dy": dy, "weight": conv.weight, "y": y, "cache": cache, "dx": gx, "dweight": gw}
    if bias:
        rec["bias"], rec["dbias"] = conv.bias, gb[0]
    # three decode steps continuing from the cache
    xs = torch.randn(B, 3, D, generator=g)
    c = cache.detach().clone()
    ys = []
    with torch.no_grad():
        for t in range(3):
            yt, c = conv(xs[:, t:t + 1], cache=c)
            ys.append(act_fn(yt))
    rec["step_x"], rec["step_y"], rec["step_cache"] = xs, torch.cat(ys, 1), c
    for k, v in rec.items():
        out[f"{name}.{k}"] = v.detach().numpy()
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "short_conv_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, "%.0f KB" % (os.path.getsize(path) / 1024))
