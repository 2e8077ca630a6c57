"""CPU restatement of the reference's RMS norm (with weight) times swish gate.  TEST INFRASTRUCTURE ONLY.

Follows the arithmetic of the reference's kernels for IS_RMS_NORM with a weight and no bias / residual, fp32 throughout
with results cast to the input type: forward fla/modules/fused_norm_gate.py:70-100, backward :254-290 (dw is the sum
over rows of dy' * xhat, which the reference accumulates per program and sums at :385-386). Pinned in
tests/test_oracle_golden.py against tests/golden/norm_gate_vectors.npz: outputs of those kernels run through
Triton's CPU interpreter by tests/golden/make_golden_norm_gate.py.
"""
import torch


def rms_norm_swish_gate(x, gate, weight, eps=1e-6):
    xf, gf, wf = x.float(), gate.float(), weight.float()
    rstd = 1.0 / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
    return (xf * rstd * wf * gf * torch.sigmoid(gf)).to(x.dtype)


def rms_norm_swish_gate_bwd(x, gate, weight, dy, eps=1e-6):
    """Returns (dx, dgate, dw); dw in fp32."""
    xf, gf, wf, df = x.float(), gate.float(), weight.float(), dy.float()
    n = xf.shape[-1]
    rstd = 1.0 / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
    xhat = xf * rstd
    s = torch.sigmoid(gf)
    dg = df * (xhat * wf) * (s + gf * s * (1 - s))
    d2 = df * gf * s
    wdy = d2 * wf
    dw = (d2 * xhat).reshape(-1, n).sum(0)
    c1 = (xhat * wdy).sum(-1, keepdim=True) / n
    dx = (wdy - xhat * c1) * rstd
    return dx.to(x.dtype), dg.to(x.dtype), dw
