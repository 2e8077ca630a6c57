"""CPU restatement of the reference's row-wise L2 normalisation.  TEST INFRASTRUCTURE ONLY.

Follows the arithmetic of the reference's kernels, fp32 throughout with the result cast to the output type:
forward fla/modules/l2norm.py:28-36, backward fla/modules/l2norm.py:70-85. Pinned in
tests/test_oracle_golden.py against tests/golden/l2norm_vectors.npz, which holds outputs of those very kernels
(run through Triton's CPU interpreter by tests/golden/make_golden_l2norm.py).
"""
import torch


def l2_norm(x: torch.Tensor, eps: float = 1e-6, output_dtype=None) -> torch.Tensor:
    xf = x.float()
    var = (xf * xf).sum(-1, keepdim=True)
    rstd = 1.0 / torch.sqrt(var + eps)
    return (xf * rstd).to(output_dtype or x.dtype)


def l2_norm_bwd(x: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf, gf = x.float(), dy.float()
    var = (xf * xf).sum(-1, keepdim=True)
    rstd = 1.0 / torch.sqrt(var + eps)
    dx = gf * rstd - (gf * xf).sum(-1, keepdim=True) * (1.0 / (var + eps)) * rstd * xf
    return dx.to(x.dtype)
