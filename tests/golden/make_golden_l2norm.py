"""Generate tests/golden/l2norm_vectors.npz from the reference's own l2norm kernels.

The reference has no CPU implementation of this step: its forward and backward are Triton kernels
(fla/modules/l2norm.py:15 and :50). They are run here, unmodified, through Triton's interpreter on CPU tensors
(TRITON_INTERPRET=1), launched with the arguments the reference's own wrappers pass (fla/modules/l2norm.py:117-128,
:159-167); only the autotuner around them is bypassed (it benchmarks on a GPU), which does not change a result.

    FLA_REFERENCE=<path to flash-linear-attention> python tests/golden/make_golden_l2norm.py
"""
import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

REF = os.environ.get("FLA_REFERENCE")
if not REF or not os.path.isfile(os.path.join(REF, "fla/modules/l2norm.py")):
    sys.exit("set FLA_REFERENCE to the path of a flash-linear-attention checkout")
spec = importlib.util.spec_from_file_location("ref_l2norm", os.path.join(REF, "fla/modules/l2norm.py"))
ref = importlib.util.module_from_spec(spec)
spec.loader.exec_module(ref)
fwd_kernel, bwd_kernel = ref.l2norm_fwd_kernel.fn, ref.l2norm_bwd_kernel.fn  # the jitted functions under the autotuner


def next_pow2(n):
    return 1 << (n - 1).bit_length()


def run(x, dy, eps_f, eps_b):
    M, N = x.shape
    y, dx = torch.empty_like(x), torch.empty_like(x)
    fwd_kernel[(M,)](x, y, x.stride(0), N, eps_f, BLOCK_N=next_pow2(N))
    bwd_kernel[(M,)](x, dy, dx, x.stride(0), N, eps_b, BLOCK_N=next_pow2(N))
    return y, dx


out = {}
g = torch.Generator().manual_seed(7)
for name, (M, N, dt, scale) in {"f32_128": (37, 128, torch.float32, 1.0), "f32_100": (9, 100, torch.float32, 3.0),
                                "f16_64": (21, 64, torch.float16, 1.0), "f32_tiny": (5, 128, torch.float32, 1e-4)}.items():
    x = (torch.randn(M, N, generator=g) * scale).to(dt)
    dy = torch.randn(M, N, generator=g).to(dt)
    # the reference's defaults: eps = 1e-6 in l2_norm / L2NormFunction for both directions (fla/modules/l2norm.py:176-192)
    y, dx = run(x, dy, 1e-6, 1e-6)
    for k, v in (("x", x), ("dy", dy), ("y", y), ("dx", dx)):
        out[f"{name}.{k}"] = v.numpy()
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "l2norm_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, {k: v.shape for k, v in out.items() if k.endswith(".x")})
