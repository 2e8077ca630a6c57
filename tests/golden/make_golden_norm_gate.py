"""Generate tests/golden/norm_gate_vectors.npz from the reference's own norm-gate kernels.

The reference's layer_norm_fwd_kernel / layer_norm_bwd_kernel (fla/modules/fused_norm_gate.py:33, :182) are run
unmodified through Triton's interpreter on CPU tensors (TRITON_INTERPRET=1), launched with the arguments their
wrappers pass for the RMS-norm + weight case (:150-172, :352-384); the wrappers themselves allocate on "cuda" and the
backward one sits under an autotuner that benchmarks on a GPU, so the jitted functions are called directly, one
program per block of rows exactly like the wrapper's grid.

    FLA_REFERENCE=<path to flash-linear-attention> python tests/golden/make_golden_norm_gate.py
"""
import importlib.util
import math
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

REF = os.environ.get("FLA_REFERENCE")
if not REF or not os.path.isfile(os.path.join(REF, "fla/modules/fused_norm_gate.py")):
    sys.exit("set FLA_REFERENCE to the path of a flash-linear-attention checkout")
stub = types.ModuleType("fla")
stub.__path__ = [os.path.join(REF, "fla")]
sys.modules["fla"] = stub
spec = importlib.util.spec_from_file_location("ref_norm_gate", os.path.join(REF, "fla/modules/fused_norm_gate.py"))
ref = importlib.util.module_from_spec(spec)
spec.loader.exec_module(ref)


def unwrap(k):
    while not type(k).__name__.startswith("Interpreted") and hasattr(k, "fn"):
        k = k.fn
    return k


fwd_kernel, bwd_kernel = unwrap(ref.layer_norm_fwd_kernel), unwrap(ref.layer_norm_bwd_kernel)


def run(x, o, w, dy, eps, programs):
    M, N = x.shape
    BLOCK_N = 1 << (N - 1).bit_length()
    y = torch.empty_like(x)
    rstd = torch.empty(M, dtype=torch.float32)
    fwd_kernel[(M,)](x, o, y, w, None, None, None, None, rstd, x.stride(0), y.stride(0), 0, 0, N, eps,
                     IS_RMS_NORM=True, BLOCK_N=BLOCK_N, HAS_RESIDUAL=False, STORE_RESIDUAL_OUT=False, HAS_WEIGHT=True, HAS_BIAS=False)
    dx, do = torch.empty_like(x), torch.empty_like(o)
    dwp = torch.empty(programs, N, dtype=torch.float32)
    rows_per_program = math.ceil(M / programs)
    bwd_kernel[(programs,)](x, o, w, None, None, dy, dx, do, dwp, None, None, None, None, rstd, x.stride(0), 0, dy.stride(0),
                            dx.stride(0), 0, 0, M, N, eps, rows_per_program, IS_RMS_NORM=True, BLOCK_N=BLOCK_N, HAS_DRESIDUAL=False,
                            STORE_DRESIDUAL=False, HAS_WEIGHT=True, HAS_BIAS=False, RECOMPUTE_OUTPUT=False)
    return y, dx, do, dwp.sum(0)


out = {}
g = torch.Generator().manual_seed(3)
for name, (M, N, dt) in {"f32_128": (37, 128, torch.float32), "f16_128": (50, 128, torch.float16), "f32_100": (9, 100, torch.float32),
                         "f16_64": (21, 64, torch.float16)}.items():
    x = torch.randn(M, N, generator=g).to(dt)
    o = torch.randn(M, N, generator=g).to(dt)
    w = (1 + 0.1 * torch.randn(N, generator=g))
    dy = torch.randn(M, N, generator=g).to(dt)
    y, dx, do, dw = run(x, o, w, dy, 1e-5, 4)
    for k, v in (("x", x), ("gate", o), ("w", w), ("dy", dy), ("y", y), ("dx", dx), ("dgate", do), ("dw", dw)):
        out[f"{name}.{k}"] = v.numpy()
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "norm_gate_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, "%.0f KB" % (os.path.getsize(path) / 1024))
