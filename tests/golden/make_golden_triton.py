"""Generate tests/golden/triton_vectors.npz from the reference's own CHUNKED kernels.

The reference's chunk ops are Triton kernels; they are run here unmodified, on CPU tensors, through Triton's
interpreter (TRITON_INTERPRET=1), forward and backward, through the reference's public functions. Two things around
them are stubbed, neither of which touches a result: the autotuner (it benchmarks configurations on a GPU; the first
configuration is run as is) and `torch.cuda.get_device_capability` (reported as (10, 0), the B200, so the reference
takes the tile sizes it would take there). numpy has no bf16, so the 16-bit cases are fp16.

    FLA_REFERENCE=<path to flash-linear-attention> python tests/golden/make_golden_triton.py
"""
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402
from triton.runtime import autotuner as _at  # noqa: E402

REF = os.environ.get("FLA_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "fla")):
    sys.exit("set FLA_REFERENCE to the path of a flash-linear-attention checkout")


def _run_first(self, *args, **kwargs):
    cfg = self.configs[0]
    self.best_config = cfg
    if cfg.pre_hook is not None:
        cfg.pre_hook({**dict(zip(self.arg_names, args)), **kwargs, **cfg.all_kwargs()})
    return self.fn.run(*args, **kwargs, **cfg.all_kwargs())


_at.Autotuner.run = _run_first
torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
stub = types.ModuleType("fla")
stub.__path__ = [os.path.join(REF, "fla")]
sys.modules["fla"] = stub

from fla.ops.delta_rule.chunk import chunk_delta_rule  # noqa: E402
from fla.ops.gated_delta_rule.chunk import chunk_gated_delta_rule  # noqa: E402
from fla.ops.gated_delta_rule.fused_recurrent import fused_recurrent_gated_delta_rule  # noqa: E402
from fla.ops.gla.chunk import chunk_gla  # noqa: E402
from fla.ops.retention.chunk import chunk_retention  # noqa: E402
from fla.ops.simple_gla.chunk import chunk_simple_gla  # noqa: E402

out = {}


def record(name, fn, inputs, grad_names, extra=None):
    """inputs: dict name -> tensor (seq-first); runs fn(inputs) -> (o, ht), backward with seeded cotangents
    (forward only when grad_names is empty)."""
    g0 = torch.Generator().manual_seed(len(out) + 11)
    xs = {n: (x.clone().requires_grad_(True) if n in grad_names else x) for n, x in inputs.items()}
    o, ht = fn(xs)
    do = torch.randn(o.shape, generator=g0).to(o.dtype)
    dht = torch.randn(ht.shape, generator=g0) * 0.1
    if grad_names:
        torch.autograd.backward([o, ht], [do, dht])
    for n, x in inputs.items():
        out[f"{name}.{n}"] = x.detach().numpy()
    out[f"{name}.o"], out[f"{name}.ht"] = o.detach().numpy(), ht.detach().numpy()
    out[f"{name}.do"], out[f"{name}.dht"] = do.numpy(), dht.numpy()
    for n in grad_names:
        out[f"{name}.d{n}"] = xs[n].grad.numpy()
    for n, x in (extra or {}).items():
        out[f"{name}.{n}"] = np.asarray(x)
    print(name, "o", tuple(o.shape), "mean |o| %.4f" % o.float().abs().mean().item(), flush=True)


def base(B, T, H, K, V, dt, seed, N=None):
    g0 = torch.Generator().manual_seed(seed)
    q = F.normalize(torch.randn(B, T, H, K, generator=g0), dim=-1).to(dt)
    k = F.normalize(torch.randn(B, T, H, K, generator=g0), dim=-1).to(dt)
    v = torch.randn(B, T, H, V, generator=g0).to(dt)
    h0 = torch.randn(N or B, H, K, V, generator=g0) * 0.1
    beta = torch.rand(B, T, H, generator=g0).sigmoid().to(dt)
    g = F.logsigmoid(torch.randn(B, T, H, generator=g0))
    return dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0), g0


f16 = torch.float16
# gated delta rule, K = V = 128, three chunks with a ragged tail, initial state
d, _ = base(1, 170, 2, 128, 128, f16, 1)
record("gdn_128", lambda x: chunk_gated_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"],
                                                   output_final_state=True, head_first=False), d, ["q", "k", "v", "g", "beta", "h0"])
# gated delta rule, packed variable-length sequences
d, _ = base(1, 200, 2, 64, 64, f16, 2, N=3)
offs = torch.tensor([0, 70, 134, 200], dtype=torch.long)
record("gdn_varlen", lambda x: chunk_gated_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"],
                                                      output_final_state=True, offsets=offs, head_first=False), d,
       ["q", "k", "v", "g", "beta", "h0"], extra={"offsets": offs.numpy()})
# delta rule, K = V = 128, ragged tail.  Forward only: the reference's backward kernel of this family unpacks three
# program ids into two names (fla/ops/delta_rule/wy_fast.py:347), which plain Python (the interpreter) rejects.
d, _ = base(1, 130, 2, 128, 128, f16, 3)
d.pop("g")
record("delta_128", lambda x: chunk_delta_rule(x["q"], x["k"], x["v"], x["beta"], initial_state=x["h0"], output_final_state=True,
                                               head_first=False), d, [])
# simple GLA (scalar gate per token and head)
d, g0 = base(2, 128, 2, 64, 64, f16, 4)
d.pop("beta")
d["q"], d["k"] = torch.randn(2, 128, 2, 64, generator=g0).to(f16), torch.randn(2, 128, 2, 64, generator=g0).to(f16)
record("simple_gla", lambda x: chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True,
                                                head_first=False), d, ["q", "k", "v", "g", "h0"])
# GLA (gate per key channel), fp32 like the first configuration
d, g0 = base(1, 128, 2, 64, 64, torch.float32, 5)
d.pop("beta")
d["q"], d["k"] = torch.randn(1, 128, 2, 64, generator=g0), torch.randn(1, 128, 2, 64, generator=g0)
d["g"] = F.logsigmoid(torch.randn(1, 128, 2, 64, generator=g0)) / 16
record("gla_f32", lambda x: chunk_gla(x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True, head_first=False),
       d, ["q", "k", "v", "g", "h0"])
# retention (per-head constant decay)
d, g0 = base(1, 128, 2, 64, 64, f16, 6)
for n in ("beta", "g"):
    d.pop(n)
d["q"], d["k"] = torch.randn(1, 128, 2, 64, generator=g0).to(f16), torch.randn(1, 128, 2, 64, generator=g0).to(f16)
record("retention", lambda x: chunk_retention(x["q"], x["k"], x["v"], initial_state=x["h0"], output_final_state=True, head_first=False),
       d, ["q", "k", "v", "h0"])
# decode form of the gated delta rule: a few tokens per sequence, forward only (the reference has no backward for it)
d, _ = base(3, 4, 2, 128, 128, f16, 7)
record("decode", lambda x: fused_recurrent_gated_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"],
                                                            output_final_state=True, head_first=False), d, [])

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "triton_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, "%.0f KB" % (os.path.getsize(path) / 1024))
