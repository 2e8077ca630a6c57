"""Generate tests/golden/f4_vectors.npz from the reference's own kernels for the remaining execution modes of the path:
`fused_chunk_gla`, `fused_chunk_retention`, `fused_chunk_delta_rule`, `parallel_simple_gla` (with the attention
matrix) and the value-channel-gate (`gv`) mode of `chunk_fwd_h` / `chunk_bwd_dh`.

The kernels are Triton; they run unmodified on CPU tensors under Triton's interpreter (TRITON_INTERPRET=1), through
the reference's public functions, forward and backward. As in make_golden_triton.py the autotuner is stubbed (first
configuration) and the device capability is reported as (10, 0). A case whose kernel the interpreter cannot run is
reported and left out. numpy has no bf16, so 16-bit cases are fp16.

    FLA_REFERENCE=<path to flash-linear-attention> python tests/golden/make_golden_f4.py
"""
import os
import sys
import traceback
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

out = {}


def record(name, fn, inputs, grad_names, with_state=True):
    g0 = torch.Generator().manual_seed(len(out) + 5)
    xs = {n: (x.clone().requires_grad_(True) if n in grad_names else x) for n, x in inputs.items()}
    res = fn(xs)
    o, second = res[0], res[1]
    do = torch.randn(o.shape, generator=g0).to(o.dtype)
    outs, gouts = [o], [do]
    if with_state and second is not None:
        dht = torch.randn(second.shape, generator=g0) * 0.1
        outs.append(second)
        gouts.append(dht)
        out[f"{name}.dht"] = dht.numpy()
    if grad_names:
        torch.autograd.backward(outs, gouts)
    for n, x in inputs.items():
        out[f"{name}.{n}"] = x.detach().numpy()
    out[f"{name}.o"], out[f"{name}.do"] = o.detach().numpy(), do.numpy()
    if second is not None:
        out[f"{name}.{'ht' if with_state else 'attn'}"] = second.detach().numpy()
    for n in grad_names:
        if xs[n].grad is not None:
            out[f"{name}.d{n}"] = xs[n].grad.numpy()
    print(name, "ok: o", tuple(o.shape), "mean |o| %.4f" % o.float().abs().mean().item(), flush=True)


def attempt(name, thunk):
    try:
        thunk()
    except Exception:
        print(f"{name}: the interpreter could not run this case:\n{traceback.format_exc()[-1500:]}", flush=True)
        for k_ in [k_ for k_ in out if k_.startswith(name + ".")]:
            del out[k_]


f16 = torch.float16
B, T, H, K, V = 1, 128, 2, 64, 64


def base(seed, dt):
    g0 = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, K, generator=g0).to(dt), torch.randn(B, T, H, K, generator=g0).to(dt)
    v = torch.randn(B, T, H, V, generator=g0).to(dt)
    h0 = torch.randn(B, H, K, V, generator=g0) * 0.1
    return dict(q=q, k=k, v=v, h0=h0), g0


def case_fused_chunk_gla():
    from fla.ops.gla import fused_chunk_gla
    d, g0 = base(31, torch.float32)
    d["g"] = F.logsigmoid(torch.randn(B, T, H, K, generator=g0)) / 16
    record("fused_chunk_gla", lambda x: fused_chunk_gla(x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True,
                                                        head_first=False), d, ["q", "k", "v", "g"])


def case_fused_chunk_retention():
    from fla.ops.retention import fused_chunk_retention
    d, _ = base(32, f16)
    record("fused_chunk_retention", lambda x: fused_chunk_retention(x["q"], x["k"], x["v"], initial_state=x["h0"], output_final_state=True,
                                                                    head_first=False), d, ["q", "k", "v"])


def case_fused_chunk_delta_rule():
    from fla.ops.delta_rule import fused_chunk_delta_rule
    d, g0 = base(33, f16)
    d["q"], d["k"] = F.normalize(d["q"].float(), dim=-1).to(f16), F.normalize(d["k"].float(), dim=-1).to(f16)
    d["beta"] = torch.rand(B, T, H, generator=g0).sigmoid().to(f16)
    record("fused_chunk_delta_rule", lambda x: fused_chunk_delta_rule(x["q"], x["k"], x["v"], x["beta"], initial_state=x["h0"],
                                                                      output_final_state=True, head_first=False), d, [])


def case_parallel_simple_gla():
    from fla.ops.simple_gla import parallel_simple_gla
    d, g0 = base(34, f16)
    d.pop("h0")
    d["g"] = F.logsigmoid(torch.randn(B, T, H, generator=g0))
    record("parallel_simple_gla", lambda x: parallel_simple_gla(x["q"], x["k"], x["v"], x["g"], output_attentions=True, head_first=False),
           d, ["q", "k", "v", "g"], with_state=False)


def case_chunk_h_gv():
    from fla.ops.common.chunk_h import chunk_bwd_dh, chunk_fwd_h
    from fla.ops.utils import chunk_local_cumsum
    d, g0 = base(35, f16)
    gv = chunk_local_cumsum(F.logsigmoid(torch.randn(B, T, H, V, generator=g0)) / 4, 64, head_first=False)
    h, ht = chunk_fwd_h(d["k"], d["v"], None, None, gv, d["h0"], True, head_first=False, chunk_size=64)
    do = torch.randn(B, T, H, V, generator=g0).to(f16)
    dht = torch.randn(B, H, K, V, generator=g0) * 0.1
    dh, dh0 = chunk_bwd_dh(d["q"], d["k"], d["v"], None, None, gv, do, d["h0"], dht, K ** -0.5, head_first=False, chunk_size=64)
    for n, x in dict(d, gv=gv, h=h, ht=ht, do=do, dht=dht, dh=dh, dh0=dh0).items():
        out[f"chunk_h_gv.{n}"] = x.detach().numpy()
    print("chunk_h_gv ok", tuple(h.shape), flush=True)


for name, fn in [("fused_chunk_gla", case_fused_chunk_gla), ("fused_chunk_retention", case_fused_chunk_retention),
                 ("fused_chunk_delta_rule", case_fused_chunk_delta_rule), ("parallel_simple_gla", case_parallel_simple_gla),
                 ("chunk_h_gv", case_chunk_h_gv)]:
    attempt(name, fn)

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "f4_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, "%.0f KB" % (os.path.getsize(path) / 1024), sorted({k_.split(".")[0] for k_ in out}))
