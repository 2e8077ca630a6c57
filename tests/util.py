"""Shared helpers of the parity tests: the reference's error metric and seeded input builders."""
import torch
import torch.nn.functional as F


def err_ratio(ref, out):
    """RMS(ref - out) / RMS(ref): the metric of the reference's tests (tests/ops/utils.py:1-14)."""
    ref, out = ref.detach().double().cpu(), out.detach().double().cpu()
    err = (ref - out).flatten().square().mean().sqrt().item()
    base = ref.flatten().square().mean().sqrt().item()
    return err / (base + 1e-30)


def assert_close(name, ref, out, ratio):
    r = err_ratio(ref, out)
    assert r < ratio, f"{name}: error ratio {r:.3e} >= {ratio:.1e}"
    return r


def t(golden, key, **kw):
    return torch.from_numpy(golden[key]).clone().to(**kw)


def make_inputs(B, T, H, K, V, dtype, seed=0, gate=None, beta=False, h0=False, normalize_qk=False, gate_div=1.0,
                device="cpu"):
    """Seeded CPU fp32 inputs cast to `dtype` (so the CPU oracle and the GPU see identical bits)."""
    g0 = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=g0)
    k = torch.randn(B, T, H, K, generator=g0)
    v = torch.randn(B, T, H, V, generator=g0)
    if normalize_qk:
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
    d = dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype))
    if gate == "scalar":
        d["g"] = F.logsigmoid(torch.randn(B, T, H, generator=g0)) / gate_div
    elif gate == "vector":
        d["g"] = F.logsigmoid(torch.randn(B, T, H, K, generator=g0)) / gate_div
    if beta:
        d["beta"] = torch.randn(B, T, H, generator=g0).sigmoid().to(dtype)
    d["do"] = torch.randn(B, T, H, V, generator=g0).to(dtype)
    return d, g0


def leafify(d, device, names):
    out = {}
    for n, x in d.items():
        x = x.to(device)
        if n in names:
            x = x.detach().clone().requires_grad_(True)
        out[n] = x
    return out
