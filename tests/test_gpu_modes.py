"""GPU parity of the remaining execution modes of the path and of the gate / beta prologue:
`fused_chunk_gla`, `fused_chunk_retention`, `fused_chunk_delta_rule`, `parallel_simple_gla` (with its attention matrix),
the value-channel-gate (gv) mode of `chunk_fwd_h` / `chunk_bwd_dh`, and `gdn_gate_beta`.
Checked against outputs of the reference's own kernels (tests/golden/f4_vectors.npz, made by
tests/golden/make_golden_f4.py under Triton's CPU interpreter) and against the CPU oracle on seeded inputs.
Bars: relative L2 <= 5e-3 for 16-bit inputs, <= 1e-5 for fp32."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from util import assert_close, err_ratio

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _f4():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "f4_vectors.npz"))


def ops():
    import fla_b200.ops as o
    return o


def _case(z, name, names, grads):
    x = {n: torch.from_numpy(z[f"{name}.{n}"]).to(DEV) for n in names}
    for n in grads:
        x[n].requires_grad_(True)
    ref = {k_[len(name) + 1:]: torch.from_numpy(z[k_]) for k_ in z.files if k_.startswith(name + ".")}
    return x, ref


def test_fused_chunk_modes_against_reference_kernel_outputs():
    z = _f4()
    o_ = ops()
    # GLA, fp32. The reference's fused backward ignores the gradient of the final state (fla/ops/gla/fused_chunk.py:497),
    # so the comparison back-propagates do only.
    x, r = _case(z, "fused_chunk_gla", ["q", "k", "v", "g", "h0"], ["q", "k", "v", "g"])
    o, ht = o_.fused_chunk_gla(x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True, head_first=False)
    res = {"o": assert_close("gla o", r["o"], o, 1e-5), "ht": assert_close("gla ht", r["ht"], ht, 1e-5)}
    torch.autograd.backward([o], [r["do"].to(DEV)])
    for n in ("q", "k", "v", "g"):
        res["d" + n] = assert_close("gla d" + n, r["d" + n], x[n].grad, 2e-5)
    print("fused_chunk_gla", {n: f"{e:.2e}" for n, e in res.items()})
    # retention, fp16
    x, r = _case(z, "fused_chunk_retention", ["q", "k", "v", "h0"], ["q", "k", "v"])
    o, ht = o_.fused_chunk_retention(x["q"], x["k"], x["v"], initial_state=x["h0"], output_final_state=True, head_first=False)
    res = {"o": assert_close("retention o", r["o"].float(), o, 5e-3), "ht": assert_close("retention ht", r["ht"], ht, 5e-3)}
    torch.autograd.backward([o], [r["do"].to(DEV)])
    for n in ("q", "k", "v"):
        res["d" + n] = assert_close("retention d" + n, r["d" + n].float(), x[n].grad, 5e-3)
    print("fused_chunk_retention", {n: f"{e:.2e}" for n, e in res.items()})
    assert x["h0"].grad is None  # the initial state is a constant in the fused modes, as in the reference


def test_parallel_simple_gla_against_reference_kernel_outputs():
    z = _f4()
    x, r = _case(z, "parallel_simple_gla", ["q", "k", "v", "g"], ["q", "k", "v", "g"])
    o, attn = ops().parallel_simple_gla(x["q"], x["k"], x["v"], x["g"], output_attentions=True, head_first=False)
    res = {"o": assert_close("o", r["o"].float(), o, 5e-3), "attn": assert_close("attn", r["attn"].float(), attn, 5e-3)}
    assert attn.shape == r["attn"].shape and attn.dtype == x["q"].dtype
    assert torch.count_nonzero(attn.float().triu(1)) == 0
    torch.autograd.backward([o], [r["do"].to(DEV)])
    for n in ("q", "k", "v", "g"):
        res["d" + n] = assert_close("d" + n, r["d" + n].float(), x[n].grad, 5e-3)
    print("parallel_simple_gla", {n: f"{e:.2e}" for n, e in res.items()})
    o2, none = ops().parallel_simple_gla(x["q"], x["k"], x["v"], x["g"], head_first=False)
    assert none is None and torch.equal(o2, o)


@pytest.mark.parametrize("head_first,use_g,T", [(False, True, 200), (True, True, 130), (False, False, 96)])
def test_parallel_simple_gla_against_oracle(head_first, use_g, T):
    B, H, K, V = 2, 3, 64, 128
    g0 = torch.Generator().manual_seed(T)
    q, k = torch.randn(B, T, H, K, generator=g0).bfloat16(), torch.randn(B, T, H, K, generator=g0).bfloat16()
    v, do = torch.randn(B, T, H, V, generator=g0).bfloat16(), torch.randn(B, T, H, V, generator=g0).bfloat16()
    g = F.logsigmoid(torch.randn(B, T, H, generator=g0)) if use_g else None
    tr = (lambda x: x.transpose(1, 2).contiguous()) if head_first else (lambda x: x)
    xs = [tr(x).to(DEV).requires_grad_(True) for x in (q, k, v)] + ([tr(g).to(DEV).requires_grad_(True)] if use_g else [])
    o, attn = ops().parallel_simple_gla(xs[0], xs[1], xs[2], xs[3] if use_g else None, output_attentions=True, head_first=head_first)
    rs = [tr(x).float().requires_grad_(True) for x in (q, k, v)] + ([tr(g).requires_grad_(True)] if use_g else [])
    if use_g:
        o_ref, _ = oracle.simple_gla(rs[0], rs[1], rs[2], rs[3], head_first=head_first)
    else:
        o_ref, _ = oracle.gla(rs[0], rs[1], rs[2], head_first=head_first)
    a_ref = oracle.simple_gla_attention(rs[0].detach(), rs[1].detach(), rs[3].detach() if use_g else None, head_first=head_first)
    res = {"o": assert_close("o", o_ref, o, 5e-3), "attn": assert_close("attn", a_ref, attn, 5e-3)}
    gg = torch.autograd.grad((o.float() * tr(do).to(DEV).float()).sum(), xs)
    gr = torch.autograd.grad((o_ref * tr(do).float()).sum(), rs)
    for n, a, b in zip(("dq", "dk", "dv", "dg"), gr, gg):
        res[n] = assert_close(n, a, b, 5e-3)
    print({n: f"{e:.2e}" for n, e in res.items()})


def test_fused_chunk_delta_rule_against_oracle():
    """The reference's own fused_chunk_delta_rule cannot produce vectors: its forward calls fwd_prepare_wy_repr without
    the `indices` argument that function requires (fla/ops/delta_rule/fused_chunk.py:339 against wy_fast.py:436) and
    raises TypeError. The mode is therefore pinned on the oracle alone, forward and all gradients."""
    B, T, H, K, V = 2, 200, 2, 128, 128
    g0 = torch.Generator().manual_seed(5)
    q = F.normalize(torch.randn(B, T, H, K, generator=g0), dim=-1).bfloat16()
    k = F.normalize(torch.randn(B, T, H, K, generator=g0), dim=-1).bfloat16()
    v, do = torch.randn(B, T, H, V, generator=g0).bfloat16(), torch.randn(B, T, H, V, generator=g0).bfloat16()
    beta = torch.rand(B, T, H, generator=g0).sigmoid().bfloat16()
    h0, dht = torch.randn(B, H, K, V, generator=g0) * 0.1, torch.randn(B, H, K, V, generator=g0)
    xs = [x.to(DEV).requires_grad_(True) for x in (q, k, v, beta, h0)]
    o, ht = ops().fused_chunk_delta_rule(*xs[:4], initial_state=xs[4], output_final_state=True, head_first=False)
    rs = [x.float().requires_grad_(True) for x in (q, k, v, beta, h0)]
    o_ref, ht_ref = oracle.delta_rule(*rs[:4], initial_state=rs[4], output_final_state=True, head_first=False)
    res = {"o": assert_close("o", o_ref, o, 5e-3), "ht": assert_close("ht", ht_ref, ht, 5e-3)}
    gg = torch.autograd.grad((o.float() * do.to(DEV).float()).sum() + (ht * dht.to(DEV)).sum(), xs)
    gr = torch.autograd.grad((o_ref * do.float()).sum() + (ht_ref * dht).sum(), rs)
    for n, a, b in zip(("dq", "dk", "dv", "dbeta", "dh0"), gr, gg):
        res[n] = assert_close(n, a, b, 2e-2 if n == "dbeta" else 8e-3)
    print({n: f"{e:.2e}" for n, e in res.items()})


def test_value_gate_state_scan_against_reference_kernel_outputs_and_oracle():
    from fla_b200.ops import common as C
    from fla_b200.utils import Geometry
    z = _f4()
    x, r = _case(z, "chunk_h_gv", ["q", "k", "v", "gv", "h0", "do", "dht"], [])
    geo = Geometry(x["k"], x["v"], None, False)
    h, ht = C.chunk_fwd_h(geo, x["k"], x["v"], gv=x["gv"], h0=x["h0"], output_final_state=True)
    dh, dh0 = C.chunk_bwd_dh(geo, x["q"], x["do"], x["k"].shape[-1] ** -0.5, gv=x["gv"], dht=x["dht"], want_dh0=True)
    res = {"h": assert_close("h", r["h"].float().flatten(0, 1), h, 5e-3), "ht": assert_close("ht", r["ht"], ht, 5e-3),
           "dh": assert_close("dh", r["dh"].float().flatten(0, 1), dh, 5e-3), "dh0": assert_close("dh0", r["dh0"], dh0, 5e-3)}
    print("gv scan vs reference kernels", {n: f"{e:.2e}" for n, e in res.items()})
    # seeded case with both channel gates, ragged length, odd head dims, fp32 and bf16
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-3)):
        B, T, H, K, V = 2, 150, 2, 96, 80
        g0 = torch.Generator().manual_seed(9)
        k, v, q, do = (torch.randn(B, T, H, d_, generator=g0).to(dt) for d_ in (K, V, K, V))
        gk = oracle.cumsum_local(F.logsigmoid(torch.randn(B, T, H, K, generator=g0)) / 4, 64, head_first=False)
        gv = oracle.cumsum_local(F.logsigmoid(torch.randn(B, T, H, V, generator=g0)) / 4, 64, head_first=False)
        h0, dht = torch.randn(B, H, K, V, generator=g0), torch.randn(B, H, K, V, generator=g0)
        geo = Geometry(k.to(DEV), v.to(DEV), None, False)
        for use_gk in (False, True):
            gkd = gk.to(DEV) if use_gk else None
            h, ht = C.chunk_fwd_h(geo, k.to(DEV), v.to(DEV), gk=gkd, gv=gv.to(DEV), h0=h0.to(DEV), output_final_state=True)
            dh, dh0 = C.chunk_bwd_dh(geo, q.to(DEV), do.to(DEV), 0.1, gk=gkd, gv=gv.to(DEV), dht=dht.to(DEV), want_dh0=True)
            hr, htr = oracle.chunk_states(k, v, gk_cumsum=gk if use_gk else None, gv_cumsum=gv, initial_state=h0)
            dhr, dh0r = oracle.chunk_state_gradients(q, do, 0.1, gk_cumsum=gk if use_gk else None, gv_cumsum=gv, dht=dht)
            res = {"h": assert_close("h", hr.flatten(0, 1), h, tol), "ht": assert_close("ht", htr, ht, tol),
                   "dh": assert_close("dh", dhr.flatten(0, 1), dh, tol), "dh0": assert_close("dh0", dh0r, dh0, tol)}
            print(dt, "gk+gv" if use_gk else "gv", {n: f"{e:.2e}" for n, e in res.items()})


@pytest.mark.parametrize("dtype,head_first,varlen", [(torch.bfloat16, False, False), (torch.float32, True, False), (torch.bfloat16, False, True)])
def test_gate_beta_prologue_matches_reference_formula(dtype, head_first, varlen):
    """g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b) (fla/layers/gated_deltanet.py:236-237) written with the
    reference's own torch expressions in fp64 autograd; plus the chunk-local cumsum produced by the same pass."""
    from fla_b200.modules import gdn_gate_beta
    from fla_b200.modules.gate_prologue import attached_cumsum
    B, T, H = (1, 333, 5) if varlen else (2, 150, 6)
    g0 = torch.Generator().manual_seed(T)
    shape = (B, H, T) if head_first else (B, T, H)
    a, b = torch.randn(*shape, generator=g0).to(dtype), torch.randn(*shape, generator=g0).to(dtype)
    A_log, dt_bias = torch.randn(H, generator=g0).abs().log(), torch.randn(H, generator=g0)
    dg, dbeta = torch.randn(*shape, generator=g0), torch.randn(*shape, generator=g0).to(dtype)
    off = torch.tensor([0, 70, 71, 200, 333]) if varlen else None
    off_dev = None if off is None else off.to(DEV)
    xs = [x.to(DEV).requires_grad_(True) for x in (a, b, A_log, dt_bias)]
    g, beta = gdn_gate_beta(*xs, offsets=off_dev, head_first=head_first)
    rs = [x.double().requires_grad_(True) for x in (a, b, A_log, dt_bias)]
    hdim = (None, slice(None), None) if head_first else (None, None, slice(None))
    g_ref = -rs[2].exp()[hdim] * F.softplus(rs[0] + rs[3][hdim])
    beta_ref = rs[1].sigmoid()
    tol = 1e-5 if dtype == torch.float32 else 5e-3
    assert g.dtype == torch.float32 and beta.dtype == dtype
    res = {"g": assert_close("g", g_ref, g, 1e-5), "beta": assert_close("beta", beta_ref, beta, tol)}
    gg = torch.autograd.grad((g * dg.to(DEV)).sum() + (beta.float() * dbeta.to(DEV).float()).sum(), xs)
    gr = torch.autograd.grad((g_ref * dg.double()).sum() + (beta_ref * dbeta.double()).sum(), rs)
    for n, x_, y_ in zip(("da", "db", "dA_log", "ddt_bias"), gr, gg):
        res[n] = assert_close(n, x_, y_, tol if n in ("da", "db") else 1e-4)
    cum = attached_cumsum(g, off_dev, head_first)
    cum_ref = oracle.cumsum_local(g_ref.float(), 64, offsets=off, head_first=head_first)
    res["cumsum"] = assert_close("cumsum", cum_ref, cum, 1e-5)
    print({n: f"{e:.2e}" for n, e in res.items()})


def test_gate_prologue_cumsum_is_used_by_the_chunk_op():
    """g made by gdn_gate_beta carries its chunk-local cumsum: chunk_gated_delta_rule takes it (one launch fewer) and
    returns the same bits as with a plain copy of g; gradients flow back to a, b, A_log, dt_bias."""
    from fla_b200 import _lib
    from fla_b200.modules import gdn_gate_beta
    B, T, H, K, V = 2, 256, 4, 128, 128
    g0 = torch.Generator().manual_seed(2)
    q = F.normalize(torch.randn(B, T, H, K, generator=g0), dim=-1).bfloat16().to(DEV)
    k = F.normalize(torch.randn(B, T, H, K, generator=g0), dim=-1).bfloat16().to(DEV)
    v = torch.randn(B, T, H, V, generator=g0).bfloat16().to(DEV)
    a = torch.randn(B, T, H, generator=g0).bfloat16().to(DEV).requires_grad_(True)
    b = torch.randn(B, T, H, generator=g0).bfloat16().to(DEV).requires_grad_(True)
    A_log = torch.zeros(H, device=DEV, requires_grad=True)
    dt_bias = torch.zeros(H, device=DEV, requires_grad=True)
    g, beta = gdn_gate_beta(a, b, A_log, dt_bias)
    n0 = _lib.LAUNCHES
    o1, _ = ops().chunk_gated_delta_rule(q, k, v, g, beta, head_first=False)
    n1 = _lib.LAUNCHES
    o2, _ = ops().chunk_gated_delta_rule(q, k, v, g.detach().clone().requires_grad_(True), beta, head_first=False)
    n2 = _lib.LAUNCHES
    assert torch.equal(o1, o2)
    assert (n1 - n0) == (n2 - n1) - 1, "the op should have skipped its own cumsum launch"
    o1.float().square().sum().backward()
    for x in (a, b, A_log, dt_bias):
        assert x.grad is not None and torch.isfinite(x.grad).all() and x.grad.abs().sum() > 0
    assert err_ratio(o1, o2) == 0
