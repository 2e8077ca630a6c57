"""GPU parity tests: the CUDA path (through the public fla.ops-style API, i.e. through the C ABI)
against the CPU oracle on identical seeded inputs, the committed golden vectors of the reference,
and size-independent properties.  Error metric and shape sweeps follow the reference's tests
(tests/ops/test_{gla,simple_gla,retention,delta,gated_delta,cumsum}.py)."""
import os

import pytest
import torch
import torch.nn.functional as F

import oracle
from util import assert_close, err_ratio, t

pytestmark = pytest.mark.gpu

DEV = "cuda"
# relative-L2 bars: bf16/fp16 5e-3, fp32 1e-5
TOL = {torch.bfloat16: 5e-3, torch.float16: 5e-3, torch.float32: 1e-5}


def ops():
    import fla_b200.ops as o
    return o


def rand_offsets(T, N, seed=42):
    g0 = torch.Generator().manual_seed(seed)
    cuts = torch.randperm(T - 1, generator=g0)[:N - 1] + 1
    return torch.cat([torch.tensor([0]), cuts.sort()[0], torch.tensor([T])]).long()


def build(B, T, H, K, V, dtype, seed, gate=None, beta=False, h0=False, norm=False, gate_div=1.0, N=None):
    g0 = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, K, generator=g0), torch.randn(B, T, H, K, generator=g0)
    v = torch.randn(B, T, H, V, generator=g0)
    if norm:
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
    d = dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype))
    if gate == "scalar":
        d["g"] = F.logsigmoid(torch.randn(B, T, H, generator=g0)) / gate_div
    if gate == "vector":
        d["g"] = (F.logsigmoid(torch.randn(B, T, H, K, generator=g0)) / gate_div).to(dtype)
    if beta:
        d["beta"] = torch.rand(B, T, H, generator=g0).sigmoid().to(dtype)
    if h0:
        d["h0"] = torch.randn(N or B, H, K, V, generator=g0) * 0.1
    d["do"] = torch.randn(B, T, H, V, generator=g0).to(dtype)
    d["dht"] = torch.randn(N or B, H, K, V, generator=g0)
    return d


def run_both(fn_gpu, fn_ref, d, names, head_first=False, tol=None, tol_over=None, check_grads=True, **kw):
    """Run `fn_gpu` on CUDA and `fn_ref` (oracle) on CPU fp32 with the same bits; compare o, ht, grads."""
    dtype = d["q"].dtype
    tol = tol or TOL[dtype]
    tol_over = tol_over or {}

    def prep(dev, cast):
        out = {}
        for n in names:
            x = d[n]
            if head_first and x.dim() >= 3 and n not in ("h0",):
                x = x.transpose(1, 2).contiguous()
            x = x.to(dev)
            if cast and x.is_floating_point():
                x = x.float()
            out[n] = x.detach().clone().requires_grad_(check_grads)
        return out

    gi, ri = prep(DEV, False), prep("cpu", True)
    do, dht = d["do"], d["dht"]
    if head_first:
        do = do.transpose(1, 2).contiguous()
    o, ht = fn_gpu(gi, head_first=head_first, **kw)
    o_ref, ht_ref = fn_ref(ri, head_first=head_first, **kw)
    res = {"o": err_ratio(o_ref, o)}
    if ht_ref is not None:
        res["ht"] = err_ratio(ht_ref, ht)
    if check_grads:
        loss = (o.float() * do.to(DEV).float()).sum()
        loss_ref = (o_ref * do.float()).sum()
        if ht_ref is not None:
            loss = loss + (ht * dht.to(DEV)).sum()
            loss_ref = loss_ref + (ht_ref * dht).sum()
        gg = torch.autograd.grad(loss, [gi[n] for n in names])
        gr = torch.autograd.grad(loss_ref, [ri[n] for n in names])
        for n, a, b in zip(names, gr, gg):
            res["d" + n] = err_ratio(a, b)
    # every ratio is printed (pytest -s) before any is judged, so one run shows the whole picture
    print({k_: f"{v_:.2e}" for k_, v_ in res.items()})
    bad = {k_: (v_, tol_over.get(k_, tol)) for k_, v_ in res.items() if not v_ < tol_over.get(k_, tol)}
    assert not bad, f"relative L2 error over the bar (value, bar): {bad}"
    return res


# ------------------------------------------------------------------------------------------------
# cumsum
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_first", [False, True])
@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("S", [0, 24])
def test_cumsum_local_and_global(dtype, head_first, reverse, S):
    from fla_b200.ops.common import chunk_global_cumsum, chunk_local_cumsum
    g0 = torch.Generator().manual_seed(1)
    shape = (2, 150, 3) + ((S,) if S else ())
    x = torch.randn(*shape, generator=g0).to(dtype)
    xs = x.transpose(1, 2).contiguous() if head_first else x
    y = chunk_local_cumsum(xs.to(DEV), 64, reverse=reverse, head_first=head_first).cpu()
    torch.testing.assert_close(y, oracle.cumsum_local(xs, 64, reverse=reverse, head_first=head_first), rtol=1e-5, atol=1e-5)
    y = chunk_global_cumsum(xs.to(DEV), dtype=torch.float32, reverse=reverse, head_first=head_first).cpu()
    torch.testing.assert_close(y, oracle.cumsum_global(xs, reverse=reverse, head_first=head_first), rtol=1e-5, atol=2e-5)


def test_cumsum_varlen_and_golden(golden):
    from fla_b200.ops.common import chunk_global_cumsum, chunk_local_cumsum
    x = torch.randn(1, 500, 4, generator=torch.Generator().manual_seed(3))
    for dt in (torch.int64, torch.int32):
        off = rand_offsets(500, 5).to(dt)
        for rev in (False, True):
            y = chunk_local_cumsum(x.to(DEV), 64, reverse=rev, offsets=off.to(DEV), head_first=False).cpu()
            torch.testing.assert_close(y, oracle.cumsum_local(x, 64, reverse=rev, offsets=off, head_first=False), rtol=1e-5, atol=1e-5)
            y = chunk_global_cumsum(x.to(DEV), reverse=rev, offsets=off.to(DEV), head_first=False).cpu()
            torch.testing.assert_close(y, oracle.cumsum_global(x, reverse=rev, offsets=off, head_first=False), rtol=1e-5, atol=2e-5)
    for name in ("s3", "s4"):
        xg = t(golden, f"cumsum.{name}.x")
        y = chunk_local_cumsum(xg.to(DEV), 64, head_first=False).cpu()
        torch.testing.assert_close(y, t(golden, f"cumsum.{name}.local"), rtol=1e-5, atol=1e-5)
        y = chunk_global_cumsum(xg.to(DEV), reverse=True, head_first=False).cpu()
        torch.testing.assert_close(y, t(golden, f"cumsum.{name}.glob_rev"), rtol=1e-5, atol=2e-5)


# ------------------------------------------------------------------------------------------------
# simple GLA / retention
# ------------------------------------------------------------------------------------------------
def _sgla_gpu(i, **kw):
    return ops().chunk_simple_gla(i["q"], i["k"], i["v"], i["g"], initial_state=i.get("h0"), output_final_state=True, **kw)


def _sgla_ref(i, scale=None, offsets=None, head_first=False, **kw):
    return oracle.simple_gla(i["q"], i["k"], i["v"], i["g"], scale=scale, initial_state=i.get("h0"),
                             output_final_state=True, offsets=offsets, head_first=head_first)


@pytest.mark.parametrize("B,T,H,K,V,dtype,head_first", [
    (2, 130, 3, 64, 64, torch.bfloat16, False),
    (2, 256, 2, 128, 128, torch.bfloat16, False),
    (2, 150, 2, 128, 128, torch.float16, True),    # tcgen05 kernels: head-first, fp16, ragged last chunk
    (1, 300, 2, 100, 60, torch.bfloat16, False),
    (2, 63, 2, 32, 64, torch.float16, True),
    (2, 200, 2, 64, 128, torch.float32, False),
    (1, 15, 2, 64, 64, torch.float32, True),
])
def test_chunk_simple_gla(B, T, H, K, V, dtype, head_first):
    d = build(B, T, H, K, V, dtype, seed=T, gate="scalar", h0=True)
    run_both(_sgla_gpu, _sgla_ref, d, ["q", "k", "v", "g", "h0"], head_first=head_first)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_chunk_simple_gla_varlen(dtype):
    T, N = 500, 4
    d = build(1, T, 3, 64, 64, dtype, seed=5, gate="scalar", h0=True, N=N)
    off = rand_offsets(T, N)
    run_both(lambda i, **kw: _sgla_gpu(i, offsets=off.to(DEV), head_first=False),
             lambda i, **kw: _sgla_ref(i, offsets=off), d, ["q", "k", "v", "g", "h0"])


def test_chunk_retention_matches_oracle_and_golden(golden):
    o_ = ops()
    d = build(2, 200, 4, 64, 64, torch.bfloat16, seed=11)
    g = oracle.retention_log_decay(4)[None, None, :].expand(2, 200, 4).contiguous()

    def gpu(i, **kw):
        return o_.chunk_retention(i["q"], i["k"], i["v"], output_final_state=True, head_first=False)

    def ref(i, **kw):
        return oracle.simple_gla(i["q"], i["k"], i["v"], g, output_final_state=True, head_first=False)
    run_both(gpu, ref, d, ["q", "k", "v"])
    # the reference's O(T^2) retention on its own seeded inputs (fp32, head-first)
    q, k, v = (t(golden, f"retention.{n}").to(DEV) for n in ("q", "k", "v"))
    o, _ = o_.chunk_retention(q, k, v, head_first=True)
    assert_close("retention golden", t(golden, "retention.o"), o, 1e-5)
    o2, _ = o_.fused_recurrent_retention(q, k, v, head_first=True)
    assert_close("recurrent retention golden", t(golden, "retention.o"), o2, 1e-5)


def test_chunk_simple_gla_golden(golden):
    names = ("q", "k", "v", "g", "h0")
    q, k, v, g, h0 = (t(golden, f"simple_gla.{n}").to(DEV).requires_grad_(True) for n in names)
    o, ht = ops().chunk_simple_gla(q, k, v, g, initial_state=h0, output_final_state=True, head_first=True)
    assert_close("o", t(golden, "simple_gla.o"), o, 1e-5)
    assert_close("ht", t(golden, "simple_gla.ht"), ht, 1e-5)
    loss = (o * t(golden, "simple_gla.do").to(DEV)).sum() + (ht * t(golden, "simple_gla.dht").to(DEV)).sum()
    for n, gx in zip(("dq", "dk", "dv", "dg", "dh0"), torch.autograd.grad(loss, (q, k, v, g, h0))):
        assert_close(n, t(golden, f"simple_gla.{n}"), gx, 1e-5)


# ------------------------------------------------------------------------------------------------
# GLA
# ------------------------------------------------------------------------------------------------
def _gla_gpu(i, **kw):
    return ops().chunk_gla(i["q"], i["k"], i["v"], i["g"], initial_state=i.get("h0"), output_final_state=True, **kw)


def _gla_ref(i, scale=None, offsets=None, head_first=False, **kw):
    return oracle.gla(i["q"], i["k"], i["v"], gk=i["g"], scale=scale, initial_state=i.get("h0"), output_final_state=True,
                      offsets=offsets, head_first=head_first)


@pytest.mark.parametrize("B,T,H,K,V,dtype,head_first,gate_div", [
    (2, 512, 4, 64, 64, torch.float32, False, 16.0),   # the fp32 configuration of the build spec
    (2, 130, 2, 64, 64, torch.float32, True, 1.0),
    (2, 200, 2, 128, 128, torch.bfloat16, False, 1.0),
    (1, 300, 2, 100, 100, torch.bfloat16, False, 20.0),
    (1, 70, 2, 32, 64, torch.float16, False, 1.0),
])
def test_chunk_gla(B, T, H, K, V, dtype, head_first, gate_div):
    d = build(B, T, H, K, V, dtype, seed=T, gate="vector", h0=True, gate_div=gate_div)
    run_both(_gla_gpu, _gla_ref, d, ["q", "k", "v", "g", "h0"], head_first=head_first)


def test_chunk_gla_varlen():
    T, N = 400, 4
    d = build(1, T, 2, 64, 64, torch.float32, seed=8, gate="vector", h0=True, N=N)
    off = rand_offsets(T, N)
    run_both(lambda i, **kw: _gla_gpu(i, offsets=off.to(DEV), head_first=False),
             lambda i, **kw: _gla_ref(i, offsets=off), d, ["q", "k", "v", "g", "h0"])


def test_chunk_gla_golden(golden):
    names = ("q", "k", "v", "gk", "h0")
    q, k, v, gk, h0 = (t(golden, f"gla.{n}").to(DEV).requires_grad_(True) for n in names)
    o, ht = ops().chunk_gla(q, k, v, gk, initial_state=h0, output_final_state=True, head_first=True)
    assert_close("o", t(golden, "gla.o"), o, 1e-5)
    assert_close("ht", t(golden, "gla.ht"), ht, 1e-5)
    loss = (o * t(golden, "gla.do").to(DEV)).sum() + (ht * t(golden, "gla.dht").to(DEV)).sum()
    for n, gx in zip(("dq", "dk", "dv", "dgk", "dh0"), torch.autograd.grad(loss, (q, k, v, gk, h0))):
        assert_close(n, t(golden, f"gla.{n}"), gx, 1e-5)


# ------------------------------------------------------------------------------------------------
# delta rule / gated delta rule
# ------------------------------------------------------------------------------------------------
def _delta_gpu(i, **kw):
    return ops().chunk_delta_rule(i["q"], i["k"], i["v"], i["beta"], initial_state=i.get("h0"), output_final_state=True, **kw)


def _delta_ref(i, scale=None, offsets=None, head_first=False, **kw):
    return oracle.delta_rule(i["q"], i["k"], i["v"], i["beta"], scale=scale, initial_state=i.get("h0"),
                             output_final_state=True, offsets=offsets, head_first=head_first)


def _gdelta_gpu(i, **kw):
    return ops().chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i.get("h0"),
                                        output_final_state=True, **kw)


def _gdelta_ref(i, scale=None, offsets=None, head_first=False, **kw):
    return oracle.gated_delta_rule(i["q"], i["k"], i["v"], i["beta"], g=i["g"], scale=scale, initial_state=i.get("h0"),
                                   output_final_state=True, offsets=offsets, head_first=head_first)


# Bars of the two delta-rule families against the fp32 oracle: 5e-3 for o, ht, dq, dv, dh0 like every other op; the
# three gradients that pass through the longest chains of 16-bit intermediates (A, w, u, v_new, the inverse) get
# dk 6e-3, dbeta and dg 1e-2. Measured over all cases of this file on the B200: dq <= 4.4e-3, dk <= 5.2e-3,
# dv <= 3.7e-3, dh0 <= 3.7e-3, dg <= 5.8e-3, dbeta <= 6.3e-3. The reference's own bars for these quantities
# (tests/ops/test_delta.py:74-93, tests/ops/test_gated_delta.py:282-294) are 7e-3..8e-3 and 2e-2; its Triton kernels
# sit at the same distance from the oracle (bench.py prints ours-vs-Triton on the same bf16 inputs: <= 4e-3).
DELTA_TOL = {"dk": 6e-3, "dbeta": 1e-2, "dg": 1e-2}


@pytest.mark.parametrize("B,T,H,K,V,dtype,head_first", [
    (2, 130, 2, 64, 64, torch.bfloat16, False),
    (2, 256, 2, 128, 128, torch.bfloat16, False),
    (2, 150, 2, 128, 128, torch.float16, True),    # tcgen05 kernels: head-first, fp16, ragged last chunk
    (1, 333, 3, 128, 128, torch.bfloat16, False),
    (1, 300, 2, 100, 60, torch.bfloat16, False),
    (2, 63, 2, 32, 64, torch.float16, True),
    (1, 7, 2, 64, 64, torch.bfloat16, False),
])
def test_chunk_delta_rule(B, T, H, K, V, dtype, head_first):
    d = build(B, T, H, K, V, dtype, seed=T, beta=True, h0=True, norm=True)
    run_both(_delta_gpu, _delta_ref, d, ["q", "k", "v", "beta", "h0"], head_first=head_first, tol_over=DELTA_TOL)


@pytest.mark.parametrize("B,T,H,K,V,dtype,head_first,gate_div", [
    (2, 130, 2, 64, 64, torch.bfloat16, False, 1.0),
    (2, 256, 2, 128, 128, torch.bfloat16, False, 1.0),
    (2, 150, 2, 128, 128, torch.float16, True, 1.0),    # tcgen05 kernels: head-first, fp16, ragged last chunk
    (1, 333, 3, 128, 128, torch.bfloat16, False, 10.0),
    (1, 40, 2, 128, 128, torch.bfloat16, False, 1.0),   # a single ragged chunk
    (1, 300, 2, 100, 60, torch.bfloat16, False, 1.0),
    (2, 63, 2, 32, 64, torch.float16, True, 1.0),
    (2, 200, 2, 64, 64, torch.bfloat16, False, 10.0),
])
def test_chunk_gated_delta_rule(B, T, H, K, V, dtype, head_first, gate_div):
    d = build(B, T, H, K, V, dtype, seed=T, gate="scalar", beta=True, h0=True, norm=True, gate_div=gate_div)
    run_both(_gdelta_gpu, _gdelta_ref, d, ["q", "k", "v", "g", "beta", "h0"], head_first=head_first, tol_over=DELTA_TOL)


@pytest.mark.parametrize("odt", [torch.int64, torch.int32])
def test_chunk_gated_delta_rule_varlen(odt):
    T, N = 700, 5
    d = build(1, T, 2, 64, 64, torch.bfloat16, seed=9, gate="scalar", beta=True, h0=True, norm=True, N=N)
    off = rand_offsets(T, N).to(odt)
    run_both(lambda i, **kw: _gdelta_gpu(i, cu_seqlens=off.to(DEV), head_first=False),
             lambda i, **kw: _gdelta_ref(i, offsets=off), d, ["q", "k", "v", "g", "beta", "h0"], tol_over=DELTA_TOL)


def test_chunk_delta_rule_varlen():
    T, N = 600, 4
    d = build(1, T, 2, 64, 64, torch.bfloat16, seed=10, beta=True, h0=True, norm=True, N=N)
    off = rand_offsets(T, N)
    run_both(lambda i, **kw: _delta_gpu(i, offsets=off.to(DEV), head_first=False),
             lambda i, **kw: _delta_ref(i, offsets=off), d, ["q", "k", "v", "beta", "h0"], tol_over=DELTA_TOL)


def test_delta_families_on_reference_golden_inputs(golden):
    """Reference fp32 vectors, cast to bf16 for the chunk kernels (which reject fp32 like the reference)."""
    o_ = ops()
    q, k, v, beta, g, h0 = (t(golden, f"gated_delta.{n}") for n in ("q", "k", "v", "beta", "g", "h0"))
    scale = float(golden["gated_delta.scale"])
    bf = lambda x: x.to(DEV).bfloat16()  # noqa: E731
    o, ht = o_.chunk_gated_delta_rule(bf(q), bf(k), bf(v), g.to(DEV), bf(beta), scale=scale, initial_state=h0.to(DEV),
                                      output_final_state=True, head_first=False)
    assert_close("gated o", t(golden, "gated_delta.o"), o, 8e-3)
    assert_close("gated ht", t(golden, "gated_delta.ht"), ht, 8e-3)
    o, ht = o_.fused_recurrent_gated_delta_rule(q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV), scale=scale,
                                                initial_state=h0.to(DEV), output_final_state=True, head_first=False)
    assert_close("recurrent gated o", t(golden, "gated_delta.o"), o, 1e-5)
    assert_close("recurrent gated ht", t(golden, "gated_delta.ht"), ht, 1e-5)
    q, k, v, beta, h0 = (t(golden, f"delta.{n}") for n in ("q", "k", "v", "beta", "h0"))
    o, ht = o_.chunk_delta_rule(bf(q), bf(k), bf(v), bf(beta), initial_state=h0.to(DEV), output_final_state=True, head_first=True)
    assert_close("delta o", t(golden, "delta.o"), o, 8e-3)
    assert_close("delta ht", t(golden, "delta.ht"), ht, 8e-3)


# ------------------------------------------------------------------------------------------------
# token-recurrent kernels
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("K,V", [(64, 64), (100, 60), (200, 128)])
@pytest.mark.parametrize("reverse", [False, True])
def test_fused_recurrent_gla(dtype, K, V, reverse):
    d = build(2, 70, 2, K, V, dtype, seed=K + V, gate="vector", h0=True)
    d["gv"] = F.logsigmoid(torch.randn(2, 70, 2, V, generator=torch.Generator().manual_seed(1))).to(dtype)
    d["dht"] = d["dht"] * 0  # the reference forbids a final-state gradient together with gate gradients
    tol = 1e-5 if dtype == torch.float32 else 5e-3

    def gpu(i, **kw):
        return ops().fused_recurrent_gla(i["q"], i["k"], i["v"], gk=i["g"], gv=i["gv"], initial_state=i["h0"],
                                         output_final_state=True, reverse=reverse, head_first=False)

    def ref(i, **kw):
        return oracle.gla(i["q"], i["k"], i["v"], gk=i["g"], gv=i["gv"], initial_state=i["h0"], output_final_state=True,
                          reverse=reverse, head_first=False)
    run_both(gpu, ref, d, ["q", "k", "v", "g", "gv", "h0"], tol=tol)


def test_fused_recurrent_simple_gla_varlen_and_golden(golden):
    T, N = 200, 3
    d = build(1, T, 2, 64, 64, torch.float32, seed=3, gate="scalar", h0=True, N=N)
    d["dht"] = d["dht"] * 0
    off = rand_offsets(T, N)

    def gpu(i, **kw):
        return ops().fused_recurrent_simple_gla(i["q"], i["k"], i["v"], i["g"], initial_state=i["h0"],
                                                output_final_state=True, offsets=off.to(DEV), head_first=False)
    run_both(gpu, lambda i, **kw: _sgla_ref(i, offsets=off), d, ["q", "k", "v", "g", "h0"])
    names = ("q", "k", "v", "gk", "h0")
    q, k, v, gk, h0 = (t(golden, f"gla.{n}").to(DEV) for n in names)
    o, ht = ops().fused_recurrent_gla(q, k, v, gk=gk, initial_state=h0, output_final_state=True, head_first=True)
    assert_close("o", t(golden, "gla.o"), o, 1e-5)
    assert_close("ht", t(golden, "gla.ht"), ht, 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("K,V,vec_beta", [(64, 64, False), (100, 60, True), (200, 128, False)])
def test_fused_recurrent_delta_rule(dtype, K, V, vec_beta):
    d = build(2, 70, 2, K, V, dtype, seed=K, beta=True, h0=True, norm=True)
    if vec_beta:
        d["beta"] = torch.rand(2, 70, 2, V, generator=torch.Generator().manual_seed(2)).sigmoid().to(dtype)
    tol = 2e-5 if dtype == torch.float32 else 6e-3

    def gpu(i, **kw):
        return ops().fused_recurrent_delta_rule(i["q"], i["k"], i["v"], i["beta"], initial_state=i["h0"],
                                                output_final_state=True, head_first=False)
    run_both(gpu, _delta_ref, d, ["q", "k", "v", "beta", "h0"], tol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_recurrent_gated_delta_rule_decode(dtype):
    """Decode: one token per call, state carried call to call, against the oracle run over the whole sequence."""
    B, T, H, K, V = 3, 9, 2, 128, 128
    d = build(B, T, H, K, V, dtype, seed=4, gate="scalar", beta=True, h0=True, norm=True)
    i = {n: x.to(DEV) for n, x in d.items()}
    S = i["h0"].float()
    outs = []
    for s in range(T):
        sl = slice(s, s + 1)
        o, S = ops().fused_recurrent_gated_delta_rule(i["q"][:, sl], i["k"][:, sl], i["v"][:, sl], i["g"][:, sl],
                                                      i["beta"][:, sl], initial_state=S, output_final_state=True,
                                                      head_first=False)
        outs.append(o)
    o = torch.cat(outs, 1)
    r = {n: (x.float() if x.is_floating_point() else x) for n, x in d.items()}
    o_ref, ht_ref = oracle.gated_delta_rule(r["q"], r["k"], r["v"], r["beta"], g=r["g"], initial_state=r["h0"],
                                            output_final_state=True, head_first=False)
    tol = 2e-5 if dtype == torch.float32 else 5e-3
    assert_close("o", o_ref, o, tol)
    assert_close("ht", ht_ref, S, tol)
    with pytest.raises(NotImplementedError):
        q = i["q"].clone().requires_grad_(True)
        o, _ = ops().fused_recurrent_gated_delta_rule(q, i["k"], i["v"], i["g"], i["beta"], head_first=False)
        o.sum().backward()


# ------------------------------------------------------------------------------------------------
# properties that do not depend on an oracle (usable at full benchmark sizes)
# ------------------------------------------------------------------------------------------------
def test_state_handoff_equals_one_shot():
    """Running T tokens in two halves, passing ht -> h0, gives the one-shot result (checkpoint/resume semantics)."""
    d = build(2, 512, 4, 128, 128, torch.bfloat16, seed=21, gate="scalar", beta=True, norm=True)
    i = {n: x.to(DEV) for n, x in d.items()}
    o_ = ops()
    o, ht = o_.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], output_final_state=True, head_first=False)
    h = 256
    o1, s1 = o_.chunk_gated_delta_rule(i["q"][:, :h], i["k"][:, :h], i["v"][:, :h], i["g"][:, :h], i["beta"][:, :h],
                                       output_final_state=True, head_first=False)
    o2, s2 = o_.chunk_gated_delta_rule(i["q"][:, h:], i["k"][:, h:], i["v"][:, h:], i["g"][:, h:], i["beta"][:, h:],
                                       initial_state=s1, output_final_state=True, head_first=False)
    assert err_ratio(o, torch.cat([o1, o2], 1)) < 1e-6
    assert err_ratio(ht, s2) < 1e-6


def test_chunk_equals_recurrent_at_benchmark_shape_and_is_deterministic():
    """B=2 slice of the headline shape (H=16, K=V=128, T=4096): chunk kernels vs the recurrent kernel, twice."""
    d = build(2, 4096, 16, 128, 128, torch.bfloat16, seed=33, gate="scalar", beta=True, h0=True, norm=True)
    i = {n: x.to(DEV) for n, x in d.items()}
    o_ = ops()
    args = (i["q"], i["k"], i["v"], i["g"], i["beta"])
    o1, h1 = o_.chunk_gated_delta_rule(*args, initial_state=i["h0"], output_final_state=True, head_first=False)
    o2, h2 = o_.chunk_gated_delta_rule(*args, initial_state=i["h0"], output_final_state=True, head_first=False)
    assert torch.equal(o1, o2) and torch.equal(h1, h2)
    o3, h3 = o_.fused_recurrent_gated_delta_rule(*args, initial_state=i["h0"], output_final_state=True, head_first=False)
    assert_close("o chunk vs recurrent", o3, o1, 5e-3)
    assert_close("ht chunk vs recurrent", h3, h1, 5e-3)


def test_linearity_in_v_at_benchmark_shape():
    """o is linear in v for fixed q, k, g, beta: f(v1 + v2) = f(v1) + f(v2) up to rounding."""
    d = build(1, 4096, 16, 128, 128, torch.bfloat16, seed=34, gate="scalar", beta=True, norm=True)
    i = {n: x.to(DEV) for n, x in d.items()}
    v2 = torch.randn_like(i["v"])
    f = lambda v: ops().chunk_gated_delta_rule(i["q"], i["k"], v, i["g"], i["beta"], head_first=False)[0].float()  # noqa: E731
    assert err_ratio(f(i["v"]) + f(v2), f(i["v"] + v2)) < 1e-2


def test_recompute_path_matches_saved_state_path(monkeypatch):
    """FLA_B200_SAVE_STATES=0 recomputes w, u, h, v_new in backward like the reference; both give the same grads."""
    import fla_b200.ops.gated_delta_rule as gdr
    import fla_b200.ops.simple_gla as sg
    d = build(2, 200, 2, 64, 64, torch.bfloat16, seed=12, gate="scalar", beta=True, h0=True, norm=True)
    names = ["q", "k", "v", "g", "beta", "h0"]

    def grads(mod, save):
        monkeypatch.setattr(mod, "SAVE_STATES", save)
        i = {n: d[n].to(DEV).clone().requires_grad_(True) for n in names}
        if mod is gdr:
            o, ht = gdr.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"],
                                               output_final_state=True, head_first=False)
            ins = [i[n] for n in names]
        else:
            o, ht = sg.chunk_simple_gla(i["q"], i["k"], i["v"], i["g"], initial_state=i["h0"], output_final_state=True,
                                        head_first=False)
            ins = [i[n] for n in ("q", "k", "v", "g", "h0")]
        return torch.autograd.grad((o.float() * d["do"].to(DEV).float()).sum() + (ht * d["dht"].to(DEV)).sum(), ins)
    for mod in (gdr, sg):
        for a_, b_ in zip(grads(mod, True), grads(mod, False)):
            assert err_ratio(a_, b_) < 1e-5  # dg is reduced with shared-memory float atomics: last-bit order effects


def test_fused_forward_entry_equals_staged_forward():
    """flab_gated_delta_rule_fwd (one call, workspace) against the stage-by-stage forward, fixed and varlen."""
    o_ = ops()
    for T, N in ((300, None), (500, 4)):
        B = 2 if N is None else 1
        d = build(B, T, 3, 128, 128, torch.bfloat16, seed=T, gate="scalar", beta=True, h0=True, norm=True, N=N)
        i = {n: x.to(DEV) for n, x in d.items()}
        off = None if N is None else rand_offsets(T, N).to(DEV)
        with torch.no_grad():  # no gradient needed -> fused entry
            o1, h1 = o_.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"],
                                               output_final_state=True, offsets=off, head_first=False)
        q = i["q"].clone().requires_grad_(True)  # gradient needed -> staged autograd path
        o2, h2 = o_.chunk_gated_delta_rule(q, i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"],
                                           output_final_state=True, offsets=off, head_first=False)
        assert torch.equal(o1, o2) and torch.equal(h1, h2)


def test_one_long_sequence_tail_matches_recurrent():
    """B=1, T=2^18, H=16: 64-bit offsets and 32-bit tile coordinates hold; the last 2048 tokens of the chunked
    forward agree with the token-recurrent kernel started from the chunked state at T-2048."""
    import torch.nn.functional as F
    from fla_b200.ops import chunk_gated_delta_rule, fused_recurrent_gated_delta_rule
    T, H, K, V, tail = 1 << 18, 16, 128, 128, 2048
    g0 = torch.Generator(device="cuda").manual_seed(5)
    q = F.normalize(torch.randn(1, T, H, K, device="cuda", generator=g0), dim=-1).bfloat16()
    k = F.normalize(torch.randn(1, T, H, K, device="cuda", generator=g0), dim=-1).bfloat16()
    v = torch.randn(1, T, H, V, device="cuda", generator=g0).bfloat16()
    g = F.logsigmoid(torch.randn(1, T, H, device="cuda", generator=g0)) * 0.1
    beta = torch.rand(1, T, H, device="cuda", generator=g0).sigmoid().bfloat16()
    with torch.no_grad():
        o, ht = chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True, head_first=False)
        cut = T - tail
        _, h_cut = chunk_gated_delta_rule(q[:, :cut], k[:, :cut], v[:, :cut], g[:, :cut], beta[:, :cut],
                                          output_final_state=True, head_first=False)
        o_t, ht_t = fused_recurrent_gated_delta_rule(q[:, cut:], k[:, cut:], v[:, cut:], g[:, cut:], beta[:, cut:],
                                                     initial_state=h_cut, output_final_state=True, head_first=False)
    assert torch.isfinite(o).all()
    assert_close("o tail", o_t, o[:, cut:], 5e-3)
    assert_close("ht", ht_t, ht, 5e-3)


@pytest.mark.gpu
def test_decoder_graph_replay_matches_functional_api():
    """The CUDA-graph decode loop (state updated in place) gives bit-identical o and state to calling
    fused_recurrent_gated_delta_rule once per token."""
    from fla_b200.decode import GatedDeltaRuleDecoder
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    torch.manual_seed(11)
    B, H, K, V, steps = 5, 3, 128, 128, 6
    dt = torch.bfloat16
    h0 = torch.randn(B, H, K, V, device="cuda") * 0.1
    dec = GatedDeltaRuleDecoder(B, H, K, V, dtype=dt, initial_state=h0)
    eager = GatedDeltaRuleDecoder(B, H, K, V, dtype=dt, initial_state=h0, use_graph=False)
    S = h0.clone()
    for t in range(steps):
        q = torch.randn(B, 1, H, K, device="cuda").to(dt)
        k = torch.nn.functional.normalize(torch.randn(B, 1, H, K, device="cuda"), dim=-1).to(dt)
        v = torch.randn(B, 1, H, V, device="cuda").to(dt)
        g = torch.nn.functional.logsigmoid(torch.randn(B, 1, H, device="cuda"))
        beta = torch.rand(B, 1, H, device="cuda").to(dt)
        o_ref, S = fused_recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=S, output_final_state=True, head_first=False)
        o = dec.step(q, k, v, g, beta)
        o2 = eager.step(q, k, v, g, beta)
        assert torch.equal(o, o_ref) and torch.equal(o2, o_ref), t
    assert torch.equal(dec.state, S) and torch.equal(eager.state, S)
    from fla_b200 import _lib
    assert _lib.load().flab_tc_error_state() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("family,B,T,gate_div", [
    ("gated", 1, 1100, 30.0),   # weak decay: the slabs' transitions M matter; ragged last slab and chunk
    ("gated", 2, 1024, 1.0),
    ("delta", 1, 1024, None),
])
def test_scan_split_into_slabs_matches_oracle(monkeypatch, family, B, T, gate_div):
    """The slab-split scans (forced at a small T) against the oracle, forward and every gradient, at the same bars
    as the one-chain scans; and the split really ran (transitions M saved)."""
    from fla_b200.ops import common as C
    monkeypatch.setattr(C, "SLAB_MIN_CHUNKS", 8)
    monkeypatch.setattr(C, "SLAB_MIN_CHUNKS_PER_SLAB", 3)
    H, K, V = 2, 128, 128
    if family == "gated":
        d = build(B, T, H, K, V, torch.bfloat16, seed=T, gate="scalar", beta=True, h0=True, norm=True, gate_div=gate_div)
        names, gpu, ref = ["q", "k", "v", "g", "beta", "h0"], _gdelta_gpu, _gdelta_ref
    else:
        d = build(B, T, H, K, V, torch.bfloat16, seed=T, beta=True, h0=True, norm=True)
        names, gpu, ref = ["q", "k", "v", "beta", "h0"], _delta_gpu, _delta_ref
    from fla_b200.utils import Geometry
    kk = d["k"].to(DEV)
    plan = C.slab_plan(Geometry(kk, d["v"].to(DEV), None, False), kk)
    assert plan is not None and plan.S >= 4
    run_both(gpu, ref, d, names, head_first=False, tol_over=DELTA_TOL)
    # forward only (no autograd): the same split
    with torch.no_grad():
        i = {n: x.to(DEV) for n, x in d.items()}
        o, ht = gpu(i, head_first=False)
        o_r, ht_r = ref({n: (x.float() if x.is_floating_point() else x) for n, x in d.items()})
    assert_close("o (no grad)", o_r, o, 5e-3)
    assert_close("ht (no grad)", ht_r, ht, 5e-3)


# ------------------------------------------------------------------------------------------------
# the step before the chunk ops: row-wise L2 normalisation (fla/modules/l2norm.py)
# ------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("shape,dtype,out_dtype", [
    ((2, 300, 4, 128), torch.bfloat16, None),
    ((2, 300, 4, 128), torch.float16, torch.float32),
    ((3, 77, 2, 64), torch.bfloat16, None),
    ((1, 50, 3, 256), torch.float32, None),
    ((1, 50, 3, 256), torch.float32, torch.bfloat16),
    ((5, 100), torch.float32, None),          # row length that takes the column-loop kernel
    ((4, 9, 72), torch.bfloat16, None),
    ((1, 1, 1, 8), torch.float16, None),
    ((0, 128), torch.bfloat16, None),         # empty input
])
def test_l2_norm_matches_oracle(shape, dtype, out_dtype):
    from fla_b200.modules import l2_norm
    g0 = torch.Generator().manual_seed(sum(shape) + 1)
    x = (torch.randn(*shape, generator=g0) * 2).to(dtype)
    dy = torch.randn(*shape, generator=g0).to(out_dtype or dtype)
    xg = x.to(DEV).requires_grad_(True)
    y = l2_norm(xg, 1e-6, out_dtype)
    assert y.shape == x.shape and y.dtype == (out_dtype or dtype)
    if x.numel() == 0:
        return
    tol = 1e-6 if (dtype == torch.float32 and out_dtype in (None, torch.float32)) else 5e-3
    assert_close("y", oracle.l2_norm(x, 1e-6, out_dtype), y, tol)
    y.backward(dy.to(DEV))
    assert_close("dx", oracle.l2_norm_bwd(x, dy.to(dtype), 1e-6), xg.grad, 1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.gpu
def test_l2_norm_reference_kernel_vectors():
    """The CUDA kernels on the inputs of tests/golden/l2norm_vectors.npz (outputs of the reference's own kernels)."""
    import numpy as np
    from fla_b200.modules.l2norm import l2norm_bwd, l2norm_fwd
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "l2norm_vectors.npz"))
    for case in ("f32_128", "f32_100", "f16_64", "f32_tiny"):
        x, dy, y, dx = (torch.from_numpy(z[f"{case}.{n}"]) for n in ("x", "dy", "y", "dx"))
        tol = 1e-6 if x.dtype == torch.float32 else 1e-3
        assert_close(f"{case} y", y, l2norm_fwd(x.to(DEV), 1e-6), tol)
        assert_close(f"{case} dx", dx, l2norm_bwd(x.to(DEV), dy.to(DEV), 1e-6), tol)


# ------------------------------------------------------------------------------------------------
# against outputs of the reference's own CHUNKED Triton kernels (tests/golden/triton_vectors.npz, produced by
# tests/golden/make_golden_triton.py under Triton's CPU interpreter): rel-L2 <= 5e-3 for 16-bit inputs, <= 1e-5 fp32
# ------------------------------------------------------------------------------------------------
def _triton_case(case, names):
    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "triton_vectors.npz"))
    x = {n: torch.from_numpy(z[f"{case}.{n}"]).to(DEV) for n in names}
    ref = {n[len(case) + 1:]: torch.from_numpy(z[n]) for n in z.files if n.startswith(case + ".")}
    return x, ref


def _compare_with_triton(case, call, names, grad_names, tol, grad_tol=None):
    x, ref = _triton_case(case, names)
    for n in grad_names:
        x[n].requires_grad_(True)
    o, ht = call(x, ref)
    print(f"{case} o: {assert_close(f'{case} o', ref['o'].float(), o, tol):.2e}  ht: {assert_close(f'{case} ht', ref['ht'].float(), ht, tol):.2e}")
    if grad_names:
        torch.autograd.backward([o, ht], [ref["do"].to(DEV), ref["dht"].to(DEV)])
        for n in grad_names:
            r_ = assert_close(f"{case} d{n}", ref[f"d{n}"].float(), x[n].grad, (grad_tol or {}).get(n, tol))
            print(f"{case} d{n}: {r_:.2e}")


@pytest.mark.gpu
def test_against_reference_chunk_kernel_outputs():
    o_ = ops()
    gd = ["q", "k", "v", "g", "beta", "h0"]
    gt = None  # measured: every output and gradient of the 16-bit cases within 6e-4, of the fp32 case within 5e-7
    _compare_with_triton("gdn_128", lambda x, r: o_.chunk_gated_delta_rule(
        x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True, head_first=False), gd, gd, 5e-3, gt)
    _compare_with_triton("gdn_varlen", lambda x, r: o_.chunk_gated_delta_rule(
        x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True,
        cu_seqlens=r["offsets"].to(DEV), head_first=False), gd, gd, 5e-3, gt)
    _compare_with_triton("delta_128", lambda x, r: o_.chunk_delta_rule(
        x["q"], x["k"], x["v"], x["beta"], initial_state=x["h0"], output_final_state=True, head_first=False),
        ["q", "k", "v", "beta", "h0"], [], 5e-3)
    sg = ["q", "k", "v", "g", "h0"]
    _compare_with_triton("simple_gla", lambda x, r: o_.chunk_simple_gla(
        x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True, head_first=False), sg, sg, 5e-3)
    _compare_with_triton("gla_f32", lambda x, r: o_.chunk_gla(
        x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True, head_first=False), sg, sg, 1e-5)
    rt = ["q", "k", "v", "h0"]
    _compare_with_triton("retention", lambda x, r: o_.chunk_retention(
        x["q"], x["k"], x["v"], initial_state=x["h0"], output_final_state=True, head_first=False), rt, rt, 5e-3)
    _compare_with_triton("decode", lambda x, r: o_.fused_recurrent_gated_delta_rule(
        x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True, head_first=False), gd, [], 5e-3)


# ------------------------------------------------------------------------------------------------
# the step after the chunk ops: RMS norm with weight times swish gate (fla/modules/fused_norm_gate.py)
# ------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("shape,dtype", [
    ((2, 300, 4, 128), torch.bfloat16),
    ((2, 130, 3, 128), torch.float16),
    ((3, 77, 2, 64), torch.bfloat16),
    ((1, 50, 3, 128), torch.float32),
    ((5, 100), torch.float32),              # row length that takes the column-loop kernel
    ((4, 9, 72), torch.bfloat16),
    ((1, 1, 1, 8), torch.float16),
    ((1, 7000, 16, 128), torch.bfloat16),   # more rows than one wave of blocks: several row passes per warp
])
def test_rms_norm_swish_gate_matches_oracle(shape, dtype):
    from fla_b200.modules import FusedRMSNormSwishGate
    g0 = torch.Generator().manual_seed(sum(shape) + 3)
    x = torch.randn(*shape, generator=g0).to(dtype)
    gate = torch.randn(*shape, generator=g0).to(dtype)
    dy = torch.randn(*shape, generator=g0).to(dtype)
    w = 1 + 0.1 * torch.randn(shape[-1], generator=g0)
    mod = FusedRMSNormSwishGate(shape[-1], eps=1e-5).to(DEV)
    with torch.no_grad():
        mod.weight.copy_(w)
    xg, gg = x.to(DEV).requires_grad_(True), gate.to(DEV).requires_grad_(True)
    y = mod(xg, gg)
    assert y.shape == x.shape and y.dtype == dtype
    tol = 1e-6 if dtype == torch.float32 else 5e-3
    assert_close("y", oracle.rms_norm_swish_gate(x, gate, w, 1e-5), y, tol)
    y.backward(dy.to(DEV))
    rx, rg, rw = oracle.rms_norm_swish_gate_bwd(x, gate, w, dy, 1e-5)
    assert_close("dx", rx, xg.grad, tol)
    assert_close("dgate", rg, gg.grad, tol)
    assert_close("dw", rw, mod.weight.grad, 1e-5 if dtype == torch.float32 else 5e-3)


@pytest.mark.gpu
def test_rms_norm_swish_gate_reference_kernel_vectors():
    """The CUDA kernels on the inputs of tests/golden/norm_gate_vectors.npz (outputs of the reference's own kernels)."""
    import numpy as np
    from fla_b200.modules import rms_norm_swish_gate_fn
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "norm_gate_vectors.npz"))
    for case in ("f32_128", "f16_128", "f32_100", "f16_64"):
        x, gate, w, dy, y, dx, dgate, dw = (torch.from_numpy(z[f"{case}.{n}"]).to(DEV) for n in ("x", "gate", "w", "dy", "y", "dx", "dgate", "dw"))
        tol = 1e-6 if x.dtype == torch.float32 else 1e-3
        x.requires_grad_(True), gate.requires_grad_(True), w.requires_grad_(True)
        out = rms_norm_swish_gate_fn(x, gate, w, eps=1e-5)
        assert_close(f"{case} y", y, out, tol)
        out.backward(dy)
        assert_close(f"{case} dx", dx, x.grad, tol)
        assert_close(f"{case} dgate", dgate, gate.grad, tol)
        assert_close(f"{case} dw", dw, w.grad, 1e-5 if x.dtype == torch.float32 else 1e-3)


# ------------------------------------------------------------------------------------------------
# the convolution in front of q, k, v (fla/modules/convolution.py ShortConvolution)
# ------------------------------------------------------------------------------------------------
def _short_conv_module(D, W, bias, act, weight, bias_t, dtype):
    from fla_b200.modules import ShortConvolution
    conv = ShortConvolution(D, W, bias=bias, activation=act).to(DEV)
    with torch.no_grad():
        conv.weight.copy_(weight.reshape(D, 1, W))
        if bias:
            conv.bias.copy_(bias_t)
    return conv


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,D,W,bias,act,dtype", [
    (2, 300, 256, 4, False, "silu", torch.bfloat16),
    (2, 100, 2048, 4, False, "silu", torch.bfloat16),   # the layer's width (16 heads x 128)
    (1, 33, 64, 3, True, None, torch.float16),
    (3, 2, 32, 4, True, "silu", torch.float32),         # shorter than the filter
    (1, 65, 40, 2, True, "silu", torch.float32),
])
def test_short_conv_matches_oracle(B, T, D, W, bias, act, dtype):
    g0 = torch.Generator().manual_seed(B * T + D + W)
    x = torch.randn(B, T, D, generator=g0).to(dtype)
    dy = torch.randn(B, T, D, generator=g0).to(dtype)
    w = torch.randn(D, W, generator=g0) * 0.5
    bt = torch.randn(D, generator=g0) * 0.1 if bias else None
    conv = _short_conv_module(D, W, bias, act, w, bt, dtype)
    xg = x.to(DEV).requires_grad_(True)
    y, cache = conv(xg, output_final_state=True)
    xr, wr = x.float().requires_grad_(True), w.clone().requires_grad_(True)
    br = None if bt is None else bt.clone().requires_grad_(True)
    y_ref, cache_ref = oracle.short_conv(xr, wr, br, act is not None)
    tol = 1e-6 if dtype == torch.float32 else 5e-3
    assert_close("y", y_ref, y, tol)
    assert torch.equal(cache.cpu().float(), cache_ref)
    y.backward(dy.to(DEV))
    gr = torch.autograd.grad((y_ref * dy.float()).sum(), [xr, wr] + ([br] if br is not None else []))
    assert_close("dx", gr[0], xg.grad, tol)
    assert_close("dweight", gr[1], conv.weight.grad.reshape(D, W), 1e-5 if dtype == torch.float32 else 5e-3)
    if bias:
        assert_close("dbias", gr[2], conv.bias.grad, 1e-5 if dtype == torch.float32 else 5e-3)
    # decode steps from the cache
    c_ref = cache_ref.to(dtype)
    for t in range(3):
        xs = torch.randn(B, 1, D, generator=g0).to(dtype)
        with torch.no_grad():
            yt, cache = conv(xs.to(DEV), cache=cache)
        yt_ref, c_ref = oracle.short_conv_step(xs, c_ref, w, bt, act is not None)
        assert_close(f"step {t}", yt_ref, yt, tol)
        assert torch.equal(cache.cpu(), c_ref)


@pytest.mark.gpu
def test_short_conv_reference_module_vectors():
    """The CUDA kernels on the inputs of tests/golden/short_conv_vectors.npz (outputs of the reference's module)."""
    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "short_conv_vectors.npz"))
    for case in ("w4_silu", "w3_bias", "w2_silu_bias"):
        g = {k[len(case) + 1:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(case + ".")}
        silu, bias = bool(g["silu"].item()), g.get("bias")
        B, T, D = g["x"].shape
        W = g["weight"].shape[-1]
        conv = _short_conv_module(D, W, bias is not None, "silu" if silu else None, g["weight"], bias, torch.float32)
        x = g["x"].to(DEV).requires_grad_(True)
        y, cache = conv(x, output_final_state=True)
        assert_close(f"{case} y", g["y"], y, 1e-6)
        assert torch.equal(cache.cpu(), g["cache"])
        y.backward(g["dy"].to(DEV))
        assert_close(f"{case} dx", g["dx"], x.grad, 1e-6)
        assert_close(f"{case} dweight", g["dweight"], conv.weight.grad, 1e-5)
        if bias is not None:
            assert_close(f"{case} dbias", g["dbias"], conv.bias.grad, 1e-5)
        with torch.no_grad():
            for t in range(3):
                yt, cache = conv(g["step_x"][:, t:t + 1].to(DEV), cache=cache)
                assert_close(f"{case} step {t}", g["step_y"][:, t:t + 1], yt, 1e-6)
        assert torch.equal(cache.cpu(), g["step_cache"])


@pytest.mark.gpu
def test_layer_pipeline_conv_norm_op_gate_matches_oracle_chain():
    """The data path of the reference's GatedDeltaNet layer around the op (fla/layers/gated_deltanet.py:205-282):
    short convolution + SiLU on q, k, v -> L2 norm of q, k -> chunk_gated_delta_rule -> RMS norm x swish gate, with this
    package's kernels end to end against the same chain of oracles, forward and the gradient of every input."""
    from fla_b200.modules import FusedRMSNormSwishGate, ShortConvolution, l2_norm
    from fla_b200.ops import chunk_gated_delta_rule
    B, T, H, D, W = 2, 200, 2, 128, 4
    dt = torch.bfloat16
    g0 = torch.Generator().manual_seed(77)
    xq, xk, xv, gate = (torch.randn(B, T, H * D, generator=g0).to(dt) for _ in range(4))
    wq, wk, wv = (torch.randn(H * D, W, generator=g0) * 0.5 for _ in range(3))
    gl = F.logsigmoid(torch.randn(B, T, H, generator=g0))
    beta = torch.rand(B, T, H, generator=g0).sigmoid().to(dt)
    wn = 1 + 0.1 * torch.randn(D, generator=g0)
    dout = torch.randn(B, T, H, D, generator=g0).to(dt)

    # this package
    convs = [_short_conv_module(H * D, W, False, "silu", w, None, dt) for w in (wq, wk, wv)]
    norm = FusedRMSNormSwishGate(D, eps=1e-5).to(DEV)
    with torch.no_grad():
        norm.weight.copy_(wn)
    ins = [t_.to(DEV).requires_grad_(True) for t_ in (xq, xk, xv, gate)]
    q, k, v = (c(x)[0].view(B, T, H, D) for c, x in zip(convs, ins[:3]))
    o, _ = chunk_gated_delta_rule(l2_norm(q), l2_norm(k), v, gl.to(DEV), beta.to(DEV), head_first=False)
    y = norm(o, ins[3].view(B, T, H, D))
    y.backward(dout.to(DEV))

    # the oracles, fp32 on the same bf16 inputs, rounding to bf16 where the kernels hand a tensor on
    rins = [t_.float().requires_grad_(True) for t_ in (xq, xk, xv, gate)]
    rq, rk, rv = (oracle.short_conv(x, w, None, True)[0].view(B, T, H, D) for x, w in zip(rins[:3], (wq, wk, wv)))
    ro, _ = oracle.gated_delta_rule(oracle.l2_norm(rq), oracle.l2_norm(rk), rv, beta.float(), g=gl, head_first=False)
    ry = oracle.rms_norm_swish_gate(ro, rins[3].view(B, T, H, D), wn, 1e-5)
    ry.backward(dout.float())

    print("layer pipeline y: %.2e" % assert_close("y", ry, y, 1e-2))
    for n, a, b in zip(("dxq", "dxk", "dxv", "dgate"), rins, ins):
        print("layer pipeline %s: %.2e" % (n, assert_close(n, a.grad, b.grad, 2e-2)))
