"""CPU: the oracle restatement against vectors produced by the reference's own naive functions
(tests/golden/make_golden.py).  This is what pins the oracle."""
import torch

import oracle
from util import assert_close, t

TOL = 2e-5  # fp32 recurrences evaluated in a different association order


def _grads(outs, douts, inputs):
    loss = sum((o * d).sum() for o, d in zip(outs, douts))
    return torch.autograd.grad(loss, inputs)


def test_gla_matches_reference_naive(golden):
    q, k, v, gk, h0 = (t(golden, f"gla.{n}").requires_grad_(True) for n in ("q", "k", "v", "gk", "h0"))
    o, ht = oracle.gla(q, k, v, gk=gk, initial_state=h0, output_final_state=True, head_first=True)
    assert_close("o", t(golden, "gla.o"), o, TOL)
    assert_close("ht", t(golden, "gla.ht"), ht, TOL)
    gr = _grads((o, ht), (t(golden, "gla.do"), t(golden, "gla.dht")), (q, k, v, gk, h0))
    for name, gx in zip(("dq", "dk", "dv", "dgk", "dh0"), gr):
        assert_close(name, t(golden, f"gla.{name}"), gx, TOL)


def test_simple_gla_matches_reference_naive(golden):
    q, k, v, g, h0 = (t(golden, f"simple_gla.{n}").requires_grad_(True) for n in ("q", "k", "v", "g", "h0"))
    o, ht = oracle.simple_gla(q, k, v, g, initial_state=h0, output_final_state=True, head_first=True)
    assert_close("o", t(golden, "simple_gla.o"), o, TOL)
    assert_close("ht", t(golden, "simple_gla.ht"), ht, TOL)
    gr = _grads((o, ht), (t(golden, "simple_gla.do"), t(golden, "simple_gla.dht")), (q, k, v, g, h0))
    for name, gx in zip(("dq", "dk", "dv", "dg", "dh0"), gr):
        assert_close(name, t(golden, f"simple_gla.{name}"), gx, TOL)


def test_retention_matches_reference_naive(golden):
    q, k, v = (t(golden, f"retention.{n}") for n in ("q", "k", "v"))
    H = q.shape[1]
    g = oracle.retention_log_decay(H)[None, :, None].expand(q.shape[0], H, q.shape[2])
    o, _ = oracle.simple_gla(q, k, v, g, head_first=True)
    assert_close("o", t(golden, "retention.o"), o, TOL)


def test_delta_rule_matches_reference_naive(golden):
    q, k, v, beta, h0 = (t(golden, f"delta.{n}").requires_grad_(True) for n in ("q", "k", "v", "beta", "h0"))
    o, ht = oracle.delta_rule(q, k, v, beta, initial_state=h0, output_final_state=True, head_first=True)
    assert_close("o", t(golden, "delta.o"), o, TOL)
    assert_close("ht", t(golden, "delta.ht"), ht, TOL)
    gr = _grads((o, ht), (t(golden, "delta.do"), t(golden, "delta.dht")), (q, k, v, beta, h0))
    for name, gx in zip(("dq", "dk", "dv", "dbeta", "dh0"), gr):
        assert_close(name, t(golden, f"delta.{name}"), gx, TOL)


def test_gated_delta_rule_matches_reference_refs(golden):
    names = ("q", "k", "v", "beta", "g", "h0")
    q, k, v, beta, g, h0 = (t(golden, f"gated_delta.{n}").requires_grad_(True) for n in names)
    scale = float(golden["gated_delta.scale"])
    o, ht = oracle.gated_delta_rule(q, k, v, beta, g=g, scale=scale, initial_state=h0, output_final_state=True,
                                    head_first=False)
    assert_close("o", t(golden, "gated_delta.o"), o, TOL)
    assert_close("ht", t(golden, "gated_delta.ht"), ht, TOL)
    # the reference's chunked restatement agrees with its recurrent one to fp32 round-off
    assert_close("o_chunk", t(golden, "gated_delta.o_chunk"), o, 1e-4)
    gr = _grads((o, ht), (t(golden, "gated_delta.do"), t(golden, "gated_delta.dht")), (q, k, v, beta, g, h0))
    for name, gx in zip(("dq", "dk", "dv", "dbeta", "dg", "dh0"), gr):
        assert_close(name, t(golden, f"gated_delta.{name}"), gx, TOL)


def test_cumsum_matches_reference(golden):
    for name in ("s3", "s4"):
        x = t(golden, f"cumsum.{name}.x")
        for key, kw in (("local", dict(reverse=False)), ("local_rev", dict(reverse=True))):
            y = oracle.cumsum_local(x, 64, head_first=False, **kw)
            torch.testing.assert_close(y, t(golden, f"cumsum.{name}.{key}"))
        for key, kw in (("glob", dict(reverse=False)), ("glob_rev", dict(reverse=True))):
            y = oracle.cumsum_global(x, head_first=False, **kw)
            torch.testing.assert_close(y, t(golden, f"cumsum.{name}.{key}"))


def test_varlen_tables_bit_exact(golden):
    offsets = t(golden, "varlen.offsets")
    assert torch.equal(oracle.chunk_indices_ref(offsets), t(golden, "varlen.indices"))
    assert torch.equal(oracle.chunk_offsets_ref(offsets), t(golden, "varlen.chunk_offsets"))


def test_oracle_varlen_equals_per_sequence_runs():
    g0 = torch.Generator().manual_seed(7)
    T, H, K, V = 50, 2, 8, 8
    q, k, v = torch.randn(1, T, H, K, generator=g0), torch.randn(1, T, H, K, generator=g0), torch.randn(1, T, H, V, generator=g0)
    g = -torch.rand(1, T, H, generator=g0)
    beta = torch.rand(1, T, H, generator=g0)
    offsets = torch.tensor([0, 13, 13 + 30, 50])
    o, ht = oracle.gated_delta_rule(q, k, v, beta, g=g, offsets=offsets, output_final_state=True, head_first=False)
    for n, (a, b) in enumerate(zip(offsets[:-1].tolist(), offsets[1:].tolist())):
        on, hn = oracle.gated_delta_rule(q[:, a:b], k[:, a:b], v[:, a:b], beta[:, a:b], g=g[:, a:b],
                                         output_final_state=True, head_first=False)
        torch.testing.assert_close(o[:, a:b], on)
        torch.testing.assert_close(ht[n:n + 1], hn)


L2_CASES = ["f32_128", "f32_100", "f16_64", "f32_tiny"]


def _l2_golden():
    import os
    import numpy as np
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "l2norm_vectors.npz"))


def test_l2norm_matches_reference_kernels():
    """oracle.l2_norm / l2_norm_bwd against outputs of the reference's Triton kernels (CPU interpreter), and the
    backward formula against autograd of the forward in fp64."""
    z = _l2_golden()
    for case in L2_CASES:
        x, dy, y, dx = (torch.from_numpy(z[f"{case}.{n}"]) for n in ("x", "dy", "y", "dx"))
        tol = 1e-6 if x.dtype == torch.float32 else 1e-3
        assert_close(f"{case} y", y, oracle.l2_norm(x, 1e-6), tol)
        assert_close(f"{case} dx", dx, oracle.l2_norm_bwd(x, dy, 1e-6), tol)
    x = torch.randn(7, 96, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(7, 96, dtype=torch.float64)
    y = x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    gx, = torch.autograd.grad((y * dy).sum(), x)
    assert_close("dx vs autograd", gx.float(), oracle.l2_norm_bwd(x.detach().float(), dy.float(), 1e-6), 1e-5)


# ------------------------------------------------------------------------------------------------
# the oracle against outputs of the reference's CHUNKED Triton kernels (tests/golden/make_golden_triton.py: the
# kernels run unmodified under Triton's CPU interpreter).  16-bit cases are fp16.
# ------------------------------------------------------------------------------------------------
def _triton_golden():
    import os
    import numpy as np
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "triton_vectors.npz"))


# measured: 2e-4 .. 5e-4 on the fp16 cases (the kernels round operands to fp16, the oracle does not), 3e-7 on fp32
TRITON_TOL = {True: 2e-3, False: 2e-6}  # 16-bit case / fp32 case


def _check_against_triton(case, call, names, grad_names):
    z = _triton_golden()
    xs = {n: torch.from_numpy(z[f"{case}.{n}"]).float().requires_grad_(n in grad_names) for n in names}
    o, ht = call(xs, z)
    tol = TRITON_TOL[z[f"{case}.q"].dtype != "float32"]
    assert_close(f"{case} o", torch.from_numpy(z[f"{case}.o"]).float(), o, tol)
    assert_close(f"{case} ht", torch.from_numpy(z[f"{case}.ht"]).float(), ht, tol)
    if grad_names:
        do, dht = torch.from_numpy(z[f"{case}.do"]).float(), torch.from_numpy(z[f"{case}.dht"]).float()
        gr = torch.autograd.grad((o * do).sum() + (ht * dht).sum(), [xs[n] for n in grad_names])
        for n, gx in zip(grad_names, gr):
            assert_close(f"{case} d{n}", torch.from_numpy(z[f"{case}.d{n}"]).float(), gx, tol)


def test_oracle_matches_reference_chunk_kernels():
    gd = ["q", "k", "v", "g", "beta", "h0"]
    _check_against_triton("gdn_128", lambda x, z: oracle.gated_delta_rule(
        x["q"], x["k"], x["v"], x["beta"], g=x["g"], initial_state=x["h0"], output_final_state=True, head_first=False), gd, gd)
    _check_against_triton("gdn_varlen", lambda x, z: oracle.gated_delta_rule(
        x["q"], x["k"], x["v"], x["beta"], g=x["g"], initial_state=x["h0"], output_final_state=True,
        offsets=torch.from_numpy(z["gdn_varlen.offsets"]), head_first=False), gd, gd)
    _check_against_triton("delta_128", lambda x, z: oracle.delta_rule(
        x["q"], x["k"], x["v"], x["beta"], initial_state=x["h0"], output_final_state=True, head_first=False),
        ["q", "k", "v", "beta", "h0"], [])
    sg = ["q", "k", "v", "g", "h0"]
    _check_against_triton("simple_gla", lambda x, z: oracle.simple_gla(
        x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True, head_first=False), sg, sg)
    _check_against_triton("gla_f32", lambda x, z: oracle.gla(
        x["q"], x["k"], x["v"], gk=x["g"], initial_state=x["h0"], output_final_state=True, head_first=False), sg, sg)
    rt = ["q", "k", "v", "h0"]
    _check_against_triton("retention", lambda x, z: oracle.simple_gla(
        x["q"], x["k"], x["v"], oracle.retention_log_decay(x["q"].shape[2])[None, None, :].expand(x["q"].shape[:3]),
        initial_state=x["h0"], output_final_state=True, head_first=False), rt, rt)
    _check_against_triton("decode", lambda x, z: oracle.gated_delta_rule(
        x["q"], x["k"], x["v"], x["beta"], g=x["g"], initial_state=x["h0"], output_final_state=True, head_first=False), gd, [])


def test_norm_gate_matches_reference_kernels():
    """oracle.rms_norm_swish_gate(_bwd) against outputs of the reference's norm-gate kernels (CPU interpreter)."""
    import os
    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "norm_gate_vectors.npz"))
    for case in ("f32_128", "f16_128", "f32_100", "f16_64"):
        x, gate, w, dy, y, dx, dgate, dw = (torch.from_numpy(z[f"{case}.{n}"]) for n in ("x", "gate", "w", "dy", "y", "dx", "dgate", "dw"))
        tol = 1e-6 if x.dtype == torch.float32 else 1e-3
        assert_close(f"{case} y", y, oracle.rms_norm_swish_gate(x, gate, w, 1e-5), tol)
        gx, gg, gw = oracle.rms_norm_swish_gate_bwd(x, gate, w, dy, 1e-5)
        assert_close(f"{case} dx", dx, gx, tol)
        assert_close(f"{case} dgate", dgate, gg, tol)
        assert_close(f"{case} dw", dw, gw, 1e-5)
    # the backward formulas against autograd of the forward, fp64
    x = torch.randn(6, 80, dtype=torch.float64, requires_grad=True)
    gate = torch.randn(6, 80, dtype=torch.float64, requires_grad=True)
    w = torch.randn(80, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(6, 80, dtype=torch.float64)
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w * gate * torch.sigmoid(gate)
    ax, ag, aw = torch.autograd.grad((y * dy).sum(), (x, gate, w))
    gx, gg, gw = oracle.rms_norm_swish_gate_bwd(x.detach().float(), gate.detach().float(), w.detach().float(), dy.float(), 1e-5)
    assert_close("dx vs autograd", ax.float(), gx, 1e-5)
    assert_close("dgate vs autograd", ag.float(), gg, 1e-5)
    assert_close("dw vs autograd", aw.float(), gw, 1e-5)


SC_CASES = ["w4_silu", "w3_bias", "w2_silu_bias"]


def _sc_golden():
    import os
    import numpy as np
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "short_conv_vectors.npz"))


def test_short_conv_matches_reference_module():
    """oracle.short_conv / short_conv_step against the reference's ShortConvolution run on CPU."""
    z = _sc_golden()
    for case in SC_CASES:
        g = {k[len(case) + 1:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(case + ".")}
        silu, bias = bool(g["silu"].item()), g.get("bias")
        x, w = g["x"].clone().requires_grad_(True), g["weight"].clone().requires_grad_(True)
        b = None if bias is None else bias.clone().requires_grad_(True)
        y, cache = oracle.short_conv(x, w, b, silu)
        assert_close(f"{case} y", g["y"], y, 1e-6)
        assert torch.equal(cache, g["cache"])
        gr = torch.autograd.grad((y * g["dy"]).sum(), [x, w] + ([b] if b is not None else []))
        assert_close(f"{case} dx", g["dx"], gr[0], 1e-6)
        assert_close(f"{case} dweight", g["dweight"], gr[1], 1e-5)
        if b is not None:
            assert_close(f"{case} dbias", g["dbias"], gr[2], 1e-5)
        c = cache
        with torch.no_grad():
            for t in range(3):
                yt, c = oracle.short_conv_step(g["step_x"][:, t:t + 1], c, w, b, silu)
                assert_close(f"{case} step {t}", g["step_y"][:, t:t + 1], yt, 1e-6)
        assert torch.equal(c, g["step_cache"])


# ------------------------------------------------------------------------------------------------
# the remaining execution modes of the same recurrences (tests/golden/make_golden_f4.py: the reference's fused_chunk /
# parallel kernels and the gv mode of its chunk_fwd_h, run under Triton's CPU interpreter)
# ------------------------------------------------------------------------------------------------
def _f4():
    import os

    import numpy as np
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "f4_vectors.npz"))


def test_oracle_matches_reference_fused_chunk_and_parallel_kernels():
    z = _f4()
    f = lambda n: torch.from_numpy(z[n]).float()  # noqa: E731
    # fused_chunk_gla (fp32): same recurrence as chunk_gla
    q, k, v, g = (f(f"fused_chunk_gla.{n}").requires_grad_(True) for n in ("q", "k", "v", "g"))
    o, ht = oracle.gla(q, k, v, gk=g, initial_state=f("fused_chunk_gla.h0"), output_final_state=True, head_first=False)
    assert_close("fused_chunk_gla o", f("fused_chunk_gla.o"), o, 1e-5)
    assert_close("fused_chunk_gla ht", f("fused_chunk_gla.ht"), ht, 1e-5)
    # (the reference's fused backward ignores the gradient of the final state: fla/ops/gla/fused_chunk.py:497, fla/ops/retention/fused_chunk.py:265)
    gr = _grads((o,), (f("fused_chunk_gla.do"),), (q, k, v, g))
    for name, gx in zip(("dq", "dk", "dv", "dg"), gr):
        assert_close("fused_chunk_gla " + name, f(f"fused_chunk_gla.{name}"), gx, 2e-5)
    # fused_chunk_retention (fp16 inputs, fp32 accumulation inside the reference kernel)
    q, k, v = (f(f"fused_chunk_retention.{n}").requires_grad_(True) for n in ("q", "k", "v"))
    H = q.shape[2]
    gr_ = oracle.retention_log_decay(H)[None, None, :].expand(q.shape[0], q.shape[1], H)
    o, ht = oracle.simple_gla(q, k, v, gr_, initial_state=f("fused_chunk_retention.h0"), output_final_state=True, head_first=False)
    assert_close("fused_chunk_retention o", f("fused_chunk_retention.o"), o, 2e-3)
    assert_close("fused_chunk_retention ht", f("fused_chunk_retention.ht"), ht, 2e-3)
    gr = _grads((o,), (f("fused_chunk_retention.do"),), (q, k, v))
    for name, gx in zip(("dq", "dk", "dv"), gr):
        assert_close("fused_chunk_retention " + name, f(f"fused_chunk_retention.{name}"), gx, 2e-3)
    # parallel_simple_gla: o, gradients, and the attention matrix
    q, k, v, g = (f(f"parallel_simple_gla.{n}").requires_grad_(True) for n in ("q", "k", "v", "g"))
    o, _ = oracle.simple_gla(q, k, v, g, head_first=False)
    assert_close("parallel_simple_gla o", f("parallel_simple_gla.o"), o, 2e-3)
    gr = _grads((o,), (f("parallel_simple_gla.do"),), (q, k, v, g))
    for name, gx in zip(("dq", "dk", "dv", "dg"), gr):
        assert_close("parallel_simple_gla " + name, f(f"parallel_simple_gla.{name}"), gx, 2e-3)
    attn = oracle.simple_gla_attention(q.detach(), k.detach(), g.detach(), head_first=False)
    assert_close("parallel_simple_gla attn", f("parallel_simple_gla.attn"), attn, 2e-3)


def test_oracle_matches_reference_value_gate_state_scan():
    """chunk_fwd_h / chunk_bwd_dh with gv (the GSA path): chunk states and the final state from the token recurrence."""
    z = _f4()
    f = lambda n: torch.from_numpy(z[n]).float()  # noqa: E731
    k, v, q, gv, h0 = f("chunk_h_gv.k"), f("chunk_h_gv.v"), f("chunk_h_gv.q"), f("chunk_h_gv.gv"), f("chunk_h_gv.h0")
    h, ht = oracle.chunk_states(k, v, gv_cumsum=gv, initial_state=h0)
    assert_close("h", f("chunk_h_gv.h"), h, 2e-3)
    assert_close("ht", f("chunk_h_gv.ht"), ht, 2e-3)
    dh, dh0 = oracle.chunk_state_gradients(q, f("chunk_h_gv.do"), scale=k.shape[-1] ** -0.5, gv_cumsum=gv, dht=f("chunk_h_gv.dht"))
    assert_close("dh", f("chunk_h_gv.dh"), dh, 2e-3)
    assert_close("dh0", f("chunk_h_gv.dh0"), dh0, 2e-3)
