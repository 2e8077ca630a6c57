"""GPU: self-check of the TMA + tcgen05 + TMEM plumbing against plain matmuls."""
import ctypes

import pytest
import torch

from fla_b200 import _lib

pytestmark = pytest.mark.gpu


def test_tc_selftest():
    lib = _lib.load()
    g0 = torch.Generator().manual_seed(0)
    a = torch.randn(64, 128, generator=g0).bfloat16().cuda()
    b = torch.randn(64, 128, generator=g0).bfloat16().cuda()
    h = torch.randn(128, 128, generator=g0).bfloat16().cuda()
    v = torch.randn(64, 64, generator=g0).bfloat16().cuda()
    out = torch.zeros(64 * 64 + 64 * 128 + 128 * 64 + 64 * 64, device="cuda")
    status = torch.full((1,), -7, dtype=torch.int32, device="cuda")
    fn = lib.flab_tc_selftest
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7
    rc = fn(a.data_ptr(), b.data_ptr(), h.data_ptr(), v.data_ptr(), out.data_ptr(), status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.flab_last_error().decode()
    torch.cuda.synchronize()
    assert status.item() == 0, f"bounded wait {status.item()} ran out"
    af, bf, hf, vf = a.float(), b.float(), h.float(), v.float()
    d1 = af @ bf.T
    want = [d1, af @ hf, af.T @ vf, d1.bfloat16().float() @ vf]
    off = 0
    for i, w in enumerate(want):
        got = out[off:off + w.numel()].view_as(w)
        off += w.numel()
        err = ((got - w).norm() / w.norm()).item()
        print(f"D{i + 1}: rel err {err:.2e}")
        assert err < 2e-3, f"product {i + 1} differs: rel err {err:.3e}"


# ---------------------------------------------------------------------------------------------
# tcgen05 state scans against a plain fp32 PyTorch restatement of the same stage
# (fla/ops/common/chunk_delta_h.py:248-423, fla/ops/common/chunk_h.py:42-215), K = 128 so that the
# tensor-core kernels take the call; ragged sequences, both layouts, 64 / 128 / 256 value columns.
# ---------------------------------------------------------------------------------------------
def _rnd(x, dt):
    return x.to(dt).float()


def _chunks(T):
    return [(t, min(t + 64, T)) for t in range(0, T, 64)]


def _ref_delta_fwd(k, w, u, g, h0, dt):
    """Per (sequence, head) tensors [T, D] fp32. Returns h [NT,K,V], v_new [T,V], final state."""
    S = h0.clone()
    hs, vn = [], torch.zeros_like(u)
    for lo, hi in _chunks(k.shape[0]):
        hs.append(_rnd(S, dt))
        gc = g[lo:hi] if g is not None else torch.zeros(hi - lo, device=k.device)
        x = _rnd(u[lo:hi] - gc.exp()[:, None] * (w[lo:hi] @ _rnd(S, dt)), dt)
        vn[lo:hi] = x
        S = S * gc[-1].exp() + k[lo:hi].T @ _rnd(x * (gc[-1] - gc).exp()[:, None], dt)
    return torch.stack(hs), vn, S


def _ref_delta_bwd(q, k, w, do, dv, g, dht, scale, dt):
    S = dht.clone()
    T = q.shape[0]
    ch = _chunks(T)
    dhs, dv2 = [None] * len(ch), torch.zeros_like(dv)
    for i in range(len(ch) - 1, -1, -1):
        lo, hi = ch[i]
        dhs[i] = _rnd(S, dt)
        gc = g[lo:hi] if g is not None else torch.zeros(hi - lo, device=q.device)
        x = _rnd(dv[lo:hi] + (gc[-1] - gc).exp()[:, None] * (k[lo:hi] @ _rnd(S, dt)), dt)
        dv2[lo:hi] = x
        dop = _rnd(do[lo:hi] * (gc.exp() * scale)[:, None], dt)
        S = S * gc[-1].exp() + q[lo:hi].T @ dop - w[lo:hi].T @ _rnd(x * gc.exp()[:, None], dt)
    return torch.stack(dhs), dv2, S


def _ref_simple(x, y, g, s0, scale, bwd, dt):
    S = s0.clone()
    ch = _chunks(x.shape[0])
    hs = [None] * len(ch)
    for i in (range(len(ch) - 1, -1, -1) if bwd else range(len(ch))):
        lo, hi = ch[i]
        hs[i] = _rnd(S, dt)
        gc = g[lo:hi] if g is not None else torch.zeros(hi - lo, device=x.device)
        f = gc.exp() * scale if bwd else (gc[-1] - gc).exp()
        S = S * gc[-1].exp() + x[lo:hi].T @ _rnd(y[lo:hi] * f[:, None], dt)
    return torch.stack(hs), S


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("V,head_first,gated,lens", [
    (128, False, True, [200, 64, 333]),
    (64, False, False, [130]),
    (256, False, True, [191]),
    (128, True, True, None),
])
def test_tc_scans_against_torch(dt, V, head_first, gated, lens):
    from fla_b200.ops import common as C
    from fla_b200.utils import Geometry
    torch.manual_seed(3)
    H, K, scale = 2, 128, 128 ** -0.5
    if lens is None:
        B, T, offsets = 2, 150, None
        seqs = [(b, 0, T) for b in range(B)]
    else:
        B, T = 1, sum(lens)
        offs = [0]
        for L in lens:
            offs.append(offs[-1] + L)
        offsets = torch.tensor(offs, dtype=torch.long, device="cuda")
        seqs = [(0, offs[i], offs[i + 1]) for i in range(len(lens))]
    N = len(seqs)

    def tok(D, s=1.0):
        shape = (B, H, T, D) if head_first else (B, T, H, D)
        return (torch.randn(shape, device="cuda") * s).to(dt)

    q, k, w = tok(K, 0.3), tok(K, 0.3), tok(K, 0.1)
    u, do, dv = tok(V), tok(V), tok(V)
    g = None
    if gated:
        graw = -torch.rand((B, H, T) if head_first else (B, T, H), device="cuda") * 0.1
        g = C.chunk_local_cumsum(graw, offsets=offsets, head_first=head_first)
    h0 = torch.randn(N, H, K, V, device="cuda") * 0.1
    dht = torch.randn(N, H, K, V, device="cuda") * 0.1
    geo = Geometry(k, u, offsets, head_first)

    h, v_new, ht = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=g, h0=h0, output_final_state=True)
    dh, dh0, dv2 = C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, g=g, dht=dht, want_dh0=True)
    hs, hts = C.chunk_fwd_h(geo, k, u, g=g, h0=h0, output_final_state=True)
    dhs, dh0s = C.chunk_bwd_dh(geo, q, do, scale, g=g, dht=dht, want_dh0=True)
    torch.cuda.synchronize()
    assert _lib.load().flab_tc_error_state() == 0

    def sl(x, b, hd, lo, hi):
        return (x[b, hd, lo:hi] if head_first else x[b, lo:hi, hd]).float()

    c0 = 0
    for n, (b, lo, hi) in enumerate(seqs):
        nt = (hi - lo + 63) // 64
        for hd in range(H):
            gg = sl(g, b, hd, lo, hi) if gated else None
            args = [sl(x, b, hd, lo, hi) for x in (q, k, w, u, do, dv)]
            qq, kk, ww, uu, dd, dvv = args
            rh, rvn, rht = _ref_delta_fwd(kk, ww, uu, gg, h0[n, hd], dt)
            got_h = h.view(-1, H, K, V)[c0:c0 + nt, hd]
            assert _rel(got_h, rh) < 1e-2, ("h", n, hd, _rel(got_h, rh))
            assert _rel(sl(v_new, b, hd, lo, hi), rvn) < 1e-2
            assert _rel(ht[n, hd], rht) < 1e-2
            rdh, rdv2, rdh0 = _ref_delta_bwd(qq, kk, ww, dd, dvv, gg, dht[n, hd], scale, dt)
            assert _rel(dh.view(-1, H, K, V)[c0:c0 + nt, hd], rdh) < 1e-2
            assert _rel(sl(dv2, b, hd, lo, hi), rdv2) < 1e-2
            assert _rel(dh0[n, hd], rdh0) < 1e-2
            rhs, rhts = _ref_simple(kk, uu, gg, h0[n, hd], 1.0, False, dt)
            assert _rel(hs.view(-1, H, K, V)[c0:c0 + nt, hd], rhs) < 1e-2
            assert _rel(hts[n, hd], rhts) < 1e-2
            rdhs, rdh0s = _ref_simple(qq, dd, gg, dht[n, hd], scale, True, dt)
            assert _rel(dhs.view(-1, H, K, V)[c0:c0 + nt, hd], rdhs) < 1e-2
            assert _rel(dh0s[n, hd], rdh0s) < 1e-2
        c0 += nt


def _ref_gk(x, y, gk, s0, scale, bwd, dt):
    """Chunk-state scan with a gate per key channel: x = k (forward) or q (backward), gk [T, K] chunk-local cumsum."""
    S = s0.clone()
    ch = _chunks(x.shape[0])
    hs = [None] * len(ch)
    for i in (range(len(ch) - 1, -1, -1) if bwd else range(len(ch))):
        lo, hi = ch[i]
        hs[i] = _rnd(S, dt)
        gc = gk[lo:hi]
        f = gc.exp() * scale if bwd else (gc[-1:] - gc).exp()
        S = S * gc[-1].exp()[:, None] + _rnd(x[lo:hi] * f, dt).T @ y[lo:hi]
    return torch.stack(hs), S


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("V,head_first,lens", [
    (128, False, [200, 64, 333]),
    (256, False, [191]),
    (128, True, None),
])
def test_tc_channel_gate_scans_against_torch(dt, V, head_first, lens):
    from fla_b200.ops import common as C
    from fla_b200.utils import Geometry
    torch.manual_seed(5)
    H, K, scale = 2, 128, 128 ** -0.5
    if lens is None:
        B, T, offsets = 2, 150, None
        seqs = [(b, 0, T) for b in range(B)]
    else:
        B, T = 1, sum(lens)
        offs = [0]
        for L in lens:
            offs.append(offs[-1] + L)
        offsets = torch.tensor(offs, dtype=torch.long, device="cuda")
        seqs = [(0, offs[i], offs[i + 1]) for i in range(len(lens))]
    N = len(seqs)

    def tok(D, s=1.0):
        shape = (B, H, T, D) if head_first else (B, T, H, D)
        return (torch.randn(shape, device="cuda") * s).to(dt)

    q, k, v, do = tok(K, 0.3), tok(K, 0.3), tok(V), tok(V)
    graw = -torch.rand((B, H, T, K) if head_first else (B, T, H, K), device="cuda") * 0.2
    gk = C.chunk_local_cumsum(graw, offsets=offsets, head_first=head_first)
    h0 = torch.randn(N, H, K, V, device="cuda") * 0.1
    dht = torch.randn(N, H, K, V, device="cuda") * 0.1
    geo = Geometry(k, v, offsets, head_first)
    hs, hts = C.chunk_fwd_h(geo, k, v, gk=gk, h0=h0, output_final_state=True)
    dhs, dh0s = C.chunk_bwd_dh(geo, q, do, scale, gk=gk, dht=dht, want_dh0=True)
    torch.cuda.synchronize()
    assert _lib.load().flab_tc_error_state() == 0

    def sl(x, b, hd, lo, hi):
        return (x[b, hd, lo:hi] if head_first else x[b, lo:hi, hd]).float()

    c0 = 0
    for n, (b, lo, hi) in enumerate(seqs):
        nt = (hi - lo + 63) // 64
        for hd in range(H):
            qq, kk, vv, dd, gg = (sl(x, b, hd, lo, hi) for x in (q, k, v, do, gk))
            rhs, rhts = _ref_gk(kk, vv, gg, h0[n, hd], 1.0, False, dt)
            assert _rel(hs.view(-1, H, K, V)[c0:c0 + nt, hd], rhs) < 1e-2
            assert _rel(hts[n, hd], rhts) < 1e-2
            rdhs, rdh0s = _ref_gk(qq, dd, gg, dht[n, hd], scale, True, dt)
            assert _rel(dhs.view(-1, H, K, V)[c0:c0 + nt, hd], rdhs) < 1e-2
            assert _rel(dh0s[n, hd], rdh0s) < 1e-2
        c0 += nt


# ---------------------------------------------------------------------------------------------
# a bounded wait that runs out: the kernel returns, the host sees FLAB_E_TIMEOUT, the context stays usable
# ---------------------------------------------------------------------------------------------
def test_bounded_wait_runs_out_and_is_reported():
    """A warp waits, with a short limit (2^20 clock ticks, about half a millisecond), on a barrier that nothing
    arrives at. The kernel must come back by itself with the id of the wait; flab_tc_check() must then return
    FLAB_E_TIMEOUT (-4) with the id in the message, the record must clear, and the next ordinary kernel must run."""
    lib = _lib.load()
    torch.cuda.synchronize()
    assert lib.flab_tc_check() == 0, lib.flab_last_error().decode()
    status = torch.full((1,), -7, dtype=torch.int32, device="cuda")
    rc = lib.flab_tc_wait_selftest(1 << 20, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.flab_last_error().decode()
    torch.cuda.synchronize()
    assert status.item() == 99
    assert lib.flab_tc_error_state() == 99
    assert lib.flab_tc_check() == -4
    assert b"wait id 99" in lib.flab_last_error()
    with pytest.raises(RuntimeError, match="wait id 99"):
        _lib.check_device_waits("selftest")          # raises and clears
    assert lib.flab_tc_error_state() == 0
    assert lib.flab_tc_wait_selftest(0, status.data_ptr(), None) == -1   # limits outside (0, 2^28] are refused
    # the context is intact: an ordinary tcgen05 launch still works
    test_tc_selftest()
    assert lib.flab_tc_check() == 0


# ---------------------------------------------------------------------------------------------
# chain of slab transitions against the same chain written with torch.matmul
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,S,H,K,V,ld_extra", [(2, 5, 3, 128, 128, 128), (1, 1, 4, 128, 256, 0), (1, 3, 2, 100, 60, 0), (1, 16, 16, 128, 128, 128)])
def test_state_chain_matches_matmul_loop(B, S, H, K, V, ld_extra):
    g0 = torch.Generator(device="cuda").manual_seed(S * 7 + K)
    M = torch.randn(B, S, H, K, K, device="cuda", generator=g0) / K ** 0.5
    wide = torch.randn(B, S, H, K, V + ld_extra, device="cuda", generator=g0)
    b = wide[..., :V]
    s0 = torch.randn(B, H, K, V, device="cuda", generator=g0)
    for reverse, transpose, start in ((False, False, s0), (True, True, s0), (False, False, None)):
        s_in, s_last = _lib.state_chain(M, b, start, want_last=True, reverse=reverse, transpose=transpose)
        cur = torch.zeros_like(s0).double() if start is None else start.double()
        order = range(S - 1, -1, -1) if reverse else range(S)
        for s in order:
            ref_in = cur
            assert torch.allclose(s_in[:, s].double(), ref_in, rtol=1e-4, atol=1e-4), (reverse, s)
            Ms = M[:, s].double().transpose(-1, -2) if transpose else M[:, s].double()
            cur = Ms @ cur + b[:, s].double()
        assert torch.allclose(s_last.double(), cur, rtol=1e-4, atol=1e-4)


def test_inplace_state_needs_the_flag():
    """flab_recurrent_delta_fwd with ht == h0 is refused unless the caller sets FLAB_F_INPLACE_STATE."""
    B, H, K, V = 2, 2, 128, 128
    q = torch.randn(B, 1, H, K, device="cuda").bfloat16()
    v = torch.randn(B, 1, H, V, device="cuda").bfloat16()
    beta = torch.ones(B, 1, H, device="cuda").bfloat16()
    g = torch.zeros(B, 1, H, device="cuda")
    st = torch.zeros(B, H, K, V, device="cuda")
    o = torch.empty_like(v)
    kw = dict(B=B, T=1, H=H, K=K, V=V, N=B, NT=B, scale=1.0, q=q, k=q, v=v, beta=beta, g=g, h0=st, ht=st, o=o)
    with pytest.raises(RuntimeError, match="FLAB_F_INPLACE_STATE"):
        _lib.call("flab_recurrent_delta_fwd", q, flags=0, **kw)
    _lib.call("flab_recurrent_delta_fwd", q, flags=_lib.F_INPLACE_STATE, **kw)
    torch.cuda.synchronize()
