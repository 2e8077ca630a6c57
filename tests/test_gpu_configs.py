"""GPU parity at the benchmark configurations' OWN shapes.

Every case runs the full configuration on the GPU (forward and backward through the public API) and checks a
sample of its units against the CPU oracle on identical bits:

* fixed-length batches (retention / delta rule, B=8 T=4096 H=16 D=128): whole (batch row, head) chains - sequences
  and heads are independent, so the oracle run on one chain with its own initial state and final-state gradient is
  the exact reference for that slice of the batch;
* the packed variable-length batch (64 sequences, H=32): whole sequences (shortest, longest, ragged) x two heads,
  with int32 and int64 offsets;
* the one-sequence case (T = 2^20, scans split into slabs): windows at both ends of the sequence; the state entering
  a window and the state gradient leaving it are taken from GPU runs over the rest of the sequence, in fp32
  (final state of the prefix, initial-state gradient of the suffix), and given to the oracle;
* decode (256 sequences x 16 heads, one token per call): every output and the states.

Bars: relative L2 error (RMS(ref - out) / RMS(ref), the metric of the reference's tests/ops/utils.py:1-14)
<= 5e-3 for outputs, states and every gradient except those in LOOSE (d beta and d g of the gated rule, which pass
through the longest chains of bf16 intermediates: 1e-2, half the reference's own bar; d k of the plain delta rule,
whose state never decays: 6e-3). Every value is printed.
"""
import pytest
import torch
import torch.nn.functional as F

import oracle
from util import assert_close, err_ratio

pytestmark = pytest.mark.gpu
DEV = "cuda"
BAR = 5e-3
# per-gradient bars at these shapes; everything not listed is held to BAR. Measured on the B200 at these shapes
# (bf16): o, ht, dq, dk, dv, dh0 of the gated rule 1.5e-3 .. 3.8e-3; its dg up to 5.8e-3 and dbeta up to 6.3e-3 (the
# reference asserts 2e-2 for both, tests/ops/test_gated_delta.py:282-294). The plain delta rule has no decay, so the
# rounding of 4096 tokens of bf16 intermediates accumulates in the state: o 4.1e-3, dq 4.4e-3, dk 5.1e-3 (bar 6e-3; the
# reference asserts 8e-3, tests/ops/test_delta.py:74-93).
LOOSE = {"gated_delta": {"dbeta": 1e-2, "dg": 1e-2}, "delta": {"dk": 6e-3}}


def ops():
    import fla_b200.ops as o
    return o


def _bar(kind, name):
    return LOOSE.get(kind, {}).get(name, BAR)


def _oracle_chain(kind, x, S_in, do, dS_out, scale=None):
    """CPU fp32 oracle on one slice. x: dict of [1, T, h, *] tensors (any device / dtype). Returns dict of o, ht and
    gradients (dq, dk, dv, [dg], [dbeta], dh0)."""
    names = [n for n in ("q", "k", "v", "g", "beta") if n in x]
    leaf = {n: x[n].detach().float().cpu().clone().requires_grad_(True) for n in names}
    S = None if S_in is None else S_in.detach().float().cpu().clone().requires_grad_(True)
    if kind == "simple_gla":
        o, ht = oracle.simple_gla(leaf["q"], leaf["k"], leaf["v"], leaf["g"], scale=scale, initial_state=S,
                                  output_final_state=True, head_first=False)
    else:
        o, ht = oracle.gated_delta_rule(leaf["q"], leaf["k"], leaf["v"], leaf["beta"], g=leaf.get("g"), scale=scale,
                                        initial_state=S, output_final_state=True, head_first=False)
    loss = (o * do.detach().float().cpu()).sum()
    if dS_out is not None:
        loss = loss + (ht * dS_out.detach().float().cpu()).sum()
    ins = [leaf[n] for n in names] + ([S] if S is not None else [])
    grads = torch.autograd.grad(loss, ins)
    out = {"o": o.detach(), "ht": ht.detach()}
    for n, gx in zip(names + (["h0"] if S is not None else []), grads):
        out["d" + n] = gx
    return out


def _report(kind, tag, want, got, skip=()):
    res = {n: err_ratio(ref, got[n]) for n, ref in want.items() if n not in skip and n in got}
    print(tag, {n: f"{e:.2e}" for n, e in res.items()})
    bad = {n: (e, _bar(kind, n)) for n, e in res.items() if not e < _bar(kind, n)}
    assert not bad, f"{tag}: relative L2 error over the bar (value, bar): {bad}"
    return res


def _fixed_inputs(kind, B, T, H, K, V, seed):
    """The distributions of the benchmark configurations (seeded CPU generator, fp32, then cast)."""
    g0 = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, K, generator=g0), torch.randn(B, T, H, K, generator=g0)
    v = torch.randn(B, T, H, V, generator=g0)
    d = {}
    if kind in ("delta", "gated_delta"):
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
        d["beta"] = torch.randn(B, T, H, generator=g0).sigmoid().bfloat16()
        d["h0"] = torch.randn(B, H, K, V, generator=g0) * 0.1
    if kind == "gated_delta":
        d["g"] = F.logsigmoid(torch.randn(B, T, H, generator=g0))
    if kind == "simple_gla":
        s = (1 - torch.tensor(2.).pow(-5. - torch.arange(H, dtype=torch.float) * 7 / 16)).log()
        d["g"] = s[None, None, :].expand(B, T, H).contiguous()
    d.update(q=q.bfloat16(), k=k.bfloat16(), v=v.bfloat16())
    d["do"] = torch.randn(B, T, H, V, generator=g0).bfloat16()
    if "h0" in d:
        d["dht"] = torch.randn(B, H, K, V, generator=g0)
    return d


def _call(kind, x, **kw):
    o_ = ops()
    if kind == "simple_gla":
        return o_.chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], head_first=False, **kw)
    if kind == "delta":
        return o_.chunk_delta_rule(x["q"], x["k"], x["v"], x["beta"], head_first=False, **kw)
    return o_.chunk_gated_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], head_first=False, **kw)


GRADS = {"simple_gla": ["q", "k", "v", "g"], "delta": ["q", "k", "v", "beta"], "gated_delta": ["q", "k", "v", "g", "beta"]}


@pytest.mark.parametrize("kind", ["simple_gla", "delta", "gated_delta"])
def test_fixed_length_configs_whole_chains_against_oracle(kind):
    """B=8 T=4096 H=16 K=V=128 bf16 (retention decay / delta rule with initial state / the headline gated delta
    rule), forward + backward on the GPU at full shape; two (row, head) chains checked end to end."""
    B, T, H, K, V = 8, 4096, 16, 128, 128
    d = _fixed_inputs(kind, B, T, H, K, V, seed=3)
    x = {n: t_.to(DEV) for n, t_ in d.items()}
    for n in GRADS[kind] + (["h0"] if "h0" in x else []):
        x[n].requires_grad_(True)
    kw = dict(initial_state=x["h0"], output_final_state=True) if "h0" in x else dict(output_final_state=True)
    o, ht = _call(kind, x, **kw)
    if "h0" in x:
        torch.autograd.backward([o, ht], [x["do"], x["dht"]])
    else:
        torch.autograd.backward([o], [x["do"]])
    for b, h in ((0, 3), (7, 15)):
        sl = {n: x[n][b:b + 1, :, h:h + 1] for n in GRADS[kind]}
        S_in = x["h0"][b:b + 1, h:h + 1] if "h0" in x else None
        dS = x["dht"][b:b + 1, h:h + 1] if "h0" in x else None
        want = _oracle_chain(kind, sl, S_in, x["do"][b:b + 1, :, h:h + 1], dS)
        got = {"o": o[b:b + 1, :, h:h + 1], "ht": ht[b:b + 1, h:h + 1]}
        for n in GRADS[kind]:
            got["d" + n] = x[n].grad[b:b + 1, :, h:h + 1]
        if "h0" in x:
            got["dh0"] = x["h0"].grad[b:b + 1, h:h + 1]
        _report(kind, f"{kind} chain ({b},{h})", want, got)


def _varlen_lengths():
    return torch.randint(256, 8193, (64,), generator=torch.Generator().manual_seed(0))


def test_packed_varlen_config_whole_sequences_against_oracle():
    """64 sequences of 256..8192 tokens packed into one row, H=32 K=V=128 bf16, gated delta rule, forward + backward
    at full shape; offsets as int32 and as int64 give identical bits; three sequences x two heads against the oracle."""
    lens = _varlen_lengths()
    off = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
    T, H, K, V, N = int(off[-1]), 32, 128, 128, 64
    gen = torch.Generator(device=DEV).manual_seed(4)
    rn = lambda *s: torch.randn(*s, device=DEV, generator=gen)  # noqa: E731
    x = dict(q=F.normalize(rn(1, T, H, K), dim=-1).bfloat16(), k=F.normalize(rn(1, T, H, K), dim=-1).bfloat16(),
             v=rn(1, T, H, V).bfloat16(), g=F.logsigmoid(rn(1, T, H)), beta=rn(1, T, H).sigmoid().bfloat16(),
             h0=rn(N, H, K, V) * 0.1)
    do, dht = rn(1, T, H, V).bfloat16(), rn(N, H, K, V)
    with torch.no_grad():
        o32, ht32 = _call("gated_delta", x, initial_state=x["h0"], output_final_state=True, cu_seqlens=off.int().to(DEV))
    for n in x:
        x[n].requires_grad_(True)
    o, ht = _call("gated_delta", x, initial_state=x["h0"], output_final_state=True, cu_seqlens=off.to(DEV))
    assert torch.equal(o, o32) and torch.equal(ht, ht32), "int32 and int64 offsets must index identically"
    torch.autograd.backward([o, ht], [do, dht])
    order = lens.argsort()
    ragged = next(int(i) for i in order[len(order) // 2:] if int(lens[i]) % 64 not in (0, 63))
    for n_seq in (int(order[0]), int(order[-1]), ragged):
        a, b = int(off[n_seq]), int(off[n_seq + 1])
        for h in (1, 30):
            sl = {n: x[n][:, a:b, h:h + 1] for n in GRADS["gated_delta"]}
            want = _oracle_chain("gated_delta", sl, x["h0"][n_seq:n_seq + 1, h:h + 1], do[:, a:b, h:h + 1], dht[n_seq:n_seq + 1, h:h + 1])
            got = {"o": o[:, a:b, h:h + 1], "ht": ht[n_seq:n_seq + 1, h:h + 1], "dh0": x["h0"].grad[n_seq:n_seq + 1, h:h + 1]}
            for n in GRADS["gated_delta"]:
                got["d" + n] = x[n].grad[:, a:b, h:h + 1]
            _report("gated_delta", f"varlen seq {n_seq} (len {b - a}) head {h}", want, got)


def test_one_long_sequence_config_windows_against_oracle():
    """B=1 T=2^20 H=16 K=V=128 bf16, gated delta rule, forward + backward (the scans run split into slabs of T).
    The first and the last 512 tokens of two heads against the oracle; the state entering the last window is the
    fp32 final state of a GPU run over the prefix, the state gradient leaving the first window is the fp32
    initial-state gradient of a GPU run over the suffix."""
    T, H, K, V, W = 1 << 20, 16, 128, 128, 512
    gen = torch.Generator(device=DEV).manual_seed(6)
    rn = lambda *s: torch.randn(*s, device=DEV, generator=gen)  # noqa: E731
    x = dict(q=F.normalize(rn(1, T, H, K), dim=-1).bfloat16(), k=F.normalize(rn(1, T, H, K), dim=-1).bfloat16(),
             v=rn(1, T, H, V).bfloat16(), g=F.logsigmoid(rn(1, T, H)), beta=rn(1, T, H).sigmoid().bfloat16(),
             h0=rn(1, H, K, V) * 0.1)
    do, dht = rn(1, T, H, V).bfloat16(), rn(1, H, K, V)
    names = GRADS["gated_delta"]
    for n in x:
        x[n].requires_grad_(True)
    o, ht = _call("gated_delta", x, initial_state=x["h0"], output_final_state=True)
    torch.autograd.backward([o, ht], [do, dht])
    o, ht = o.detach(), ht.detach()
    grads = {n: x[n].grad for n in x}
    x = {n: t_.detach() for n, t_ in x.items()}
    assert all(torch.isfinite(g_).all() for g_ in grads.values())
    heads = (0, 15)
    # ---- last window: state at the cut from a forward over the prefix
    cut = T - W
    with torch.no_grad():
        _, S_cut = _call("gated_delta", {n: x[n][:, :cut] for n in names}, initial_state=x["h0"], output_final_state=True)
    for h in heads:
        sl = {n: x[n][:, cut:, h:h + 1] for n in names}
        want = _oracle_chain("gated_delta", sl, S_cut[:, h:h + 1], do[:, cut:, h:h + 1], dht[:, h:h + 1])
        got = {"o": o[:, cut:, h:h + 1], "ht": ht[:, h:h + 1]}
        for n in names:
            got["d" + n] = grads[n][:, cut:, h:h + 1]
        _report("gated_delta", f"long sequence, last {W} tokens, head {h}", want, got, skip=("dh0",))
    # ---- first window: gradient of the state at the cut from a forward + backward over the suffix
    with torch.no_grad():
        _, S_w = _call("gated_delta", {n: x[n][:, :W] for n in names}, initial_state=x["h0"], output_final_state=True)
    S_w = S_w.clone().requires_grad_(True)
    suffix = {n: x[n][:, W:].clone().requires_grad_(True) for n in names}  # (a gradient-requiring input selects the staged path)
    o_s, ht_s = _call("gated_delta", suffix, initial_state=S_w, output_final_state=True)
    torch.autograd.backward([o_s, ht_s], [do[:, W:], dht])
    dS_w = S_w.grad
    del o_s, ht_s, suffix
    for h in heads:
        sl = {n: x[n][:, :W, h:h + 1] for n in names}
        want = _oracle_chain("gated_delta", sl, x["h0"][:, h:h + 1], do[:, :W, h:h + 1], dS_w[:, h:h + 1])
        got = {"o": o[:, :W, h:h + 1], "dh0": grads["h0"][:, h:h + 1]}
        for n in names:
            got["d" + n] = grads[n][:, :W, h:h + 1]
        _report("gated_delta", f"long sequence, first {W} tokens, head {h}", want, got, skip=("ht",))


def test_decode_config_against_oracle():
    """256 sequences x 16 heads, K=V=128, one token per call, four calls with the fp32 state carried: every output and
    every state against the oracle."""
    B, H, K, V, steps = 256, 16, 128, 128, 4
    g0 = torch.Generator().manual_seed(8)
    q = F.normalize(torch.randn(B, steps, H, K, generator=g0), dim=-1).bfloat16()
    k = F.normalize(torch.randn(B, steps, H, K, generator=g0), dim=-1).bfloat16()
    v = torch.randn(B, steps, H, V, generator=g0).bfloat16()
    g = F.logsigmoid(torch.randn(B, steps, H, generator=g0))
    beta = torch.randn(B, steps, H, generator=g0).sigmoid().bfloat16()
    h0 = torch.randn(B, H, K, V, generator=g0) * 0.1
    S = h0.to(DEV)
    outs = []
    for s in range(steps):
        sl = slice(s, s + 1)
        o, S = ops().fused_recurrent_gated_delta_rule(q[:, sl].to(DEV), k[:, sl].to(DEV), v[:, sl].to(DEV), g[:, sl].to(DEV),
                                                      beta[:, sl].to(DEV), initial_state=S, output_final_state=True, head_first=False)
        outs.append(o)
    o_ref, S_ref = oracle.gated_delta_rule(q.float(), k.float(), v.float(), beta.float(), g=g, initial_state=h0,
                                           output_final_state=True, head_first=False)
    print("decode o", f"{assert_close('decode o', o_ref, torch.cat(outs, 1), BAR):.2e}",
          "state", f"{assert_close('decode state', S_ref, S, 1e-4):.2e}")
