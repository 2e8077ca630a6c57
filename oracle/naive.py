"""Token-by-token recurrences (ground truth).  All functions take seq-first tensors [B,T,H,*] or
head-first [B,H,T,*], an optional `offsets` for packed variable-length batches, compute in
`dtype` (fp32 by default, fp64 for tight checks) and are differentiable with torch.autograd, which
is how the reference's own tests obtain reference gradients."""

from typing import Optional

import torch


def _split(x, offsets, head_first):
    """-> list of per-sequence head-first tensors [1,H,T_n,...] plus a function to re-assemble."""
    if x is None:
        return None
    if not head_first:
        x = x.transpose(1, 2)
    if offsets is None:
        return [x]
    off = [int(o) for o in offsets.tolist()]
    return [x[:, :, a:b] for a, b in zip(off[:-1], off[1:])]


def _run(step_fn, tensors, initial_state, output_final_state, offsets, head_first, K, V, dtype, reverse=False):
    """Drive `step_fn(S, t, seq_tensors) -> (S, o_t)` over every sequence."""
    seqs = [_split(x, offsets, head_first) for x in tensors]
    n_seq = len(seqs[0])
    outs, finals = [], []
    for n in range(n_seq):
        cur = [None if s is None else s[n].to(dtype) for s in seqs]
        Bn, H, Tn = cur[0].shape[:3]
        if initial_state is not None:
            S = (initial_state if offsets is None else initial_state[n:n + 1]).to(dtype)
        else:
            S = cur[0].new_zeros(Bn, H, K, V)
        o = [None] * Tn
        order = range(Tn - 1, -1, -1) if reverse else range(Tn)
        for t in order:
            S, o[t] = step_fn(S, t, cur)
        outs.append(torch.stack(o, 2) if Tn > 0 else cur[0].new_zeros(Bn, H, 0, V))
        finals.append(S)
    o = torch.cat(outs, 2) if offsets is not None else outs[0]
    if not head_first:
        o = o.transpose(1, 2)
    ht = torch.cat(finals, 0) if output_final_state else None
    return o, ht


def gla(q, k, v, gk=None, gv=None, g=None, scale=None, initial_state=None, output_final_state=False, reverse=False,
        offsets=None, head_first=True, dtype=torch.float32):
    """S <- diag(e^{gk}) S diag(e^{gv}) e^{g} + k^T v;  o = (q*scale) S.
    fla/ops/gla/naive.py:12-41 (gk only) generalised with the optional gates of
    fla/ops/common/fused_recurrent.py:98-124."""
    K, V = q.shape[-1], v.shape[-1]
    scale = K ** -0.5 if scale is None else scale

    def step(S, t, c):
        q_, k_, v_, gk_, gv_, g_ = c
        if gk_ is not None:
            S = S * gk_[:, :, t].exp()[..., None]
        if gv_ is not None:
            S = S * gv_[:, :, t].exp()[..., None, :]
        if g_ is not None:
            S = S * g_[:, :, t].exp()[..., None, None]
        S = S + k_[:, :, t, :, None] * v_[:, :, t, None, :]
        return S, ((q_[:, :, t] * scale)[..., None] * S).sum(-2)

    return _run(step, [q, k, v, gk, gv, g], initial_state, output_final_state, offsets, head_first, K, V, dtype, reverse)


def simple_gla(q, k, v, g, scale=None, initial_state=None, output_final_state=False, reverse=False, offsets=None,
               head_first=True, dtype=torch.float32):
    """Scalar log decay per token and head; fla/ops/simple_gla/naive.py:30-54."""
    return gla(q, k, v, g=g, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
               reverse=reverse, offsets=offsets, head_first=head_first, dtype=dtype)


def retention_log_decay(n_heads: int) -> torch.Tensor:
    """log(1 - 2^(-5-h)); fla/ops/retention/chunk.py:56."""
    return (1 - torch.tensor(2., dtype=torch.float).pow(-5. - torch.arange(n_heads, dtype=torch.float))).log()


def gated_delta_rule(q, k, v, beta, g=None, scale=None, initial_state=None, output_final_state=False, offsets=None,
                     head_first=True, dtype=torch.float32):
    """S <- e^{g} S;  v' = beta (v - S^T k);  S <- S + k v'^T;  o = S^T (q*scale).
    tests/ops/test_gated_delta.py:30-71 (reference test oracle); g=None gives the plain delta rule of
    fla/ops/delta_rule/naive.py:7-34.  beta is [B,T,H] or, for the recurrent op, [B,T,H,V]."""
    K, V = q.shape[-1], v.shape[-1]
    scale = K ** -0.5 if scale is None else scale

    def step(S, t, c):
        q_, k_, v_, b_, g_ = c
        if g_ is not None:
            S = S * g_[:, :, t].exp()[..., None, None]
        bt = b_[:, :, t]
        if bt.dim() == 2:
            bt = bt[..., None]
        vn = (v_[:, :, t] - (S * k_[:, :, t, :, None]).sum(-2)) * bt
        S = S + k_[:, :, t, :, None] * vn[:, :, None, :]
        return S, torch.einsum('bhk,bhkv->bhv', q_[:, :, t] * scale, S)

    return _run(step, [q, k, v, beta, g], initial_state, output_final_state, offsets, head_first, K, V, dtype)


def delta_rule(q, k, v, beta, **kw):
    """fla/ops/delta_rule/naive.py:7-34."""
    return gated_delta_rule(q, k, v, beta, g=None, **kw)


def _seq_bounds(T, offsets):
    if offsets is None:
        return [(0, T)]
    off = [int(o) for o in offsets.tolist()]
    return list(zip(off[:-1], off[1:]))


def cumsum_local(x, chunk_size=64, reverse=False, offsets=None, head_first=True):
    """Inclusive cumsum restarted every `chunk_size` tokens of every sequence, fp32;
    tests/ops/test_cumsum.py:24-31 restated."""
    if head_first:
        x = x.transpose(1, 2)
    x = x.float()
    y = torch.zeros_like(x)
    for a, b in _seq_bounds(x.shape[1], offsets):
        for c in range(a, b, chunk_size):
            e = min(c + chunk_size, b)
            seg = x[:, c:e]
            y[:, c:e] = seg.flip(1).cumsum(1).flip(1) if reverse else seg.cumsum(1)
    return y.transpose(1, 2) if head_first else y


def cumsum_global(x, reverse=False, offsets=None, head_first=True):
    """Inclusive cumsum over every whole sequence, fp32; tests/ops/test_cumsum.py:33-40 restated."""
    if head_first:
        x = x.transpose(1, 2)
    x = x.float()
    y = torch.zeros_like(x)
    for a, b in _seq_bounds(x.shape[1], offsets):
        seg = x[:, a:b]
        y[:, a:b] = seg.flip(1).cumsum(1).flip(1) if reverse else seg.cumsum(1)
    return y.transpose(1, 2) if head_first else y


def simple_gla_attention(q, k, g=None, scale=None, head_first=True, dtype=torch.float32):
    """A[b,h,i,j] = scale <q_i, k_j> exp(G_i - G_j) for j <= i, else 0, G = cumsum of g over the sequence: the attention
    matrix the reference's parallel form can return (fla/ops/simple_gla/parallel.py:95-131). Returns [B,H,T,T]."""
    if not head_first:
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        g = None if g is None else g.transpose(1, 2)
    q, k = q.to(dtype), k.to(dtype)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    A = torch.einsum("bhik,bhjk->bhij", q, k) * scale
    if g is not None:
        G = g.to(dtype).cumsum(-1)
        A = A * (G[..., :, None] - G[..., None, :]).clamp(max=0).exp()
    return A.tril()


def _chunk_bounds(T, chunk_size):
    return [(a, min(a + chunk_size, T)) for a in range(0, T, chunk_size)]


def chunk_states(k, v, gk_cumsum=None, gv_cumsum=None, initial_state=None, chunk_size=64, dtype=torch.float32):
    """State at the start of every chunk and the final state, for seq-first [B,T,H,*] inputs and chunk-local cumulative
    log gates per key channel (gk) and / or value channel (gv): fla/ops/common/chunk_h.py:83-133 restated
    (S <- diag(e^{gk_L}) S diag(e^{gv_L}) + (k e^{gk_L - gk})^T (v e^{gv_L - gv})). Returns (h [B,NT,H,K,V], ht)."""
    B, T, H, K = k.shape
    V = v.shape[-1]
    S = torch.zeros(B, H, K, V, dtype=dtype) if initial_state is None else initial_state.to(dtype).clone()
    hs = []
    for a, b in _chunk_bounds(T, chunk_size):
        hs.append(S.clone())
        kc, vc = k[:, a:b].to(dtype), v[:, a:b].to(dtype)
        if gk_cumsum is not None:
            gl = gk_cumsum[:, b - 1].to(dtype)
            S = S * gl.exp()[..., None]
            kc = kc * (gl[:, None] - gk_cumsum[:, a:b].to(dtype)).exp()
        if gv_cumsum is not None:
            gl = gv_cumsum[:, b - 1].to(dtype)
            S = S * gl.exp()[..., None, :]
            vc = vc * (gl[:, None] - gv_cumsum[:, a:b].to(dtype)).exp()
        S = S + torch.einsum("bthk,bthv->bhkv", kc, vc)
    return torch.stack(hs, 1), S


def chunk_state_gradients(q, do, scale, gk_cumsum=None, gv_cumsum=None, dht=None, chunk_size=64, dtype=torch.float32):
    """Reverse walk of the same recurrence: gradient of the state after every chunk and of the initial state
    (fla/ops/common/chunk_h.py:205-267). Returns (dh [B,NT,H,K,V], dh0)."""
    B, T, H, K = q.shape
    V = do.shape[-1]
    D = torch.zeros(B, H, K, V, dtype=dtype) if dht is None else dht.to(dtype).clone()
    dhs = []
    for a, b in reversed(_chunk_bounds(T, chunk_size)):
        dhs.append(D.clone())
        qc, dc = q[:, a:b].to(dtype) * scale, do[:, a:b].to(dtype)
        if gk_cumsum is not None:
            D = D * gk_cumsum[:, b - 1].to(dtype).exp()[..., None]
            qc = qc * gk_cumsum[:, a:b].to(dtype).exp()
        if gv_cumsum is not None:
            D = D * gv_cumsum[:, b - 1].to(dtype).exp()[..., None, :]
            dc = dc * gv_cumsum[:, a:b].to(dtype).exp()
        D = D + torch.einsum("bthk,bthv->bhkv", qc, dc)
    return torch.stack(dhs[::-1], 1), D
