# -*- coding: utf-8 -*-
"""Stage-level launch wrappers: one Python function per C-ABI entry point, allocating outputs with
torch and passing raw pointers.  Names follow the reference's launch wrappers in
fla/ops/common/{chunk_h,chunk_o,chunk_delta_h}.py, fla/ops/utils/cumsum.py and the wy_fast modules."""

from typing import Optional, Tuple

import torch

from .. import _lib
from .._lib import CHUNK, F_REVERSE
from ..utils import Geometry, prepare_varlen


def _geo(x: torch.Tensor, offsets, head_first: bool) -> Geometry:
    """Geometry for a [B,T,H] / [B,T,H,S] tensor (cumsum entry points)."""
    if x.dim() == 3:
        k = x.unsqueeze(-1)
    else:
        k = x
    return Geometry(k, None, offsets, head_first)


def _cumsum(x, reverse, offsets, head_first, local, out_dtype=torch.float32):
    x = x.contiguous()
    if offsets is not None:
        assert x.shape[0] == 1, "Only batch size 1 is supported when offsets are provided"
    if x.dim() not in (3, 4):
        raise ValueError(f"Unsupported input shape {x.shape}; expected [B,T,H] / [B,T,H,D] "
                         f"(or the head-first permutations)")
    geo = _geo(x, offsets, head_first)
    y = torch.empty_like(x, dtype=torch.float32)
    S = x.shape[-1] if x.dim() == 4 else 0
    kind = "vector" if x.dim() == 4 else "scalar"
    entry = f"flab_chunk_{'local' if local else 'global'}_cumsum_{kind}"
    _lib.call(entry, x, B=geo.B, T=geo.T, H=geo.H, N=geo.N, NT=geo.NT, head_first=head_first,
              flags=F_REVERSE if reverse else 0, S=S, varlen=geo.varlen, dtype=x.dtype, x=x, y=y)
    return y if out_dtype in (None, torch.float32) else y.to(out_dtype)


def chunk_local_cumsum(g: torch.Tensor, chunk_size: int = CHUNK, reverse: bool = False,
                       offsets: Optional[torch.Tensor] = None, indices=None, head_first: bool = True) -> torch.Tensor:
    """Per-chunk inclusive cumulative sum, fp32 result (fla/ops/utils/cumsum.py:389)."""
    if chunk_size != CHUNK:
        raise ValueError(f"chunk_size is fixed at {CHUNK}")
    return _cumsum(g, reverse, offsets, head_first, True)


def chunk_global_cumsum(s: torch.Tensor, dtype: Optional[torch.dtype] = None, reverse: bool = False,
                        offsets: Optional[torch.Tensor] = None, head_first: bool = True) -> torch.Tensor:
    """Whole-sequence inclusive cumulative sum (fla/ops/utils/cumsum.py:369)."""
    return _cumsum(s, reverse, offsets, head_first, False, dtype or s.dtype)


def _state_buffers(geo: Geometry, ref: torch.Tensor, want_final: bool):
    h = torch.empty(geo.NT, geo.H, geo.K, geo.V, dtype=ref.dtype, device=ref.device)
    ht = torch.empty(geo.N, geo.H, geo.K, geo.V, dtype=torch.float32, device=ref.device) if want_final else None
    return h, ht


def _f32(x):
    return None if x is None else x.float().contiguous()


def chunk_fwd_h(geo: Geometry, k, v, g=None, gk=None, gv=None, h0=None, output_final_state=False):
    """State at the start of every chunk (fla/ops/common/chunk_h.py:282). Returns (h, ht). g, gk, gv are
    chunk-local cumulative log gates (fp32): per token, per key channel, per value channel (the path of the
    reference's GSA op, fla/ops/gsa/chunk.py:664-675)."""
    h, ht = _state_buffers(geo, k, output_final_state)
    _lib.call("flab_chunk_fwd_h", k, **geo.kw(), k=k, v=v, g=g, gk=gk, gv=gv, h0=_f32(h0), h=h, ht=ht)
    return h, ht


def chunk_bwd_dh(geo: Geometry, q, do, scale, g=None, gk=None, gv=None, dht=None, want_dh0=False):
    """Reverse state-gradient scan (fla/ops/common/chunk_h.py:338). Returns (dh, dh0)."""
    dh, dh0 = _state_buffers(geo, q, want_dh0)
    _lib.call("flab_chunk_bwd_dh", q, **geo.kw(), scale=scale, q=q, d_o=do, g=g, gk=gk, gv=gv, dht=_f32(dht), dh=dh, dh0=dh0)
    return dh, dh0


def chunk_fwd_o(geo: Geometry, q, k, v, h, g=None, scale=1.0):
    """Intra-chunk output (fla/ops/common/chunk_o.py:444)."""
    o = torch.empty_like(v)
    _lib.call("flab_chunk_fwd_o", q, **geo.kw(), scale=scale, q=q, k=k, v=v, h=h, g=g, o=o)
    return o


def chunk_bwd_dv(geo: Geometry, q, k, g, do, dh, scale):
    """dv including the inter-chunk term (fla/ops/common/chunk_o.py:499)."""
    dv = torch.empty_like(do)
    _lib.call("flab_chunk_bwd_dv", q, **geo.kw(), scale=scale, q=q, k=k, g=g, d_o=do, dh=dh, dv=dv)
    return dv


def chunk_bwd_dv_local(geo: Geometry, q, k, g, do, scale):
    """Intra-chunk part of dv (fla/ops/common/chunk_o.py:551)."""
    dv = torch.empty_like(do)
    _lib.call("flab_chunk_bwd_dv_local", q, **geo.kw(), scale=scale, q=q, k=k, g=g, d_o=do, dv=dv)
    return dv


def chunk_bwd_dqkwg(geo: Geometry, q, k, v, h, dh, do, scale, g=None, w=None, dv=None):
    """dq, dk, dw, dg (fla/ops/common/chunk_o.py:602). dg is w.r.t. the cumsummed gate, fp32."""
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dw = torch.empty_like(w) if w is not None else None
    dg = torch.empty(g.shape, dtype=torch.float32, device=g.device) if g is not None else None
    _lib.call("flab_chunk_bwd_dqkwg", q, **geo.kw(), scale=scale, q=q, k=k, v=v, h=h, dh=dh, d_o=do, g=g, w=w,
              dv=dv, dq=dq, dk=dk, dw=dw, dg=dg)
    return dq, dk, dw, dg


def fwd_prepare_wy_repr(geo: Geometry, k, v, beta, g=None):
    """WY factors of the (gated) delta rule (fla/ops/delta_rule/wy_fast.py:436,
    fla/ops/gated_delta_rule/wy_fast.py:320). Returns (aw, au, w, u); au is None without gates."""
    shape_a = (*beta.shape, CHUNK)
    aw = torch.empty(shape_a, dtype=k.dtype, device=k.device)
    au = torch.empty(shape_a, dtype=k.dtype, device=k.device) if g is not None else None
    w, u = torch.empty_like(k), torch.empty_like(v)
    _lib.call("flab_wy_fwd", k, **geo.kw(), k=k, v=v, beta=beta, g=g, aw=aw, au=au, w=w, u=u)
    return aw, au, w, u


def fwd_recompute_w_u(geo: Geometry, k, v, beta, aw, au=None):
    """w, u from stored inverse factors (fla/ops/delta_rule/wy_fast.py:532)."""
    w, u = torch.empty_like(k), torch.empty_like(v)
    _lib.call("flab_wy_recompute", k, **geo.kw(), k=k, v=v, beta=beta, aw=aw, au=au, w=w, u=u)
    return w, u


def bwd_prepare_wy_repr(geo: Geometry, k, v, beta, aw, dw, du, g=None, au=None, dk_in=None, dg_in=None):
    """Backward of the WY transform (fla/ops/delta_rule/wy_fast.py:619,
    fla/ops/gated_delta_rule/wy_fast.py:565). Returns (dk, dv, dbeta, dg). `dk_in` (optional, same dtype as
    k) is added to the returned dk inside the kernel, in fp32, before the single rounding. `dg_in` (optional, gated:
    the fp32 dg of chunk_bwd_dqkwg): the returned dg is then the finished gradient of the raw gate, the reverse
    chunk-local cumsum of (dg_in + this stage's dg), formed inside the same kernel."""
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    dbeta = torch.empty(beta.shape, dtype=torch.float32, device=k.device)
    dg = torch.empty(beta.shape, dtype=torch.float32, device=k.device) if g is not None else None
    _lib.call("flab_wy_bwd", k, **geo.kw(), k=k, v=v, beta=beta, g=g, aw=aw, au=au, dw=dw, du=du, dk=dk, dv=dv,
              dbeta=dbeta, dg=dg, x=dk_in, dgk=dg_in if g is not None else None)
    return dk, dv, dbeta, dg


def chunk_gated_delta_rule_fwd_h(geo: Geometry, k, w, u, g=None, h0=None, output_final_state=False):
    """Delta-rule state scan (fla/ops/common/chunk_delta_h.py:248). Returns (h, v_new, ht)."""
    h, ht = _state_buffers(geo, k, output_final_state)
    v_new = torch.empty_like(u)
    _lib.call("flab_delta_fwd_h", k, **geo.kw(), k=k, w=w, u=u, g=g, h0=_f32(h0), h=h, v_new=v_new, ht=ht)
    return h, v_new, ht


def chunk_gated_delta_rule_bwd_dhu(geo: Geometry, q, k, w, do, dv, scale, g=None, dht=None, want_dh0=False):
    """Reverse delta-rule scan (fla/ops/common/chunk_delta_h.py:323). Returns (dh, dh0, dv2)."""
    dh, dh0 = _state_buffers(geo, q, want_dh0)
    dv2 = torch.empty_like(dv)
    _lib.call("flab_delta_bwd_dhu", q, **geo.kw(), scale=scale, q=q, k=k, w=w, g=g, dht=_f32(dht), d_o=do, dv=dv,
              dh=dh, dh0=dh0, dv2=dv2)
    return dh, dh0, dv2


# ---------------------------------------------------------------------------------------------
# Delta-rule scans of a FEW LONG sequences, split into slabs along T on one GPU
# ---------------------------------------------------------------------------------------------
# The scan is a serial chain per (sequence, head, 128 value columns); with one 2^20-token sequence and 16 heads that is
# 16 CTAs on 148 SMs.  The chain is affine in the state, S_out = M S_in + b per slab, so the sequence is cut into S
# slabs that are scanned as S independent sequences, twice: a first pass from the initial state [0 | I] over the
# value columns [u | 0] yields every slab's (b, M) at once, the slabs' true initial states follow from S - 1 small
# matrix products, and the second pass starts every slab from its true state.  The backward scan is the transposed
# chain (dS_in = M^T dS_out + c): its first pass runs from zero to get c, M is kept from the forward.  This is the
# single-GPU form of the hand-off in fla_b200.parallel (there a slab per rank, here a slab per group of SMs).
SLAB_MIN_CHUNKS = 256        # chunks per sequence below which the split is not tried
SLAB_MIN_CHUNKS_PER_SLAB = 64
_SLAB_VARLEN = {}


class SlabPlan:
    """How the sequences of one call are cut: `S` slabs per sequence, `lengths` of all B * S slabs in order."""

    def __init__(self, B, T, S, chunks_per_slab, device):
        self.B, self.T, self.S = B, T, S
        L = chunks_per_slab * CHUNK
        per_seq = [min(L, T - i * L) for i in range(S)]
        key = (B, T, S, chunks_per_slab, str(device))
        if key not in _SLAB_VARLEN:
            if len(_SLAB_VARLEN) > 16:
                _SLAB_VARLEN.clear()
            from ..utils import varlen_from_lengths
            _SLAB_VARLEN[key] = varlen_from_lengths(per_seq * B, device)
        self.varlen = _SLAB_VARLEN[key]

    def geometry(self, k, v):
        """Packed geometry of the slabs over `[B, T, H, D]` tensors viewed as `[1, B * T, H, D]`."""
        return Geometry.packed(k.view(1, -1, *k.shape[2:]), v.view(1, -1, *v.shape[2:]), self.varlen)


def slab_plan(geo: Geometry, k: torch.Tensor) -> Optional[SlabPlan]:
    """A plan when the call is a few long fixed-length sequences in the domain of the tensor-core scan, else None."""
    import os
    if os.environ.get("FLA_B200_NO_SLABS") or os.environ.get("FLA_B200_NO_TC"):
        return None
    if geo.varlen is not None or geo.head_first or k.dtype not in (torch.bfloat16, torch.float16):
        return None
    if geo.K != 128 or geo.V % 128 != 0:
        return None
    nts = -(-geo.T // CHUNK)
    chains = geo.B * geo.H * (geo.V // 128)
    sms = torch.cuda.get_device_properties(k.device).multi_processor_count
    S = min(sms // chains, nts // SLAB_MIN_CHUNKS_PER_SLAB, 16)
    if nts < SLAB_MIN_CHUNKS or S < 2:
        return None
    per = -(-nts // S)
    return SlabPlan(geo.B, geo.T, -(-nts // per), per, k.device)


def slab_delta_fwd_pass1(plan: SlabPlan, geo: Geometry, k, w, u, g=None):
    """First pass of the forward scan over slabs: every slab's transition. Returns `bm` `[B, S, H, K, V + K]` fp32, the
    final state of each slab started from `[0 | I]` over the value columns `[u | 0]`: columns `[:V]` are the slab's
    offset b, columns `[V:]` its matrix M (S_out = M S_in + b)."""
    from .._lib import F_STATE_ONLY
    B, S, H, K, V = plan.B, plan.S, geo.H, geo.K, geo.V
    dev = k.device
    gv = None if g is None else g.view(1, -1, H)
    h0_ext = torch.zeros(B * S, H, K, V + K, dtype=torch.float32, device=dev)
    h0_ext[..., V:] = torch.eye(K, dtype=torch.float32, device=dev)
    ht_ext = torch.empty_like(h0_ext)
    ge = plan.geometry(k, u)
    ge.V = V + K  # the state is V + K columns wide; u supplies the first V (S = V), the rest read as zero
    _lib.call("flab_delta_fwd_h", k, **ge.kw(), flags=F_STATE_ONLY, S=V, k=k, w=w, u=u, g=gv, h0=h0_ext, ht=ht_ext)
    return ht_ext.view(B, S, H, K, V + K)


def slab_delta_fwd_pass2(plan: SlabPlan, geo: Geometry, bm, k, w, u, g=None, h0=None, output_final_state=False):
    """Second pass: the slabs' true initial states from the chain S <- M_s S + b_s (one launch), then the scan proper.
    Returns (h, v_new, ht, M) with M `[B, S, H, K, K]` fp32 kept for the backward scan."""
    B, S, H, K, V = plan.B, plan.S, geo.H, geo.K, geo.V
    dev = k.device
    gv = None if g is None else g.view(1, -1, H)
    b_, M = bm[..., :V], bm[..., V:].contiguous()
    S_in, _ = _lib.state_chain(M, b_, h0)
    gs = plan.geometry(k, u)
    h = torch.empty(geo.NT, H, K, V, dtype=k.dtype, device=dev)
    v_new = torch.empty_like(u)
    ht_s = torch.empty(B * S, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    _lib.call("flab_delta_fwd_h", k, **gs.kw(), k=k, w=w, u=u, g=gv, h0=S_in.view(B * S, H, K, V), h=h, v_new=v_new, ht=ht_s)
    ht = ht_s.view(B, S, H, K, V)[:, -1].contiguous() if output_final_state else None
    return h, v_new, ht, M


def slab_delta_fwd_h(plan: SlabPlan, geo: Geometry, k, w, u, g=None, h0=None, output_final_state=False):
    """`chunk_gated_delta_rule_fwd_h` over slabs. Returns (h, v_new, ht, M) with M `[B, S, H, K, K]` fp32, the slabs'
    state transitions (kept for the backward scan)."""
    bm = slab_delta_fwd_pass1(plan, geo, k, w, u, g=g)
    return slab_delta_fwd_pass2(plan, geo, bm, k, w, u, g=g, h0=h0, output_final_state=output_final_state)


def slab_total_transition(bm: torch.Tensor, V: int):
    """The transition of the WHOLE sequence from those of its slabs: the chain started from `[0 | I]`. bm: `[B, S, H, K,
    V + K]` from `slab_delta_fwd_pass1`. Returns (b `[B, H, K, V]`, M `[B, H, K, K]`)."""
    B, S, H, K, W = bm.shape
    ext0 = torch.zeros(B, H, K, W, dtype=torch.float32, device=bm.device)
    ext0[..., V:] = torch.eye(K, dtype=torch.float32, device=bm.device)
    _, tot = _lib.state_chain(bm[..., V:].contiguous(), bm, ext0, want_s_in=False, want_last=True)
    return tot[..., :V].contiguous(), tot[..., V:].contiguous()


def slab_delta_bwd_pass1(plan: SlabPlan, geo: Geometry, q, k, w, do, dv, scale, g=None):
    """First pass of the reverse scan over slabs: c `[B, S, H, K, V]` fp32, the state gradient every slab hands to its
    predecessor when it receives zero."""
    from .._lib import F_STATE_ONLY
    B, S, H, K, V = plan.B, plan.S, geo.H, geo.K, geo.V
    gv = None if g is None else g.view(1, -1, H)
    gs = plan.geometry(k, dv)
    c_ = torch.empty(B * S, H, K, V, dtype=torch.float32, device=q.device)
    _lib.call("flab_delta_bwd_dhu", q, **gs.kw(), scale=scale, flags=F_STATE_ONLY, q=q, k=k, w=w, g=gv, d_o=do, dv=dv, dh0=c_)
    return c_.view(B, S, H, K, V)


def slab_delta_bwd_dhu(plan: SlabPlan, geo: Geometry, M, q, k, w, do, dv, scale, g=None, dht=None, want_dh0=False, c_=None):
    """`chunk_gated_delta_rule_bwd_dhu` over slabs, with the transitions M of the forward (`c_`: the result of
    `slab_delta_bwd_pass1` when the caller already has it). Returns (dh, dh0, dv2)."""
    B, S, H, K, V = plan.B, plan.S, geo.H, geo.K, geo.V
    dev = q.device
    gv = None if g is None else g.view(1, -1, H)
    gs = plan.geometry(k, dv)
    if c_ is None:
        c_ = slab_delta_bwd_pass1(plan, geo, q, k, w, do, dv, scale, g=g)
    # the transposed chain, right to left: D_out[s] = gradient of the state leaving slab s
    D_out, _ = _lib.state_chain(M, c_, dht, reverse=True, transpose=True)
    # pass 2
    dh = torch.empty(geo.NT, H, K, V, dtype=q.dtype, device=dev)
    dv2 = torch.empty_like(dv)
    dh0_s = torch.empty(B * S, H, K, V, dtype=torch.float32, device=dev) if want_dh0 else None
    _lib.call("flab_delta_bwd_dhu", q, **gs.kw(), scale=scale, q=q, k=k, w=w, g=gv, dht=D_out.view(B * S, H, K, V), d_o=do, dv=dv,
              dh=dh, dh0=dh0_s, dv2=dv2)
    dh0 = dh0_s.view(B, S, H, K, V)[:, 0].contiguous() if want_dh0 else None
    return dh, dh0, dv2


__all__ = [n for n in dir() if n.startswith(("chunk_", "fwd_", "bwd_", "slab_"))] + ["prepare_varlen", "Geometry"]
