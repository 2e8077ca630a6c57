# -*- coding: utf-8 -*-
"""Token-recurrent ops: the generic gated recurrence (fla/ops/common/fused_recurrent.py:545), the
delta rule (fla/ops/delta_rule/fused_recurrent.py:478) and the gated delta rule
(fla/ops/gated_delta_rule/fused_recurrent.py:210).  These are the decode kernels and the oracles the
reference's chunk tests compare against."""

from typing import Optional, Tuple

import torch

from .. import _lib
from .._lib import F_BETA_VECTOR, F_REVERSE
from ..utils import Geometry, autocast_custom_bwd, autocast_custom_fwd, contiguous
from .common import chunk_global_cumsum


def _f32(x):
    return None if x is None else x.float().contiguous()


def fused_recurrent_fwd(geo, q, k, v, g, gk, gv, scale, initial_state, output_final_state, reverse):
    o = torch.empty(v.shape, dtype=torch.float32, device=v.device)
    ht = torch.empty(geo.N, geo.H, geo.K, geo.V, dtype=torch.float32, device=v.device) if output_final_state else None
    _lib.call("flab_recurrent_fwd", q, **geo.kw(), scale=scale, flags=F_REVERSE if reverse else 0,
              q=q, k=k, v=v, g=_f32(g), gk=_f32(gk), gv=_f32(gv), h0=_f32(initial_state), o=o, ht=ht)
    return o, ht


def fused_recurrent_bwd(geo, q, k, v, g, gk, gv, o, do, dht, scale, initial_state, reverse):
    dq = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    dk = torch.empty(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.empty(v.shape, dtype=torch.float32, device=q.device)
    dh0 = torch.empty_like(initial_state, dtype=torch.float32) if initial_state is not None else None
    _lib.call("flab_recurrent_bwd", q, **geo.kw(), scale=scale, flags=F_REVERSE if reverse else 0,
              q=q, k=k, v=v, g=_f32(g), gk=_f32(gk), gv=_f32(gv), h0=_f32(initial_state), d_o=do.contiguous(),
              dht=_f32(dht), dq=dq, dk=dk, dv=dv, dh0=dh0)
    off, hf = geo.offsets_tensor, geo.head_first
    dg = dgk = dgv = None
    # gate gradients: reverse running sums of q*dq - k*dk (fla/ops/common/fused_recurrent.py:445-466)
    if g is not None:
        dg = chunk_global_cumsum((dq * q.float() - dk * k.float()).sum(-1), reverse=not reverse, offsets=off, head_first=hf)
    if gk is not None:
        dgk = chunk_global_cumsum(dq * q.float() - dk * k.float(), reverse=not reverse, offsets=off, head_first=hf)
    if gv is not None:
        dgv = chunk_global_cumsum(do.float() * o.float() - dv * v.float(), reverse=not reverse, offsets=off, head_first=hf)
    return dq, dk, dv, dg, dgk, dgv, dh0


class FusedRecurrentFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, g, gk, gv, scale, initial_state, output_final_state, reverse, offsets, head_first):
        geo = Geometry(k, v, offsets, head_first)
        o, ht = fused_recurrent_fwd(geo, q, k, v, g, gk, gv, scale, initial_state, output_final_state, reverse)
        ctx.save_for_backward(q, k, v, g, gk, gv, initial_state, o)
        ctx.geo, ctx.scale, ctx.reverse = geo, scale, reverse
        return o.to(q.dtype), ht

    @staticmethod
    @contiguous
    @autocast_custom_bwd
    def backward(ctx, do, dht):
        q, k, v, g, gk, gv, initial_state, o = ctx.saved_tensors
        if dht is not None and not dht.eq(0).all():
            for gate in (g, gk, gv):
                if gate is not None:
                    assert gate.requires_grad is False, \
                        "Cannot load final state gradient and use gates at the same time"
        dq, dk, dv, dg, dgk, dgv, dh0 = fused_recurrent_bwd(ctx.geo, q, k, v, g, gk, gv, o, do, dht, ctx.scale,
                                                             initial_state, ctx.reverse)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg, dgk, dgv, None, dh0, None, None, None, None


def fused_recurrent(q, k, v, g=None, gk=None, gv=None, scale=None, initial_state=None, output_final_state=False,
                    reverse=False, offsets=None, head_first=True):
    if scale is None:
        scale = k.shape[-1] ** -0.5
    return FusedRecurrentFunction.apply(q, k, v, g, gk, gv, scale, initial_state, output_final_state, reverse,
                                        offsets, head_first)


# ---------------------------------------------------------------------------------------------
# delta rule
# ---------------------------------------------------------------------------------------------
_CALLS = 0  # calls of recurrent_delta_fwd so far: every other call walks the state tiles in descending order


def recurrent_delta_fwd(geo, q, k, v, beta, g, scale, initial_state, output_final_state, want_u):
    """One launch of the token-recurrent (gated) delta rule. Successive calls alternate the order in which the kernel
    walks the (sequence, head) state tiles: in a decode loop the state a step reads is the one the previous step wrote,
    and the tiles that step wrote last are still in L2 when this one starts on them."""
    global _CALLS
    _CALLS += 1
    o = torch.empty_like(v)
    u = torch.empty_like(v) if want_u else None
    ht = torch.empty(geo.N, geo.H, geo.K, geo.V, dtype=torch.float32, device=v.device) if output_final_state else None
    flags = F_BETA_VECTOR if (beta is not None and beta.dim() == v.dim()) else 0
    if _CALLS & 1:
        flags |= _lib.F_DESCENDING
    _lib.call("flab_recurrent_delta_fwd", q, **geo.kw(), scale=scale, flags=flags, q=q, k=k, v=v,
              beta=None if beta is None else beta.to(q.dtype).contiguous(), g=_f32(g), h0=_f32(initial_state),
              o=o, u=u, ht=ht)
    return o, u, ht


class FusedRecurrentDeltaRuleFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    def forward(ctx, q, k, v, beta, scale, initial_state, output_final_state, offsets, head_first):
        geo = Geometry(k, v, offsets, head_first)
        o, u, ht = recurrent_delta_fwd(geo, q, k, v, beta, None, scale, initial_state, output_final_state, True)
        ctx.save_for_backward(q, k, u, beta, initial_state)
        ctx.geo, ctx.scale = geo, scale
        return o, ht

    @staticmethod
    @contiguous
    def backward(ctx, do, dht):
        q, k, u, beta, initial_state = ctx.saved_tensors
        geo = ctx.geo
        dq = torch.empty(q.shape, dtype=torch.float32, device=q.device)
        dk = torch.empty(k.shape, dtype=torch.float32, device=q.device)
        dv = torch.empty(u.shape, dtype=torch.float32, device=q.device)
        db = torch.empty(beta.shape, dtype=torch.float32, device=q.device)
        dh0 = torch.empty_like(initial_state, dtype=torch.float32) if initial_state is not None else None
        flags = F_BETA_VECTOR if beta.dim() == u.dim() else 0
        _lib.call("flab_recurrent_delta_bwd", q, **geo.kw(), scale=ctx.scale, flags=flags, q=q, k=k, v=u,
                  beta=beta.to(q.dtype).contiguous(), h0=_f32(initial_state), d_o=do, dht=_f32(dht),
                  dq=dq, dk=dk, dv=dv, dbeta=db, dh0=dh0)
        return dq.to(q), dk.to(k), dv.to(u), db.to(beta), None, dh0, None, None, None


class FusedRecurrentGatedDeltaRuleFunction(torch.autograd.Function):

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, offsets, head_first):
        geo = Geometry(k, v, offsets, head_first)
        o, _, ht = recurrent_delta_fwd(geo, q, k, v, beta, g, scale, initial_state, output_final_state, False)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        # same contract as fla/ops/gated_delta_rule/fused_recurrent.py:203-208
        raise NotImplementedError(
            "Backward pass is not implemented yet and we do not have plans to implement it "
            "because we haven't figured out how to compute dg without materializing the full "
            "hidden states for all time steps.")
