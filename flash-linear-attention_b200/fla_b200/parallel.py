# -*- coding: utf-8 -*-
"""Multi-GPU use of the path (one process per GPU, torch.distributed).

* Units of work are (sequence, head) pairs with no data flow between them, so batches shard with no
  collective at all: `shard_batch_heads` (fixed length) and `shard_sequences` (packed variable length,
  token-balanced) only plan who owns what.
* One very long sequence is split along T ("sequence parallel"): every recurrence on this path is affine in
  the state, S_out = M S_in + b with M a [K,K] matrix per head that does not depend on S_in.  A rank
  obtains (M, b) of its slab from ONE extra state scan whose value dimension is widened by K identity
  columns, the boundary states are then passed rank to rank (point-to-point send/recv, [H,K,V] fp32 = 1 MiB
  at H=16, K=V=128), and a local correction pass recomputes the slab with its true initial state.
  Backward uses the same structure with the transposed transition: the gradient of a slab's initial state is
  dS_in = M^T dS_out + c, where c is what the slab's own outputs contribute (a reverse scan with dS_out = 0);
  the chain runs from the last rank to the first, then every rank runs its full backward with the true dS_out.
  The reference has no such mode; its unused two-level scan (fla/ops/common/chunk_h_split.py:164-260) only
  covers diagonal decay.
"""

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------------------------
# optional stage timing (CUDA events on the current stream), used by the benchmark
# ---------------------------------------------------------------------------------------------
STAGE_EVENTS = None  # set to {} to record (start, end) event pairs per stage name; None = off (the default)


class _stage:
    """`with _stage("name"):` brackets a stage with CUDA events when STAGE_EVENTS is a dict; free otherwise."""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if STAGE_EVENTS is not None and torch.cuda.is_available():
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.a.record()

    def __exit__(self, *exc):
        if STAGE_EVENTS is not None and torch.cuda.is_available():
            self.b.record()
            STAGE_EVENTS.setdefault(self.name, []).append((self.a, self.b))


def stage_times_ms():
    """Total milliseconds per recorded stage (synchronises); clears the record."""
    torch.cuda.synchronize()
    out = {n: sum(a.elapsed_time(b) for a, b in evs) for n, evs in (STAGE_EVENTS or {}).items()}
    if STAGE_EVENTS is not None:
        STAGE_EVENTS.clear()
    return out


# ---------------------------------------------------------------------------------------------
# planners (pure host logic)
# ---------------------------------------------------------------------------------------------
def shard_batch_heads(B: int, H: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Slices of the batch and head axes owned by `rank`: the batch is split first, heads only when there are
    more ranks than batch rows. Every (row, head) pair is owned by exactly one rank."""
    if world <= B:
        lo, hi = (B * rank) // world, (B * (rank + 1)) // world
        return slice(lo, hi), slice(0, H)
    if world % B != 0 or H % (world // B) != 0:
        raise ValueError(f"cannot split B={B}, H={H} evenly over {world} ranks")
    per_row = world // B
    b, part = rank // per_row, rank % per_row
    hs = H // per_row
    return slice(b, b + 1), slice(part * hs, (part + 1) * hs)


def shard_sequences(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Token-balanced partition of whole sequences (longest-processing-time greedy). Returns, per rank, the
    ids of its sequences in ascending order."""
    order = sorted(range(len(lengths)), key=lambda i: -int(lengths[i]))
    load = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        owned[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(o) for o in owned]


def rebased_offsets(lengths: Sequence[int], ids: Sequence[int]) -> torch.Tensor:
    """`offsets` ([len(ids)+1], int64) of the packed batch made of the sequences `ids`."""
    out = [0]
    for i in ids:
        out.append(out[-1] + int(lengths[i]))
    return torch.tensor(out, dtype=torch.long)


def gather_packed(x: torch.Tensor, offsets: Sequence[int], ids: Sequence[int]) -> torch.Tensor:
    """Rows of the packed tensor x [1, T, ...] that belong to the sequences `ids`, re-packed."""
    return torch.cat([x[:, int(offsets[i]):int(offsets[i + 1])] for i in ids], dim=1)


# ---------------------------------------------------------------------------------------------
# sequence parallel state hand-off
# ---------------------------------------------------------------------------------------------
def handoff_states(M: torch.Tensor, b: torch.Tensor, S0: Optional[torch.Tensor], group=None,
                   reverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chain S_out = M S_in + b across the ranks of `group`.

    M: [H,K,K], b: [H,K,V] fp32 of THIS rank's slab. The chain starts at rank 0 (at the last rank when
    `reverse`) with S0 (zeros when None). Returns (S_in, S_out) of this rank. One blocking recv and one send per
    rank; on GPUs this is NCCL point-to-point over NVLink.
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    first, step = (world - 1, -1) if reverse else (0, 1)
    prev, nxt = rank - step, rank + step

    def _finish(work, what, peer):
        # A peer that has left, or a link error, surfaces here: on the host, as an exception that names the hop, after the
        # process group's timeout at the latest, and before any kernel of this rank has consumed the buffer.
        try:
            work.wait()
        except Exception as e:  # noqa: BLE001 - whatever the backend raises
            raise RuntimeError(f"sequence-parallel state hand-off: {what} rank {peer} failed on rank {rank}: {e}") from e

    if rank == first:
        S_in = torch.zeros_like(b) if S0 is None else S0.to(b.dtype).reshape(b.shape).contiguous()
    else:
        S_in = torch.empty_like(b)
        src = dist.get_global_rank(group, prev) if group is not None else prev
        _finish(dist.irecv(S_in, src=src, group=group), "receive from", prev)
    if b.is_cuda:
        from . import _lib  # one launch of the library's own chain kernel (fp32 FFMA), no library GEMM on this path
        H, K, V = b.shape
        _, S_out = _lib.state_chain(M.contiguous().view(1, 1, H, K, K), b.contiguous().view(1, 1, H, K, V), S_in.view(1, H, K, V),
                                    want_s_in=False, want_last=True)
        S_out = S_out.view(H, K, V)
    else:  # CPU tensors occur only in the gloo tests of this host logic
        S_out = torch.baddbmm(b, M, S_in)
    if 0 <= nxt < world:
        dst = dist.get_global_rank(group, nxt) if group is not None else nxt
        _finish(dist.isend(S_out, dst=dst, group=group), "send to", nxt)
    return S_in, S_out


def broadcast_from(x: torch.Tensor, src_rank: int, group=None) -> torch.Tensor:
    dist.broadcast(x, src=dist.get_global_rank(group, src_rank) if group is not None else src_rank, group=group)
    return x


def _fwd_slab(q, k, v, g, beta, scale, S_in_of):
    """Forward of one rank's slab. `S_in_of(M, b)` maps the slab's transition to its true initial state (this is
    where the communication happens). Returns (o, S_out, saved tensors for backward).

    A rank's slab is itself a few long chains, so when it is long enough its two scans run split into sub-slabs over the
    SMs (`ops.common.slab_*`): the first pass gives every sub-slab's transition, their composition (one launch of the
    chain kernel) is the rank's (M, b), and the second pass starts from the state received from the previous rank."""
    from .ops import common as C
    from .utils import Geometry
    geo = Geometry(k, v, None, False)
    H, K, V = geo.H, geo.K, geo.V
    g_cum = C.chunk_local_cumsum(g, head_first=False)
    aw, au, w, u = C.fwd_prepare_wy_repr(geo, k, v, beta, g=g_cum)
    import os
    plan = C.slab_plan(geo, k)
    timer = _stage("state_pass_fwd")
    timer.__enter__()
    bm = None
    if plan is not None:
        bm = C.slab_delta_fwd_pass1(plan, geo, k, w, u, g=g_cum)
        b, M = C.slab_total_transition(bm, V)
        b, M = b[0], M[0]
    else:
        # one widened scan: value columns [u | 0], initial state [0 | I]  ->  final state [b | M]
        h0_ext = torch.cat([torch.zeros(1, H, K, V, device=k.device), torch.eye(K, device=k.device).expand(1, H, K, K)], dim=-1).contiguous()
        if k.dtype in (torch.bfloat16, torch.float16) and K == 128 and V % 64 == 0 and not os.environ.get("FLA_B200_NO_TC"):
            # state-only scan: nothing but the final state is stored, u itself is read (columns past V are zero-filled)
            from . import _lib
            geo_ext = Geometry(k, u, None, False)
            geo_ext.V = V + K
            ht_ext = torch.empty_like(h0_ext)
            _lib.call("flab_delta_fwd_h", k, **geo_ext.kw(), flags=_lib.F_STATE_ONLY, S=V, k=k, w=w, u=u, g=g_cum, h0=h0_ext, ht=ht_ext)
        else:
            u_ext = torch.cat([u, torch.zeros_like(k)], dim=-1)
            geo_ext = Geometry(k, u_ext, None, False)
            _, _, ht_ext = C.chunk_gated_delta_rule_fwd_h(geo_ext, k, w, u_ext, g=g_cum, h0=h0_ext, output_final_state=True)
        b, M = ht_ext[0, :, :, :V].contiguous(), ht_ext[0, :, :, V:].contiguous()
    timer.__exit__()
    with _stage("handoff_fwd"):
        S_in, S_out = S_in_of(M, b)
    # correction pass with the true initial state
    M_sub = None
    if plan is not None:
        h, v_new, _, M_sub = C.slab_delta_fwd_pass2(plan, geo, bm, k, w, u, g=g_cum, h0=S_in.unsqueeze(0), output_final_state=False)
    else:
        h, v_new, _ = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=g_cum, h0=S_in.unsqueeze(0), output_final_state=False)
    o = C.chunk_fwd_o(geo, q, k, v_new, h, g=g_cum, scale=scale)
    return o, S_out, (g_cum, aw, au, w, h, v_new, geo, M, S_in, M_sub)


def sp_chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, group=None):
    """Forward of chunk_gated_delta_rule for ONE sequence split along T over the ranks of `group`.

    Every rank passes its own contiguous slab (seq-first, B = 1, slab length a multiple of 64 except on the last
    rank); rank r's slab follows rank r-1's. `initial_state` ([1,H,K,V]) is read on rank 0. Returns (o of the
    slab, final state of the whole sequence on every rank or None). Forward only.
    """
    assert q.shape[0] == 1, "sequence parallel mode takes one sequence (B = 1) per call"
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    assert rank == world - 1 or q.shape[1] % 64 == 0, "slabs before the last one must be multiples of 64 tokens"
    scale = k.shape[-1] ** -0.5 if scale is None else scale
    q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
    S0 = None if initial_state is None else initial_state.float()[0]
    o, S_out, _ = _fwd_slab(q, k, v, g.float(), beta.to(k.dtype), scale, lambda M, b: handoff_states(M, b, S0, group))
    ht = None
    if output_final_state:
        ht = broadcast_from(S_out.clone(), world - 1, group).unsqueeze(0)
    return o, ht


class SPChunkGatedDeltaRuleFunction(torch.autograd.Function):
    """chunk_gated_delta_rule on one T-slab per rank, differentiable. Collective calls happen inside forward and
    backward, so every rank of `group` must run both, in the same order."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, group):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
        beta_k = beta.to(k.dtype)
        S0 = None if initial_state is None else initial_state.float()[0]
        o, S_out, saved = _fwd_slab(q, k, v, g.float(), beta_k, scale, lambda M, b: handoff_states(M, b, S0, group))
        g_cum, aw, au, w, h, v_new, geo, M, S_in, M_sub = saved
        ht = broadcast_from(S_out.clone(), world - 1, group).unsqueeze(0) if output_final_state else None
        ctx.save_for_backward(q, k, v, g_cum, beta_k, aw, au, w, h, v_new, M, S_in, M_sub)
        ctx.geo, ctx.scale, ctx.group, ctx.g_dtype, ctx.beta_dtype = geo, scale, group, g.dtype, beta.dtype
        ctx.has_h0 = initial_state is not None
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        from .ops import common as C
        from .ops.gated_delta_rule import chunk_gated_delta_rule_bwd
        q, k, v, g_cum, beta, aw, au, w, h, v_new, M, S_in, M_sub = ctx.saved_tensors
        geo, scale, group = ctx.geo, ctx.scale, ctx.group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        do = do.contiguous()
        # what this slab's outputs alone contribute to the gradient of its initial state (dS_out = 0)
        dv = C.chunk_bwd_dv_local(geo, q, k, g_cum, do, scale)
        import os
        timer = _stage("state_pass_bwd")
        timer.__enter__()
        plan = C.slab_plan(geo, k) if M_sub is not None else None
        slab_c = None
        if plan is not None:
            # split reverse scan: every sub-slab's contribution, composed right to left from zero (one launch)
            from . import _lib
            slab_c = C.slab_delta_bwd_pass1(plan, geo, q, k, w, do, dv, scale, g=g_cum)
            _, c = _lib.state_chain(M_sub, slab_c, None, want_s_in=False, want_last=True, reverse=True, transpose=True)
        elif k.dtype in (torch.bfloat16, torch.float16) and geo.K == 128 and geo.V % 64 == 0 and not os.environ.get("FLA_B200_NO_TC"):
            from . import _lib  # state-only scan: only the gradient handed to the predecessor is stored
            c = torch.empty(1, geo.H, geo.K, geo.V, dtype=torch.float32, device=k.device)
            _lib.call("flab_delta_bwd_dhu", q, **geo.kw(), scale=scale, flags=_lib.F_STATE_ONLY, q=q, k=k, w=w, g=g_cum, d_o=do, dv=dv, dh0=c)
        else:
            _, c, _ = C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, g=g_cum, dht=None, want_dh0=True)
        # the gradient of the whole-sequence final state enters at the last rank
        timer.__exit__()
        ext = None if dht is None or rank != world - 1 else dht.float()[0]
        with _stage("handoff_bwd"):
            dS_out, dS_in = handoff_states(M.transpose(1, 2).contiguous(), c[0], ext, group, reverse=True)
        dq, dk, dv, db, dg, _ = chunk_gated_delta_rule_bwd(geo, q, k, v, g_cum, beta, aw, au, scale, S_in.unsqueeze(0), do,
                                                          dS_out.unsqueeze(0), saved=(w, h, v_new, M_sub), dv_local=dv, slab_c=slab_c)
        dh0 = dS_in.unsqueeze(0) if (ctx.has_h0 and rank == 0) else None
        if ctx.has_h0 and rank != 0:
            dh0 = torch.zeros_like(dS_in).unsqueeze(0)
        return dq, dk, dv, dg.to(ctx.g_dtype), db.to(ctx.beta_dtype), None, dh0, None, None


def sp_chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, group=None):
    """Differentiable chunk_gated_delta_rule for ONE sequence split along T over the ranks of `group` (same slab
    rules as `sp_chunk_gated_delta_rule_fwd`). `initial_state` and its gradient live on rank 0; a gradient of the
    returned final state is taken from the LAST rank only (the state is that rank's, broadcast to the others)."""
    assert q.shape[0] == 1, "sequence parallel mode takes one sequence (B = 1) per call"
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    assert rank == world - 1 or q.shape[1] % 64 == 0, "slabs before the last one must be multiples of 64 tokens"
    scale = k.shape[-1] ** -0.5 if scale is None else scale
    return SPChunkGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state, group)
