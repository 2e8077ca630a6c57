"""CPU (gloo, world_size > 1): the host logic of the multi-GPU paths - shard planners and the sequence-parallel
state hand-off - with the oracle standing in for the kernels."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from fla_b200.parallel import (gather_packed, handoff_states, rebased_offsets, shard_batch_heads, shard_sequences)


def test_shard_batch_heads_covers_every_pair_once():
    for B, H, world in ((8, 16, 1), (8, 16, 2), (8, 16, 4), (8, 16, 8), (2, 16, 8), (1, 32, 8)):
        seen = torch.zeros(B, H, dtype=torch.int32)
        for r in range(world):
            bs, hs = shard_batch_heads(B, H, world, r)
            seen[bs, hs] += 1
        assert torch.all(seen == 1)
    with pytest.raises(ValueError):
        shard_batch_heads(3, 5, 8, 0)


def test_shard_sequences_is_a_balanced_partition():
    g0 = torch.Generator().manual_seed(0)
    lengths = torch.randint(256, 8193, (64,), generator=g0).tolist()
    for world in (1, 2, 4, 8):
        owned = shard_sequences(lengths, world)
        assert sorted(i for o in owned for i in o) == list(range(64))
        loads = [sum(lengths[i] for i in o) for o in owned]
        assert max(loads) - min(loads) <= max(lengths)  # LPT bound
        off = rebased_offsets(lengths, owned[0])
        assert off[0] == 0 and off[-1] == loads[0] and len(off) == len(owned[0]) + 1


def test_gather_packed_roundtrip():
    lengths = [3, 5, 2, 7]
    offsets = [0, 3, 8, 10, 17]
    x = torch.arange(17).view(1, 17, 1)
    y = gather_packed(x, offsets, [1, 3])
    assert y.flatten().tolist() == list(range(3, 8)) + list(range(10, 17))


def _worker(rank, world, port, reverse, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(1234)  # same stream on every rank: every rank can rebuild everyone's (M, b)
        H, K, V = 2, 8, 6
        Ms = torch.randn(world, H, K, K) * 0.3
        bs = torch.randn(world, H, K, V)
        S0 = torch.randn(H, K, V)
        S_in, S_out = handoff_states(Ms[rank], bs[rank], S0, reverse=reverse)
        order = list(range(world - 1, -1, -1)) if reverse else list(range(world))
        S = S0
        for r in order:
            if r == rank:
                torch.testing.assert_close(S_in, S)
            S = bs[r] + Ms[r] @ S
            if r == rank:
                torch.testing.assert_close(S_out, S)
        ret[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,reverse", [(2, False), (3, False), (3, True)])
def test_handoff_states_gloo(world, reverse):
    port = 29600 + world * 2 + int(reverse)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, reverse, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def _sp_worker(rank, world, port, ret):
    """Sequence-parallel gated delta rule with the ORACLE as the local scan: checks that chaining (M, b) pairs
    obtained from identity-widened scans reproduces the one-shot recurrence."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g0 = torch.Generator().manual_seed(5)
        T, H, K, V = 64 * world, 2, 8, 8
        q, k = torch.randn(1, T, H, K, generator=g0), torch.nn.functional.normalize(torch.randn(1, T, H, K, generator=g0), dim=-1)
        v, beta = torch.randn(1, T, H, V, generator=g0), torch.rand(1, T, H, generator=g0)
        g = -torch.rand(1, T, H, generator=g0)
        S0 = torch.randn(1, H, K, V, generator=g0) * 0.1
        o_ref, ht_ref = oracle.gated_delta_rule(q, k, v, beta, g=g, initial_state=S0, output_final_state=True, head_first=False)
        sl = slice(64 * rank, 64 * (rank + 1))
        # local (M, b): run the recurrence on [v | 0] with initial state [0 | I]
        v_ext = torch.cat([v[:, sl], torch.zeros(1, 64, H, K)], -1)
        h0_ext = torch.cat([torch.zeros(1, H, K, V), torch.eye(K).expand(1, H, K, K)], -1)
        _, ht_ext = oracle.gated_delta_rule(q[:, sl], k[:, sl], v_ext, beta[:, sl], g=g[:, sl], initial_state=h0_ext,
                                            output_final_state=True, head_first=False)
        b, M = ht_ext[0, :, :, :V].contiguous(), ht_ext[0, :, :, V:].contiguous()
        S_in, S_out = handoff_states(M, b, S0[0])
        o, _ = oracle.gated_delta_rule(q[:, sl], k[:, sl], v[:, sl], beta[:, sl], g=g[:, sl], initial_state=S_in[None],
                                       output_final_state=True, head_first=False)
        torch.testing.assert_close(o, o_ref[:, sl], rtol=1e-4, atol=1e-4)
        if rank == world - 1:
            torch.testing.assert_close(S_out[None], ht_ref, rtol=1e-4, atol=1e-4)
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_chain_reproduces_one_shot_gloo():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_sp_worker, args=(world, 29650, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def _worker_missing_peer(rank, world, port, ret):
    """Rank 0 never takes part in the hand-off (it leaves between steps, nothing of its own in flight); rank 1, which
    waits for rank 0's state, must get an exception that names the hop within the process group's timeout."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 0:
            ret[rank] = "left"
            return
        H, K, V = 1, 4, 4
        try:
            handoff_states(torch.eye(K).expand(H, K, K).contiguous(), torch.zeros(H, K, V), None)
            ret[rank] = "no error"
        except RuntimeError as e:
            ret[rank] = str(e)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # the group is already broken on the surviving rank
            pass


def test_handoff_reports_a_peer_that_left():
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_missing_peer, args=(2, 29651, ret), nprocs=2, join=True)
        assert ret[0] == "left"
        assert "receive from rank 0 failed on rank 1" in ret[1], ret[1]
