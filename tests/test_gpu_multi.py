"""GPU (needs >= 2 devices): sequence-parallel forward and backward over NCCL, first against the CPU oracle run over
the whole sequence, then against the single-GPU result."""
import os
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

import oracle
from util import err_ratio

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    # a short process-group timeout: a rank that fails must end its peers' collectives with an error, not leave them waiting
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=timedelta(seconds=120))
    try:
        from fla_b200.ops import chunk_gated_delta_rule
        from fla_b200.parallel import sp_chunk_gated_delta_rule_fwd
        g0 = torch.Generator().manual_seed(11)
        T, H, K, V = 1024 * world + 37, 4, 128, 128   # ragged tail on the last rank
        q = F.normalize(torch.randn(1, T, H, K, generator=g0), dim=-1).bfloat16().cuda()
        k = F.normalize(torch.randn(1, T, H, K, generator=g0), dim=-1).bfloat16().cuda()
        v = torch.randn(1, T, H, V, generator=g0).bfloat16().cuda()
        # weak decay: after a slab the initial state must still matter, or the transition matrix M is never exercised
        g = (F.logsigmoid(torch.randn(1, T, H, generator=g0)) * 0.01).cuda()
        beta = torch.rand(1, T, H, generator=g0).sigmoid().bfloat16().cuda()
        h0 = (torch.randn(1, H, K, V, generator=g0) * 0.1).cuda()
        with torch.no_grad():
            o_ref, ht_ref = chunk_gated_delta_rule(q, k, v, g, beta, initial_state=h0, output_final_state=True, head_first=False)
        lo, hi = 1024 * rank, (1024 * (rank + 1) if rank < world - 1 else T)
        sl = slice(lo, hi)
        o, ht = sp_chunk_gated_delta_rule_fwd(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], initial_state=h0,
                                              output_final_state=True)
        torch.cuda.synchronize()
        o_or, ht_or = oracle.gated_delta_rule(q.float().cpu(), k.float().cpu(), v.float().cpu(), beta.float().cpu(), g=g.cpu(),
                                              initial_state=h0.cpu(), output_final_state=True, head_first=False)
        ret[rank] = (err_ratio(o_ref[:, sl], o), err_ratio(ht_ref, ht), err_ratio(o_or[:, sl], o), err_ratio(ht_or, ht))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_forward_matches_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, 29700, ret), nprocs=world, join=True)
        for r in range(world):
            eo, eh, oo, oh = ret[r]
            print(f"rank {r}: vs oracle o {oo:.2e} ht {oh:.2e}; vs one GPU o {eo:.2e} ht {eh:.2e}")
            assert oo < 5e-3 and oh < 5e-3
            assert eo < 5e-3 and eh < 5e-3


def _worker_bwd(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    # a short process-group timeout: a rank that fails must end its peers' collectives with an error, not leave them waiting
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=timedelta(seconds=120))
    try:
        from fla_b200.ops import chunk_gated_delta_rule
        from fla_b200.parallel import sp_chunk_gated_delta_rule
        g0 = torch.Generator().manual_seed(12)
        T, H, K, V = 512 * world + 21, 2, 128, 128   # ragged tail on the last rank
        q = F.normalize(torch.randn(1, T, H, K, generator=g0), dim=-1).bfloat16().cuda()
        k = F.normalize(torch.randn(1, T, H, K, generator=g0), dim=-1).bfloat16().cuda()
        v = torch.randn(1, T, H, V, generator=g0).bfloat16().cuda()
        # weak decay: after a slab the initial state must still matter, or the transition matrix M is never exercised
        g = (F.logsigmoid(torch.randn(1, T, H, generator=g0)) * 0.01).cuda()
        beta = torch.rand(1, T, H, generator=g0).sigmoid().bfloat16().cuda()
        h0 = (torch.randn(1, H, K, V, generator=g0) * 0.1).cuda()
        do = torch.randn(1, T, H, V, generator=g0).bfloat16().cuda()
        dht = (torch.randn(1, H, K, V, generator=g0) * 0.1).cuda()
        # single-GPU reference gradients
        full = [x.clone().requires_grad_(True) for x in (q, k, v, g, beta, h0)]
        o_ref, ht_ref = chunk_gated_delta_rule(*full[:5], initial_state=full[5], output_final_state=True, head_first=False)
        torch.autograd.backward((o_ref, ht_ref), (do, dht))
        lo, hi = 512 * rank, (512 * (rank + 1) if rank < world - 1 else T)
        sl = slice(lo, hi)
        mine = [x[:, sl].clone().requires_grad_(True) for x in (q, k, v, g, beta)]
        h0_r = h0.clone().requires_grad_(True)
        o, ht = sp_chunk_gated_delta_rule(*mine, initial_state=h0_r, output_final_state=True)
        torch.autograd.backward((o, ht), (do[:, sl], dht))
        torch.cuda.synchronize()
        errs = {n: err_ratio(f.grad[:, sl], m.grad) for n, f, m in zip(("dq", "dk", "dv", "dg", "dbeta"), full, mine)}
        errs["o"] = err_ratio(o_ref[:, sl], o)
        if rank == 0:
            errs["dh0"] = err_ratio(full[5].grad, h0_r.grad)
        # first tier: the CPU oracle over the whole sequence
        cpu = [x.detach().float().cpu().requires_grad_(True) for x in (q, k, v, g, beta, h0)]
        o_or, ht_or = oracle.gated_delta_rule(cpu[0], cpu[1], cpu[2], cpu[4], g=cpu[3], initial_state=cpu[5], output_final_state=True,
                                              head_first=False)
        torch.autograd.backward((o_or, ht_or), (do.float().cpu(), dht.cpu()))
        for n, f, m in zip(("dq", "dk", "dv", "dg", "dbeta"), cpu, mine):
            errs["oracle " + n] = err_ratio(f.grad[:, sl], m.grad)
        errs["oracle o"] = err_ratio(o_or[:, sl], o)
        if rank == 0:
            errs["oracle dh0"] = err_ratio(cpu[5].grad, h0_r.grad)
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_backward_matches_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_bwd, args=(world, 29720, ret), nprocs=world, join=True)
        for r in range(world):
            print(f"rank {r}:", {n: f"{e:.2e}" for n, e in ret[r].items()})
            for n, e in ret[r].items():
                assert e < (2e-2 if n.split()[-1] in ("dg", "dbeta") else 8e-3), (r, n, e)
