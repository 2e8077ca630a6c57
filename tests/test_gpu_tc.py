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
