"""Generate tests/golden/ref_vectors.npz from the reference's own naive PyTorch functions.

Run where a checkout of the reference is available, with FLA_REFERENCE set to its path:
    FLA_REFERENCE=<path to flash-linear-attention> python tests/golden/make_golden.py
The reference package is imported through a stub parent module so that its top-level __init__
(which registers HF model configs) does not run.  Everything is CPU fp32, seeded.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

REF = os.environ.get("FLA_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "fla")):
    sys.exit("set FLA_REFERENCE to the path of a flash-linear-attention checkout")
stub = types.ModuleType("fla")
stub.__path__ = [os.path.join(REF, "fla")]
sys.modules["fla"] = stub

from fla.ops.delta_rule.naive import delta_rule_recurrence  # noqa: E402
from fla.ops.gla.naive import naive_recurrent_gla  # noqa: E402
from fla.ops.retention.naive import naive_retention  # noqa: E402
from fla.ops.simple_gla.naive import torch_simple_gla_recurrent  # noqa: E402


def load_file(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


tgd = load_file(os.path.join(REF, "tests/ops/test_gated_delta.py"), "ref_test_gated_delta")
tcs = load_file(os.path.join(REF, "tests/ops/test_cumsum.py"), "ref_test_cumsum")

out = {}


def put(prefix, **kw):
    for k, v in kw.items():
        out[f"{prefix}.{k}"] = v.detach().cpu().numpy() if torch.is_tensor(v) else np.asarray(v)


def leaf(*shape, gen, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).requires_grad_(True)


def grads(outs, douts, inputs):
    loss = sum((o * d).sum() for o, d in zip(outs, douts) if o is not None)
    return torch.autograd.grad(loss, inputs)


B, H, T, K, V = 2, 2, 70, 16, 24

# ---- GLA (head-first, per-channel gates), fla/ops/gla/naive.py
g0 = torch.Generator().manual_seed(0)
q, k, v = leaf(B, H, T, K, gen=g0), leaf(B, H, T, K, gen=g0), leaf(B, H, T, V, gen=g0)
gk = (F.logsigmoid(torch.randn(B, H, T, K, generator=g0)) / 4).requires_grad_(True)
h0 = leaf(B, H, K, V, gen=g0)
do, dht = torch.randn(B, H, T, V, generator=g0), torch.randn(B, H, K, V, generator=g0)
o, ht = naive_recurrent_gla(q, k, v, gk, initial_state=h0, output_final_state=True)
dq, dk, dv, dg, dh0 = grads((o, ht), (do, dht), (q, k, v, gk, h0))
put("gla", q=q, k=k, v=v, gk=gk, h0=h0, do=do, dht=dht, o=o, ht=ht, dq=dq, dk=dk, dv=dv, dgk=dg, dh0=dh0)

# ---- simple GLA (head-first, scalar gates), fla/ops/simple_gla/naive.py
g0 = torch.Generator().manual_seed(1)
q, k, v = leaf(B, H, T, K, gen=g0), leaf(B, H, T, K, gen=g0), leaf(B, H, T, V, gen=g0)
g = F.logsigmoid(torch.randn(B, H, T, generator=g0)).requires_grad_(True)
h0 = leaf(B, H, K, V, gen=g0)
do, dht = torch.randn(B, H, T, V, generator=g0), torch.randn(B, H, K, V, generator=g0)
o, ht = torch_simple_gla_recurrent(q, k, v, g, initial_state=h0, output_final_state=True)
dq, dk, dv, dg, dh0 = grads((o, ht), (do, dht), (q, k, v, g, h0))
put("simple_gla", q=q, k=k, v=v, g=g, h0=h0, do=do, dht=dht, o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)

# ---- retention (O(T^2) form, head-first, no state), fla/ops/retention/naive.py
g0 = torch.Generator().manual_seed(2)
q = torch.randn(B, 4, T, K, generator=g0)
k = torch.randn(B, 4, T, K, generator=g0)
v = torch.randn(B, 4, T, V, generator=g0)
o = naive_retention(q, k, v)
put("retention", q=q, k=k, v=v, o=o)

# ---- delta rule (head-first), fla/ops/delta_rule/naive.py
g0 = torch.Generator().manual_seed(3)
q = leaf(B, H, T, K, gen=g0)
k = F.normalize(torch.randn(B, H, T, K, generator=g0), p=2, dim=-1).requires_grad_(True)
v = leaf(B, H, T, V, gen=g0)
beta = torch.rand(B, H, T, generator=g0).sigmoid().requires_grad_(True)
h0 = leaf(B, H, K, V, gen=g0, scale=0.1)
do, dht = torch.randn(B, H, T, V, generator=g0), torch.randn(B, H, K, V, generator=g0)
o, ht = delta_rule_recurrence(q, k, v, beta, initial_state=h0.clone(), output_final_state=True)
dq, dk, dv, db, dh0 = grads((o, ht), (do, dht), (q, k, v, beta, h0))
put("delta", q=q, k=k, v=v, beta=beta, h0=h0, do=do, dht=dht, o=o, ht=ht, dq=dq, dk=dk, dv=dv, dbeta=db, dh0=dh0)

# ---- gated delta rule (seq-first, explicit scale), tests/ops/test_gated_delta.py:30-158
g0 = torch.Generator().manual_seed(4)
q = leaf(B, T, H, K, gen=g0)
k = F.normalize(torch.randn(B, T, H, K, generator=g0), p=2, dim=-1).requires_grad_(True)
v = leaf(B, T, H, V, gen=g0)
beta = torch.rand(B, T, H, generator=g0).sigmoid().requires_grad_(True)
g = F.logsigmoid(torch.rand(B, T, H, generator=g0)).requires_grad_(True)
h0 = leaf(B, H, K, V, gen=g0, scale=0.1)
do, dht = torch.randn(B, T, H, V, generator=g0), torch.randn(B, H, K, V, generator=g0)
scale = 0.37
o, ht = tgd.recurrent_gated_delta_rule_ref(q, k, v, beta, g, scale=scale, initial_state=h0, output_final_state=True,
                                           head_first=False)
dq, dk, dv, db, dg, dh0 = grads((o, ht), (do, dht), (q, k, v, beta, g, h0))
o2, ht2 = tgd.chunk_gated_delta_rule_ref(q, k, v, g, beta, scale=scale, initial_state=h0, output_final_state=True,
                                         head_first=False)
put("gated_delta", q=q, k=k, v=v, beta=beta, g=g, h0=h0, do=do, dht=dht, scale=scale, o=o, ht=ht, dq=dq, dk=dk,
    dv=dv, dbeta=db, dg=dg, dh0=dh0, o_chunk=o2, ht_chunk=ht2)

# ---- cumsums, tests/ops/test_cumsum.py:24-40 (seq-first, chunk 64)
g0 = torch.Generator().manual_seed(5)
s3, s4 = torch.randn(2, 150, 3, generator=g0), torch.randn(2, 150, 3, 8, generator=g0)
for name, s in (("s3", s3), ("s4", s4)):
    put(f"cumsum.{name}", x=s,
        local=tcs.cumsum_local_reference(s, reverse=False, head_first=False, chunk_size=64),
        local_rev=tcs.cumsum_local_reference(s, reverse=True, head_first=False, chunk_size=64),
        glob=tcs.cumsum_global_reference(s, reverse=False, head_first=False),
        glob_rev=tcs.cumsum_global_reference(s, reverse=True, head_first=False))

# ---- variable-length chunk tables: the expressions of fla/ops/gated_delta_rule/chunk.py:204-207 and
#      fla/ops/common/chunk_h.py:274-279, evaluated by importing those modules' helpers
from fla.ops.common.chunk_h import prepare_varlen_inputs as ref_chunk_offsets  # noqa: E402
from fla.ops.gla.chunk import prepare_varlen_inputs as ref_indices  # noqa: E402

offsets = torch.tensor([0, 1, 64, 65, 200, 456, 1000, 1000 + 63, 1063 + 128], dtype=torch.long)
idx = ref_indices(offsets, 64)
co = ref_chunk_offsets(offsets, 64)
put("varlen", offsets=offsets, indices=idx, chunk_offsets=co)

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, f"{os.path.getsize(path) / 1024:.0f} KiB", len(out), "arrays")
