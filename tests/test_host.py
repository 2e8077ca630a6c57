"""CPU: the C-ABI library loads and exports every symbol the header declares; host-side logic
(variable-length tables, argument checks) behaves like the reference's."""
import ctypes
import os
import re

import pytest
import torch

import oracle
from conftest import ROOT
from fla_b200 import _lib
from fla_b200.utils import chunk_tables


def header_symbols():
    text = open(os.path.join(ROOT, "include", "flab200.h")).read()
    return sorted(set(re.findall(r"\b(flab_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    syms = header_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/flab200.h but not exported"
    assert lib.flab_abi_version() == 1
    assert set(_lib.ENTRY_POINTS) <= set(syms)


def test_args_struct_matches_header_field_order():
    text = open(os.path.join(ROOT, "include", "flab200.h")).read()
    body = text[text.index("typedef struct flab_args {"):text.index("} flab_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S).replace("typedef struct flab_args {", "")
    names = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        parts = decl.replace("*", " ").replace(",", " ").split()
        names += [p for p in parts if p not in ("int32_t", "float", "const", "void", "size_t")]
    assert names == [f[0] for f in _lib.FlabArgs._fields_]


def test_bad_arguments_are_rejected_without_a_gpu():
    lib = _lib.load()
    a = _lib.FlabArgs()
    rc = lib.flab_chunk_fwd_h(ctypes.byref(a), None)
    assert rc == -1
    assert b"positive" in lib.flab_last_error()


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_chunk_tables_bit_exact(dtype, golden):
    offsets = torch.from_numpy(golden["varlen.offsets"]).to(dtype)
    lengths = (offsets[1:] - offsets[:-1]).tolist()
    indices, chunk_offsets = chunk_tables(lengths)
    assert torch.equal(torch.tensor(indices, dtype=dtype), oracle.chunk_indices_ref(offsets))
    assert torch.equal(torch.tensor(chunk_offsets, dtype=dtype), oracle.chunk_offsets_ref(offsets))
    assert torch.equal(torch.tensor(indices), torch.from_numpy(golden["varlen.indices"]))
    assert torch.equal(torch.tensor(chunk_offsets), torch.from_numpy(golden["varlen.chunk_offsets"]))


def test_wrapper_argument_checks_match_reference():
    from fla_b200.ops import chunk_delta_rule, chunk_gated_delta_rule, chunk_gla, chunk_simple_gla
    q = torch.zeros(2, 8, 2, 16, dtype=torch.bfloat16)
    g3 = torch.zeros(2, 8, 2)
    off = torch.tensor([0, 4, 8])
    with pytest.raises(ValueError, match="batch size is expected to be 1"):
        chunk_simple_gla(q, q, q, g3, offsets=off, head_first=False)
    with pytest.raises(RuntimeError, match="head-first"):
        chunk_gla(q[:1], q[:1], q[:1], q[:1].float(), offsets=off, head_first=True)
    with pytest.raises(ValueError, match="number of initial states"):
        chunk_simple_gla(q[:1], q[:1], q[:1], g3[:1], offsets=off, head_first=False,
                         initial_state=torch.zeros(3, 2, 16, 16))
    with pytest.raises(AssertionError, match="float32"):
        chunk_delta_rule(q.float(), q.float(), q.float(), g3, head_first=False)
    with pytest.raises(AssertionError, match="float32"):
        chunk_gated_delta_rule(q.float(), q.float(), q.float(), g3, g3, head_first=False)
    with pytest.raises(AssertionError, match="Scale must be positive"):
        chunk_gated_delta_rule(q, q, q, g3, g3.bfloat16(), scale=-1.0, head_first=False)
    with pytest.raises(ValueError, match="either"):
        chunk_simple_gla(q[:1], q[:1], q[:1], g3[:1], offsets=off, cu_seqlens=off, head_first=False)


def test_no_cpu_fallback():
    from fla_b200.ops import chunk_simple_gla
    q = torch.zeros(1, 8, 2, 16, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        chunk_simple_gla(q, q, q, torch.zeros(1, 8, 2), head_first=False)
