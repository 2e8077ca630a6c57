# -*- coding: utf-8 -*-
"""ctypes binding of libflab200.so (the C ABI declared in include/flab200.h).

The shared library is the product: there is no Python or CPU fallback.  Importing this module
without the built library raises immediately with the build command.
"""

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLA_B200_LIB", os.path.join(_HERE, "libflab200.so"))

CHUNK = 64

_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}

F_REVERSE = 1 << 0
F_BETA_VECTOR = 1 << 1
F_INPLACE_STATE = 1 << 2
F_DESCENDING = 1 << 3
F_STATE_ONLY = 1 << 4
F_TRANSPOSE = 1 << 5

_PTR_FIELDS = [
    "q", "k", "v", "g", "gk", "gv", "beta", "w", "u", "aw", "au", "h", "h0", "ht", "v_new", "o",
    "d_o", "dh", "dht", "dh0", "dq", "dk", "dv", "dv2", "dw", "du", "dg", "dgk", "dgv", "dbeta",
    "a", "da", "x", "y", "ws",
]


class FlabArgs(ctypes.Structure):
    """Mirror of `struct flab_args` (include/flab200.h)."""
    _fields_ = (
        [(n, ctypes.c_int32) for n in ("B", "T", "H", "K", "V", "N", "NT", "dtype", "head_first", "flags")]
        + [("scale", ctypes.c_float), ("S", ctypes.c_int32)]
        + [(n, ctypes.c_void_p) for n in ("cu_seqlens", "chunk_indices", "chunk_offsets")]
        + [(n, ctypes.c_void_p) for n in _PTR_FIELDS]
        + [("ws_bytes", ctypes.c_size_t)]
    )


ENTRY_POINTS = [
    "flab_chunk_local_cumsum_scalar", "flab_chunk_local_cumsum_vector",
    "flab_chunk_global_cumsum_scalar", "flab_chunk_global_cumsum_vector",
    "flab_chunk_fwd_h", "flab_chunk_bwd_dh", "flab_chunk_fwd_o", "flab_chunk_bwd_dv",
    "flab_chunk_bwd_dv_local", "flab_chunk_bwd_dqkwg", "flab_wy_fwd", "flab_wy_recompute",
    "flab_wy_bwd", "flab_delta_fwd_h", "flab_delta_bwd_dhu", "flab_gla_fwd_intra", "flab_gla_fwd_o",
    "flab_gla_bwd_dav", "flab_gla_bwd_dqkg", "flab_recurrent_fwd", "flab_recurrent_bwd",
    "flab_recurrent_delta_fwd", "flab_recurrent_delta_bwd", "flab_gated_delta_rule_fwd",
    "flab_gated_delta_rule_fwd_noalloc", "flab_simple_gla_attn",
]

_lib = None
LAUNCHES = 0  # kernels launched through this module (one per successful call)
# FLA_B200_CHECK=1: synchronise after every call and turn a device-side wait that ran out into an exception
# (FLAB_E_TIMEOUT). Off by default: the check costs a device synchronisation per launch.
CHECK_EVERY_CALL = os.environ.get("FLA_B200_CHECK", "0") == "1"


def load() -> ctypes.CDLL:
    """Load the shared library once; fail loudly if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found. Build it with `make -C flash-linear-attention_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    lib.flab_last_error.restype = ctypes.c_char_p
    lib.flab_abi_version.restype = ctypes.c_int
    for name in ENTRY_POINTS:
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(FlabArgs), ctypes.c_void_p]
    lib.flab_gated_delta_rule_fwd_workspace.restype = ctypes.c_size_t
    lib.flab_gated_delta_rule_fwd_workspace.argtypes = [ctypes.POINTER(FlabArgs)]
    for name in ("flab_tc_error_state", "flab_tc_check", "flab_tc_error_clear"):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = []
    lib.flab_tc_wait_selftest.restype = ctypes.c_int
    lib.flab_tc_wait_selftest.argtypes = [ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    lib.flab_l2norm_fwd.restype = ctypes.c_int
    lib.flab_l2norm_fwd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_float, ctypes.c_void_p]
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    lib.flab_rms_norm_swish_gate_partials.restype = ci
    lib.flab_rms_norm_swish_gate_partials.argtypes = [ll, ci, ci]
    lib.flab_rms_norm_swish_gate_fwd.restype = ci
    lib.flab_rms_norm_swish_gate_fwd.argtypes = [vp, vp, vp, vp, vp, ll, ci, ci, cf, vp]
    lib.flab_rms_norm_swish_gate_bwd.restype = ci
    lib.flab_rms_norm_swish_gate_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ll, ci, ci, vp]
    lib.flab_short_conv_fwd.restype = ci
    lib.flab_short_conv_fwd.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]
    lib.flab_short_conv_bwd.restype = ci
    lib.flab_short_conv_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]
    lib.flab_short_conv_update.restype = ci
    lib.flab_short_conv_update.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]
    lib.flab_l2norm_bwd.restype = ctypes.c_int
    lib.flab_l2norm_bwd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_float, ctypes.c_void_p]
    ap = ctypes.POINTER(FlabArgs)
    lib.flab_gdn_gate_fwd.restype = ci
    lib.flab_gdn_gate_fwd.argtypes = [ap, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.flab_gdn_gate_bwd.restype = ci
    lib.flab_gdn_gate_bwd.argtypes = [ap, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.flab_state_chain.restype = ci
    lib.flab_state_chain.argtypes = [vp, vp, ll, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]
    _lib = lib
    return lib


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    assert t.is_contiguous(), "flab200 kernels need contiguous tensors"
    return t.data_ptr()


def fill_args(ref: torch.Tensor, *, B, T, H, K=0, V=0, N=None, NT=0, dtype=None, head_first=False,
              flags=0, scale=1.0, S=0, varlen=None, ws_bytes=0, **tensors) -> FlabArgs:
    """Build a `flab_args` struct; `tensors` maps slot names to tensors (None = absent)."""
    a = FlabArgs()
    a.ws_bytes = ws_bytes
    a.B, a.T, a.H, a.K, a.V = B, T, H, K, V
    a.N = N if N is not None else B
    a.NT = NT
    a.dtype = _DTYPES[dtype if dtype is not None else ref.dtype]
    a.head_first = int(bool(head_first))
    a.flags = flags
    a.scale = float(scale)
    a.S = S
    if varlen is not None:
        a.cu_seqlens = varlen.cu_seqlens.data_ptr()
        a.chunk_indices = varlen.chunk_indices.data_ptr()
        a.chunk_offsets = varlen.chunk_offsets.data_ptr()
    for name, t in tensors.items():
        if name not in _PTR_FIELDS:
            raise KeyError(f"unknown flab_args slot {name!r}")
        if t is not None:
            if t.device != ref.device:
                raise RuntimeError(f"slot {name}: tensor on {t.device}, expected {ref.device}")
            setattr(a, name, _ptr(t))
    return a


def call(entry: str, ref: torch.Tensor, **kw):
    """Launch one entry point on the current stream of `ref`'s device (see `fill_args`).

    `varlen` is the tuple produced by `fla_b200.utils.prepare_varlen` or None.
    """
    lib = load()
    if not ref.is_cuda:
        raise RuntimeError("flab200 kernels run on CUDA tensors only (no CPU fallback)")
    a = fill_args(ref, **kw)
    with torch.cuda.device(ref.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = getattr(lib, entry)(ctypes.byref(a), ctypes.c_void_p(stream))
    if rc != 0:
        raise RuntimeError(f"{entry} failed ({rc}): {lib.flab_last_error().decode()}")
    global LAUNCHES
    LAUNCHES += 1
    if CHECK_EVERY_CALL:
        check_device_waits(entry)


def check_device_waits(what: str = "flab200") -> None:
    """Synchronise and raise if a bounded wait inside one of the library's kernels has run out since the last
    check (the kernel returned normally, but its outputs are invalid). Clears the record."""
    lib = load()
    rc = lib.flab_tc_check()
    if rc != 0:
        msg = lib.flab_last_error().decode()
        lib.flab_tc_error_clear()
        raise RuntimeError(f"{what} failed ({rc}): {msg}")


def state_chain(M: torch.Tensor, b: torch.Tensor, s0: Optional[torch.Tensor], *, want_s_in: bool = True, want_last: bool = False,
                reverse: bool = False, transpose: bool = False):
    """`flab_state_chain`: M `[B,S,H,K,K]`, b `[B,S,H,K,V]` (may be a column slice of a wider contiguous buffer), s0
    `[B,H,K,V]` or None, all fp32 CUDA. Returns (s_in `[B,S,H,K,V]` or None, s_last `[B,H,K,V]` or None)."""
    lib = load()
    B, S, H, K, _ = M.shape
    V = b.shape[-1]
    assert M.is_cuda and M.dtype == b.dtype == torch.float32 and M.is_contiguous()
    assert b.stride(-1) == 1 and b.stride(-3) == K * b.stride(-2) and b.stride(-4) == H * b.stride(-3) and b.stride(0) == S * b.stride(1), \
        "b must be a column slice of a contiguous [B,S,H,K,ldb] buffer"
    s0 = None if s0 is None else s0.float().contiguous()
    s_in = torch.empty(B, S, H, K, V, dtype=torch.float32, device=M.device) if want_s_in else None
    s_last = torch.empty(B, H, K, V, dtype=torch.float32, device=M.device) if want_last else None
    flags = (F_REVERSE if reverse else 0) | (F_TRANSPOSE if transpose else 0)
    with torch.cuda.device(M.device):
        rc = lib.flab_state_chain(M.data_ptr(), b.data_ptr(), b.stride(-2), None if s0 is None else s0.data_ptr(),
                                  None if s_in is None else s_in.data_ptr(), None if s_last is None else s_last.data_ptr(),
                                  B, S, H, K, V, flags, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"flab_state_chain failed ({rc}): {lib.flab_last_error().decode()}")
    global LAUNCHES
    LAUNCHES += 1
    return s_in, s_last
