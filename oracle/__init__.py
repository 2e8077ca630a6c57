"""CPU restatement of the reference's linear-attention algorithms.  TEST INFRASTRUCTURE ONLY.

This package is the checker the CUDA kernels are compared against (tests/, the smoke test and the
cpu_baseline / reference arm of bench.py).  Nothing under fla_b200/ imports it, and it must never be
used as a fallback compute path.

Parity pin: every function here is checked in tests/test_oracle_golden.py against vectors produced
by the reference's own naive PyTorch functions (tests/golden/make_golden.py, run against the
reference checkout) - see each function's docstring for the reference file:line it restates.  The L2-norm
functions are pinned against outputs of the reference's Triton kernels run through Triton's CPU interpreter
(tests/golden/make_golden_l2norm.py), and so are the chunk ops a second time: the reference's chunked Triton kernels,
forward and backward, run under the same interpreter (tests/golden/make_golden_triton.py ->
tests/golden/triton_vectors.npz; the oracle agrees with them to 2e-4 .. 5e-4 on fp16 inputs and 3e-7 on fp32).
"""

from .indexing import chunk_indices_ref, chunk_offsets_ref  # noqa: F401
from .l2norm import l2_norm, l2_norm_bwd  # noqa: F401
from .short_conv import short_conv, short_conv_step  # noqa: F401
from .norm_gate import rms_norm_swish_gate, rms_norm_swish_gate_bwd  # noqa: F401
from .naive import (chunk_state_gradients, chunk_states, cumsum_global, cumsum_local, delta_rule, gated_delta_rule, gla,  # noqa: F401
                    retention_log_decay, simple_gla, simple_gla_attention)
