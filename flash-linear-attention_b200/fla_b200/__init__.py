# -*- coding: utf-8 -*-
"""fla_b200 — B200 (sm_100a) CUDA implementation of the chunked linear-attention hot path of
flash-linear-attention, behind the reference's `fla.ops` call signatures.

    from fla_b200.ops.gated_delta_rule import chunk_gated_delta_rule

`install_as_fla_ops()` registers the op modules under the names `fla.ops.<family>` so that code
written against the reference imports these kernels instead.
"""

import sys
import types

__version__ = "0.1.0"


def install_as_fla_ops():
    """Alias `fla.ops.{gla,simple_gla,retention,delta_rule,gated_delta_rule}` to this package."""
    from . import ops
    from .ops import delta_rule, gated_delta_rule, gla, retention, simple_gla
    root = sys.modules.get("fla")
    if root is None:
        root = types.ModuleType("fla")
        root.__path__ = []
        sys.modules["fla"] = root
    sys.modules["fla.ops"] = ops
    root.ops = ops
    for name, mod in (("gla", gla), ("simple_gla", simple_gla), ("retention", retention),
                      ("delta_rule", delta_rule), ("gated_delta_rule", gated_delta_rule)):
        sys.modules[f"fla.ops.{name}"] = mod


def install_as_fla_modules():
    """Alias `fla.modules.l2norm` and `fla.modules.fused_norm_gate` to this package's CUDA implementation."""
    from . import modules
    from .modules import l2norm
    root = sys.modules.get("fla")
    if root is None:
        root = types.ModuleType("fla")
        root.__path__ = []
        sys.modules["fla"] = root
    sys.modules["fla.modules"] = modules
    sys.modules["fla.modules.l2norm"] = l2norm
    from .modules import fused_norm_gate
    sys.modules["fla.modules.fused_norm_gate"] = fused_norm_gate
    from .modules import convolution
    sys.modules["fla.modules.convolution"] = convolution
    root.modules = modules

