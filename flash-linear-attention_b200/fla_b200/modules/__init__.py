# -*- coding: utf-8 -*-
"""Steps right before / after the chunk ops in the reference's layers (fla/modules)."""
from .convolution import ShortConvolution
from .fused_norm_gate import FusedRMSNormSwishGate, rms_norm_swish_gate_fn
from .gate_prologue import gdn_gate_beta
from .l2norm import L2NormFunction, l2_norm, l2norm_bwd, l2norm_fwd

__all__ = ["L2NormFunction", "l2_norm", "l2norm_fwd", "l2norm_bwd", "FusedRMSNormSwishGate", "rms_norm_swish_gate_fn",
           "ShortConvolution", "gdn_gate_beta"]
