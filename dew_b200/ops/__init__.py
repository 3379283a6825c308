"""Hot ops: sm_100a kernels on the GPU, PyTorch references on the CPU."""
from . import library, selection
from .functional import (l2_normalize, adamw_, attention, attention_reference, ema_, gated_rms_norm, gemm, grad_norm_, linear,
                         linear_cross_entropy, linear_cross_entropy_reference, packed_swiglu, linear_swiglu, rms_norm,
                         rms_norm_reference, rope, rope_reference, rope_tables, stream_rms_norm, swiglu)

__all__ = ["l2_normalize", "library", "selection", "gemm", "linear", "rms_norm", "stream_rms_norm", "gated_rms_norm", "packed_swiglu", "linear_swiglu",
           "swiglu", "rope", "rope_tables", "attention", "linear_cross_entropy", "adamw_", "ema_", "grad_norm_",
           "attention_reference", "rms_norm_reference", "rope_reference", "linear_cross_entropy_reference"]
