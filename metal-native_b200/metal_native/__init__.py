"""metal_native -- the fused INT4/INT8 dequantise + matmul operator of MetalNative,
rebuilt for NVIDIA B200 (sm_100a).

Only the dequant-matmul path of the reference package (``python/metal_native``) exists
here.  As in the reference, the operator lives in ``metal_native._C``; it is re-exported
at package level for convenience.
"""
from . import _C
from ._C import (MetalNativeError, dequant_matmul, dequant_matmul_fused, dequant_matmul_swiglu, dequantize,
                 dequantize_flat, fused_residual_norm, synchronize)
from .quant_weight_cache import QuantFormat, QuantWeightCache
from .packing import pack_int4
from .phase_pipeline import InferencePhase, PhaseConfig, PhasePipeline

__all__ = ["_C", "MetalNativeError", "dequant_matmul", "dequant_matmul_fused", "dequant_matmul_swiglu", "dequantize",
           "dequantize_flat", "fused_residual_norm", "synchronize", "QuantWeightCache", "QuantFormat", "pack_int4", "InferencePhase",
           "PhaseConfig", "PhasePipeline"]
__version__ = _C.version()
