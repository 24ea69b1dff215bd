"""B200-native GPTQ engine behind the call surface of IST-DASLab/MoE-Quant.

    from moe_quant_b200 import gptq            # stands in for  src.gptq
    from moe_quant_b200.packing import pack_weight

All numerics run in libmoequant_sm100.so (hand-written sm_100a CUDA, C ABI in
include/moequant.h).  Importing the package does not load the library; the first
operation does, and raises if it is missing.
"""
from . import dist_utils, gptq, gptq_loop, linalg_utils, model_utils, ops, packing, quant_utils  # noqa: F401
from .gptq import GPTQ, QuantizationOrder, quantize_many, quantize_tied  # noqa: F401
from .ops import Precision, set_default_precision  # noqa: F401
from .packing import pack_to_int32, pack_weight  # noqa: F401

__all__ = ["GPTQ", "QuantizationOrder", "quantize_tied", "quantize_many", "Precision", "set_default_precision", "pack_weight",
           "pack_to_int32"]
