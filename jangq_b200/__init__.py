"""jangq_b200 — B200-native JANG affine quantized-inference path.

Host side: torch tensors + ctypes into libjangq_b200.so (hand-written sm_100a
kernels).  The op names follow the MLX calls the reference makes.
"""
from ._lib import JangqError
from .linear import JANGLinear
from .ops import ALLOWED_BITS, ALLOWED_GROUP_SIZES, dequantize, quantize, quantized_matmul
from .moe import ExpertBank, gather_qmm, moe_layer, route_softmax_topk
from .plan import GemvPlan

__all__ = ["JangqError", "ALLOWED_BITS", "ALLOWED_GROUP_SIZES", "quantize", "dequantize", "quantized_matmul",
           "JANGLinear", "GemvPlan", "ExpertBank", "gather_qmm", "moe_layer", "route_softmax_topk"]
