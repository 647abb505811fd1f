"""jangq_b200 — B200-native JANG affine quantized-inference path.

Host side: torch tensors + ctypes into libjangq_b200.so (hand-written sm_100a
kernels).  The op names follow the MLX calls the reference makes.
"""
from ._lib import JangqError
from .linear import JANGEmbedding, JANGLinear, JANGSwitchLinear
from .ops import ALLOWED_BITS, ALLOWED_GROUP_SIZES, dequantize, embedding, hadamard_rotate, hadamard_signs, quantize, quantize_imatrix, quantized_matmul
from .moe import ExpertBank, gather_qmm, moe_layer, route_softmax_topk
from .plan import GemvPlan
from .tensor_quant import QuantizedTensor, dequantize_tensor, quantize_tensor
from .turboquant import TurboQuantLinear, TurboQuantSwitchLinear, tq_quantize_weight
from .bundle import is_jang_model, load_jang_model, load_modules as load_jang_modules, open_bundle, repack_v1_to_v2, write_bundle

__all__ = ["JangqError", "QuantizedTensor", "quantize_tensor", "dequantize_tensor", "ALLOWED_BITS", "ALLOWED_GROUP_SIZES", "quantize", "quantize_imatrix", "dequantize", "embedding", "hadamard_rotate", "hadamard_signs", "quantized_matmul",
           "JANGLinear", "JANGSwitchLinear", "JANGEmbedding", "GemvPlan", "ExpertBank", "gather_qmm", "moe_layer", "route_softmax_topk",
           "TurboQuantLinear", "TurboQuantSwitchLinear", "tq_quantize_weight", "is_jang_model", "load_jang_model", "open_bundle", "load_jang_modules", "write_bundle", "repack_v1_to_v2"]
