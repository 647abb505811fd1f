"""ctypes binding of libjangq_b200.so (the C ABI declared in include/jangq_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails,
an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libjangq_b200.so")

JQ_OK, JQ_EINVAL, JQ_EUNSUPPORTED, JQ_EWORKSPACE, JQ_ECUDA, JQ_ETIMEOUT = range(6)
JQ_F32, JQ_F16, JQ_BF16 = 0, 1, 2
JQ_QUANT_F16_TINY_GUARD = 1
JQ_QUANT_MSE_EXHAUSTIVE = 2
JQ_QUANT_IEEE_DIV = 4
JQ_GEMV_STATIC_WEIGHTS = 1
JQ_GATHER_FEW_LOCAL = 2
QGEMV_MAX_M = 16
QGEMV_MAX_BATCH = 8
MOE_TILE_M = 128

_DTYPE_ID = {torch.float32: JQ_F32, torch.float16: JQ_F16, torch.bfloat16: JQ_BF16}


class JangqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"jangq_b200 status {status}: {message}")
        self.status = status


class JqGemvDesc(C.Structure):
    _fields_ = [("x", C.c_void_p), ("codes", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
                ("y", C.c_void_p), ("N", C.c_int64), ("K", C.c_int64), ("ldx", C.c_int64), ("ldy", C.c_int64),
                ("bits", C.c_int32), ("group_size", C.c_int32)]


class JqStreamOp(C.Structure):
    _fields_ = [("x", C.c_void_p), ("codes", C.c_void_p * 4), ("scales", C.c_void_p * 4), ("biases", C.c_void_p * 4),
                ("y", C.c_void_p * 4), ("N", C.c_int64 * 4), ("K", C.c_int64), ("count", C.c_int32), ("bits", C.c_int32),
                ("group_size", C.c_int32)]


class JqStreamProgram(C.Structure):
    _fields_ = [("workspace", C.c_void_p), ("n_ops", C.c_int32), ("act_dtype", C.c_int32), ("kmax", C.c_int32),
                ("maxrows", C.c_int32), ("warps", C.c_int32), ("grid", C.c_int32)]


_i64, _i32, _p = C.c_int64, C.c_int, C.c_void_p

# name -> (restype, argtypes); every symbol include/jangq_b200.h declares
SIGNATURES = {
    "jq_version": (C.c_int, []),
    "jq_status_string": (C.c_char_p, [_i32]),
    "jq_last_error": (C.c_char_p, []),
    "jq_quantize": (C.c_int, [_p, _i32, _i64, _i64, _i32, _i32, _i32, _i32, _p, _p, _p, _p]),
    "jq_quantize_rtn": (C.c_int, [_p, _i32, _i64, _i64, _i32, _i32, _i32, _i32, _p, _p, _p, _p]),
    "jq_quantize_mse": (C.c_int, [_p, _i32, _i64, _i64, _i32, _i32, _i32, _i32, _p, _p, _p, _p]),
    "jq_dequantize": (C.c_int, [_p, _p, _p, _i32, _i64, _i64, _i32, _i32, _p, _i32, _p]),
    "jq_qgemv": (C.c_int, [_p, _i32, _i64, _i64, _p, _p, _p, _i32, _i64, _i64, _i32, _i32, _p, _i32, _i64, _p]),
    "jq_qgemv_ex": (C.c_int, [_p, _i32, _i64, _i64, _p, _p, _p, _i32, _i64, _i64, _i32, _i32, _p, _i32, _i64, _i32, _p]),
    "jq_qgemm": (C.c_int, [_p, _i32, _i64, _i64, _p, _p, _p, _i32, _i64, _i64, _i32, _i32, _p, _i32, _i64, _p]),
    "jq_qgemv_batched": (C.c_int, [C.POINTER(JqGemvDesc), _i32, _i64, _i32, _i32, _p]),
    "jq_qgemv_batched_ex": (C.c_int, [C.POINTER(JqGemvDesc), _i32, _i64, _i32, _i32, _i32, _p]),
    "jq_ep_pack_slots": (C.c_int, [_p, _i64, _p, _p, _i64, _i32, _i64, _i32, _i32, _i64, _p, _p, _p, _p, _p]),
    "jq_qgemv_batched_norm": (C.c_int, [_p, _p, _i64, _i32, C.c_float, _p, C.POINTER(JqGemvDesc), _i32, _i32, _i32, _i32, _p]),
    "jq_qgemv_stream_workspace_bytes": (C.c_size_t, [C.POINTER(JqStreamOp), _i32]),
    "jq_qgemv_stream_prepare": (C.c_int, [C.POINTER(JqStreamOp), _i32, _i32, _p, C.c_size_t, C.POINTER(JqStreamProgram), _p]),
    "jq_qgemv_stream_run": (C.c_int, [C.POINTER(JqStreamProgram), _p]),
    "jq_device_status": (C.c_int, []),
    "jq_moe_sort_max_tiles": (C.c_size_t, [_i64, _i32, _i32]),
    "jq_moe_sort": (C.c_int, [_p, _i64, _i32, _i32, _p, _p, _p, _i32, _p, _p, _p, _p]),
    "jq_gather_rows": (C.c_int, [_p, _i64, _p, _p, _i32, _p, _i64, _i64, _i64, _i32, _p]),
    "jq_moe_gemm": (C.c_int, [_p, _i32, _i64, _i64, _p, _p, _p, _p, _i64, _p, _p, _p, _p, _i32, _i64, _i64, _i32, _i32,
                              _p, _i64, _p]),
    "jq_moe_gemm_tiled": (C.c_int, [_p, _i32, _i64, _i64, _p, _p, _p, _p, _i64, _i32, _p, _p, _p, _p, _i32, _i64, _i64, _i32,
                                    _i32, _p, _i64, _p]),
    "jq_moe_gemm_static": (C.c_int, [_p, _i32, _i64, _i64, _p, _i32, _p, _p, _p, _p, _i32, _i64, _i64, _i32, _i32, _p,
                                     _i64, _p]),
    "jq_moe_swiglu": (C.c_int, [_p, _p, _i64, _p, _p, _p, _p, _i64, _i64, _i64, C.c_float, _i32, _p]),
    "jq_moe_combine": (C.c_int, [_p, _i64, _p, _p, _i64, _i32, _i64, _p, _i64, _p, _i32, _p]),
    "jq_moe_combine_shared": (C.c_int, [_p, _i64, _p, _p, _i64, _i32, _i64, _p, _i64, _p, _i64, _p, _i32, _p]),
    "jq_gather_qgemv2": (C.c_int, [_p, _i32, _i64, _i32, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i32, _i32, _i64, _i64,
                                   _i32, _i32, _p, _p, _i64, _i32, _i32, _p]),
    "jq_gather_qgemv_swiglu": (C.c_int, [_p, _p, _i32, _i64, _p, C.c_float, _p, _i64, _p, _p, _p, _p, _i32, _i32, _i64, _i64,
                                         _i32, _i32, _p, _i64, _i32, _i32, _p, _p]),
    "jq_moe_topk": (C.c_int, [_p, _i32, _i64, _i64, _i32, _i32, _i32, C.c_float, _p, _p, _p]),
    "jq_moe_route": (C.c_int, [_p, _i32, _i64, _i64, _i64, _p, _i32, _i32, _i32, C.c_float, _p, _p, _p, _p, _p]),
    "jq_moe_route_norm": (C.c_int, [_p, _p, _i32, _i64, _i64, C.c_float, _p, _p, _i32, _i32, _i32, C.c_float, _p, _p, _p,
                                    _p, _p]),
    "jq_residual_rmsnorm": (C.c_int, [_p, _p, _p, _i32, _i64, _i64, C.c_float, _p, _i32, _p]),
    "jq_device_status_clear": (C.c_int, []),
    "jq_hadamard_rotate": (C.c_int, [_p, _i32, _i64, _i64, _i64, _p, _p, _i32, _i64, _p]),
    "jq_quantize_imatrix": (C.c_int, [_p, _i32, _p, _i64, _i64, _i32, _i32, _i32, _p, _p, _p, _p]),
    "jq_embedding": (C.c_int, [_p, _i64, _p, _p, _p, _i32, _i64, _i64, _i32, _i32, _p, _i32, _p]),
    "jq_tq_gather_matmul": (C.c_int, [_p, _i64, _i32, _p, _i64, _p, _p, _p, _i32, _i64, _i64, _i32, _p, _i64, _p]),
    "jq_tq_fused_gate_up_swiglu": (C.c_int, [_p, _i64, _i32, _p, _i64, _p, _p, _p, _p, _p, _i32, _i64, _i64, _i32,
                                             C.c_float, _p, _i64, _p]),
    "jq_tq_quantize": (C.c_int, [_p, _i64, _i64, _i32, _p, _p, _p, _p]),
    "jq_ep_buffer_bytes": (C.c_size_t, [_i64, _i64]),
    "jq_ep_combine_residual_rmsnorm": (C.c_int, [_p, _p, _i32, _i64, _i64, C.c_float, _p, _i32, _p, _i32, _i32, _i64,
                                                 _p, _i32, _p]),
    "jq_gather_qgemv": (C.c_int, [_p, _i32, _i64, _i32, _p, _i64, _p, _p, _p, _p, _i32, _i32, _i64, _i64, _i32, _i32,
                                  _p, _i64, _p]),
}

_lock = threading.Lock()
_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise JangqError(JQ_ECUDA, f"{LIB_PATH} is missing: build it with `python -m jangq_b200.build` "
                                       "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != JQ_OK:
        lib = load()
        detail = lib.jq_last_error().decode() or lib.jq_status_string(status).decode()
        raise JangqError(status, detail)


def dtype_id(dt: torch.dtype) -> int:
    try:
        return _DTYPE_ID[dt]
    except KeyError:
        raise JangqError(JQ_EINVAL, f"unsupported dtype {dt}; use float32, float16 or bfloat16") from None


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise JangqError(JQ_EINVAL, "jangq_b200 ops take CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise JangqError(JQ_EINVAL, f"tensors on different devices: {dev} vs {t.device}")
    return dev
