"""Prefill GEMM wrapper (jq_qgemm): used by ops.quantized_matmul for many activation rows."""
from __future__ import annotations

import torch

from . import _lib


def qgemm(x2: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, K: int, bits: int,
          group_size: int, out: torch.Tensor) -> None:
    """out[M,N] = x2[M,K] . deq(wq)[N,K]^T on the tensor cores.  Sidecars are converted to the
    activation dtype if they differ (the kernel computes fma(q, scale, bias) in that type)."""
    lib = _lib.load()
    if scales.dtype != x2.dtype:
        scales, biases = scales.to(x2.dtype), biases.to(x2.dtype)
    if x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
        if x2.stride(0) % 8:
            raise _lib.JangqError(_lib.JQ_EINVAL, "qgemm needs K to be a multiple of 8")
    M, N = x2.shape[0], wq.shape[0]
    _lib.check(lib.jq_qgemm(x2.data_ptr(), _lib.dtype_id(x2.dtype), M, x2.stride(0), wq.data_ptr(), scales.data_ptr(),
                            biases.data_ptr(), _lib.dtype_id(scales.dtype), N, K, bits, group_size, out.data_ptr(),
                            _lib.dtype_id(out.dtype), out.stride(0), _lib.stream_ptr(x2.device)))
