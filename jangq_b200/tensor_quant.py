"""Host mirror of the reference's per-block tensor quantizer.

`quantize_tensor(weights, bit_allocation, block_size, method)` and `dequantize_tensor(qt, block_size)` keep the
names, argument meaning, return type and error behaviour of jang_tools/quantize.py:211-337; the arithmetic runs in the
CUDA kernels (`jq_quantize_rtn`, `jq_quantize_mse`, `jq_dequantize`).  Blocks are consecutive `block_size` runs of the
flattened tensor (quantize.py:238-258), zero-padded at the end, so the tensor is handed to the kernels as a
[n_blocks, block_size] matrix with one group per row.  numpy arrays are copied to the current CUDA device and the
results copied back; CUDA tensors stay on their device and the result holds CUDA tensors.
"""
from __future__ import annotations

from typing import NamedTuple

import numpy as np
import torch

from . import _lib
from ._lib import JangqError
from .ops import ALLOWED_BITS, ALLOWED_GROUP_SIZES, dequantize, quantize

DEFAULT_BLOCK_SIZE = 64


class QuantizedTensor(NamedTuple):
    """Result of quantizing a weight tensor (quantize.py:20-27)."""

    qweight: object          # packed codes, uint8, LSB-first bit stream over all blocks
    scales: object           # per-block scales, float16
    biases: object           # per-block biases (-scale * zero point), float16
    bits: int
    shape: tuple


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise JangqError(_lib.JQ_EINVAL, "jangq_b200 needs a CUDA device (there is no CPU path)")
    return torch.device("cuda", torch.cuda.current_device())


def quantize_tensor(weights, bit_allocation, block_size: int = DEFAULT_BLOCK_SIZE, method: str = "mse") -> QuantizedTensor:
    """Quantize a tensor at one bit width with per-block scale and bias.

    method="rtn": min/max zero-point rounding; method="mse" (the default, as in the reference): the clip-ratio
    search for 2-4 bits, RTN arithmetic above.  Raises ValueError where the reference does (block count mismatch,
    mixed or unsupported bit widths).
    """
    as_numpy = not isinstance(weights, torch.Tensor)
    shape = tuple(weights.shape)
    n_weights = int(np.prod(shape)) if len(shape) else 1
    bit_allocation = np.asarray(bit_allocation.cpu() if isinstance(bit_allocation, torch.Tensor) else bit_allocation)
    n_blocks = len(bit_allocation)
    expected_blocks = (n_weights + block_size - 1) // block_size
    if n_blocks != expected_blocks:
        raise ValueError(f"bit_allocation has {n_blocks} blocks but weight has "
                         f"{n_weights} values ({expected_blocks} blocks at block_size={block_size})")
    unique_bits = set(int(b) for b in np.unique(bit_allocation))
    if len(unique_bits) != 1:
        raise ValueError(f"quantize_tensor expects uniform bit width per tensor, "
                         f"got {unique_bits}. Use profile-based allocation.")
    bits = unique_bits.pop()
    if bits not in ALLOWED_BITS:
        raise ValueError(f"Invalid bit width {bits}. Allowed: {sorted(ALLOWED_BITS)}")
    if method not in ("rtn", "mse"):
        raise ValueError(f"unknown method {method!r}: 'rtn' or 'mse'")
    if block_size not in ALLOWED_GROUP_SIZES:
        raise JangqError(_lib.JQ_EUNSUPPORTED, f"block_size {block_size}: the kernels take {ALLOWED_GROUP_SIZES}")

    if as_numpy:
        flat = torch.from_numpy(np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)).to(_device())
    else:
        _lib.require_cuda(weights)
        flat = weights.reshape(-1).float()               # quantize.py:240: the arithmetic is float32
    pad = n_blocks * block_size - n_weights
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    wq, scales, biases = quantize(flat.reshape(n_blocks, block_size), block_size, bits, mode=method)
    qweight = wq.reshape(-1).view(torch.uint8)
    scales, biases = scales.reshape(-1), biases.reshape(-1)
    if as_numpy:
        return QuantizedTensor(qweight.cpu().numpy(), scales.cpu().numpy(), biases.cpu().numpy(), bits, shape)
    return QuantizedTensor(qweight, scales, biases, bits, shape)


def dequantize_tensor(qt: QuantizedTensor, block_size: int = DEFAULT_BLOCK_SIZE):
    """code * scale + bias in float32, in the original shape (quantize.py:292-337)."""
    as_numpy = not isinstance(qt.qweight, torch.Tensor)
    if block_size not in ALLOWED_GROUP_SIZES:
        raise JangqError(_lib.JQ_EUNSUPPORTED, f"block_size {block_size}: the kernels take {ALLOWED_GROUP_SIZES}")
    dev = _device() if as_numpy else _lib.require_cuda(qt.qweight, qt.scales, qt.biases)
    to_dev = (lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)) if as_numpy else (lambda t: t)
    scales, biases = to_dev(qt.scales).reshape(-1, 1), to_dev(qt.biases).reshape(-1, 1)
    n_blocks = scales.shape[0]
    words = block_size * qt.bits // 32
    qweight = to_dev(qt.qweight).reshape(-1)
    if qweight.numel() != n_blocks * words * 4:
        raise ValueError(f"qweight holds {qweight.numel()} bytes, {n_blocks} blocks of {block_size} "
                         f"{qt.bits}-bit codes take {n_blocks * words * 4}")
    wq = qweight.view(torch.int32).reshape(n_blocks, words)
    flat = dequantize(wq, scales, biases, block_size, qt.bits, dtype=torch.float32).reshape(-1)
    total = int(np.prod(qt.shape)) if len(qt.shape) else 1
    out = flat[:total].reshape(qt.shape)
    return out.cpu().numpy() if as_numpy else out
