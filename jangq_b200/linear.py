"""Quantized linear modules with the reference's constructor signatures.

    JANGLinear        <-> jang_tools/jangrt/linear.py:22-45
    JANGSwitchLinear  <-> SwitchProj, jang_tools/dsv41/model.py:847-857

Buffers keep the reference's names (`weight`, `scales`, `biases`, optional
`bias`) and shapes, so a state dict written by the reference's converter loads
with `load_state_dict` after a uint32 -> int32 view.
"""
from __future__ import annotations

import torch
from torch import nn

from . import ops


class JANGLinear(nn.Module):
    """Affine-quantized linear: y = quantized_matmul(x, weight, scales, biases) (+ bias)."""

    def __init__(self, in_features: int, out_features: int, bits: int = 4, group_size: int = 64,
                 bias: bool = False, device=None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.bits, self.group_size = bits, group_size
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.zeros((out_features, in_features * bits // 32), dtype=torch.int32,
                                                   device=device))
        self.register_buffer("scales", torch.zeros((out_features, in_features // group_size), dtype=dtype,
                                                   device=device))
        self.register_buffer("biases", torch.zeros((out_features, in_features // group_size), dtype=dtype,
                                                   device=device))
        self.register_buffer("bias", torch.zeros((out_features,), dtype=dtype, device=device) if bias else None)
        # set by freeze(): the weights will not be written any more, so decode launches may overlap
        # their predecessor on the stream (JQ_GEMV_STATIC_WEIGHTS)
        self.static_weights = False

    def freeze(self):
        """Declare the quantized weights final (call after loading, with the device idle)."""
        self.static_weights = True
        return self

    @classmethod
    def from_float(cls, w: torch.Tensor, bits: int = 4, group_size: int = 64, bias: torch.Tensor | None = None):
        """Quantize a float [out, in] CUDA tensor (mx.quantize semantics, source dtype = w.dtype)."""
        out_f, in_f = w.shape
        m = cls(in_f, out_f, bits, group_size, bias is not None, device=w.device,
                dtype=w.dtype if w.dtype != torch.float32 else torch.bfloat16)
        wq, s, b = ops.quantize(w, group_size, bits, sidecar_dtype=m.scales.dtype)
        m.weight, m.scales, m.biases = wq, s, b
        if bias is not None:
            m.bias = bias.to(m.scales.dtype)
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = ops.quantized_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                                 group_size=self.group_size, bits=self.bits, static_weights=self.static_weights)
        return y if self.bias is None else y + self.bias

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bits={self.bits}, group_size={self.group_size}"
