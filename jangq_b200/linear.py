"""Quantized linear modules with the reference's constructor signatures.

    JANGLinear        <-> jang_tools/jangrt/linear.py:22-45
    JANGSwitchLinear  <-> SwitchProj, jang_tools/dsv41/model.py:847-857
    JANGEmbedding     <-> nn.QuantizedEmbedding of the bundles (jang-runtime/Metal/JANGEmbedding.metal:57-98)

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


class JANGSwitchLinear(nn.Module):
    """Stacked quantized experts of one projection with the fields and call shape of the reference's
    SwitchProj (jang_tools/dsv41/model.py:847-857): `weight` [E, out, in*bits/32], `scales` and `biases`
    [E, out, in/group_size], one bit width for the whole stack; `module(x, idx, sorted_indices)` is
    gather_qmm(x, weight, scales, biases, rhs_indices=idx, transpose=True, ...).

    Shapes as MLX broadcasts them at the reference's call sites (model.py:1207-1230): x [T, 1, 1, in] with idx
    [T, k] gives [T, k, 1, out]; x [R, 1, in] (rows already gathered per pair) with idx [R] gives [R, 1, out];
    a plain x [R, in] with idx [R] gives [R, out]."""

    def __init__(self, n_experts: int, in_dim: int, out_dim: int, bits: int, group_size: int = 64, device=None,
                 dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.bits, self.group_size = bits, group_size
        self.n_experts, self.in_features, self.out_features = n_experts, in_dim, out_dim
        self.register_buffer("weight", torch.zeros((n_experts, out_dim, in_dim * bits // 32), dtype=torch.int32,
                                                   device=device))
        self.register_buffer("scales", torch.zeros((n_experts, out_dim, in_dim // group_size), dtype=dtype,
                                                   device=device))
        self.register_buffer("biases", torch.zeros((n_experts, out_dim, in_dim // group_size), dtype=dtype,
                                                   device=device))
        self._bank = None
        self._bank_key = None

    @classmethod
    def from_float(cls, w: torch.Tensor, bits: int = 4, group_size: int = 64):
        """Quantize float experts [E, out, in] on the GPU (mx.quantize semantics)."""
        E, out_f, in_f = w.shape
        m = cls(E, in_f, out_f, bits, group_size, device=w.device,
                dtype=w.dtype if w.dtype != torch.float32 else torch.bfloat16)
        m.weight, m.scales, m.biases = ops.quantize(w, group_size, bits, sidecar_dtype=m.scales.dtype)
        return m

    @property
    def bank(self):
        """The ExpertBank (device pointer tables) over the current buffers, rebuilt when they were replaced."""
        from .moe import ExpertBank
        key = (self.weight.data_ptr(), self.scales.data_ptr(), self.biases.data_ptr())
        if self._bank is None or self._bank_key != key:
            self._bank = ExpertBank(self.weight, self.scales, self.biases, self.bits, self.group_size)
            self._bank_key = key
        return self._bank

    def forward(self, x: torch.Tensor, idx: torch.Tensor, sorted_indices: bool = False) -> torch.Tensor:
        from .moe import gather_qmm
        if x.dim() >= 3 and x.shape[-2] != 1:
            raise ops.JangqError(ops._lib.JQ_EUNSUPPORTED, "JANGSwitchLinear takes one activation row per index "
                                                          f"(x.shape[-2] == 1), got {tuple(x.shape)}")
        # sorted_indices only tells MLX that idx is ascending; the result is the same either way
        y = gather_qmm(x.reshape(-1, x.shape[-1]), self.bank, rhs_indices=idx, group_size=self.group_size,
                       bits=self.bits)
        if x.dim() >= 3:
            return y.reshape(tuple(idx.shape) + (1, self.out_features))
        return y.reshape(tuple(idx.shape) + (self.out_features,))

    def extra_repr(self) -> str:
        return (f"experts={self.n_experts}, in={self.in_features}, out={self.out_features}, bits={self.bits}, "
                f"group_size={self.group_size}")


class JANGEmbedding(nn.Module):
    """Quantized embedding table (nn.QuantizedEmbedding of the reference's bundles): rows are dequantized on
    lookup; `as_linear(x)` is the tied output head, quantized_matmul over the same table."""

    def __init__(self, num_embeddings: int, dims: int, bits: int = 4, group_size: int = 64, device=None,
                 dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.bits, self.group_size = bits, group_size
        self.num_embeddings, self.dims = num_embeddings, dims
        self.register_buffer("weight", torch.zeros((num_embeddings, dims * bits // 32), dtype=torch.int32, device=device))
        self.register_buffer("scales", torch.zeros((num_embeddings, dims // group_size), dtype=dtype, device=device))
        self.register_buffer("biases", torch.zeros((num_embeddings, dims // group_size), dtype=dtype, device=device))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids, self.weight, self.scales, self.biases, self.group_size, self.bits)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                                    group_size=self.group_size, bits=self.bits)
