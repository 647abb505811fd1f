"""JANGTQ: rotated codebook weights on the GPU.

    compute_codebook            <-> jang_tools/turboquant/codebook.py:48-102 (Lloyd-Max centroids per (dim, bits))
    tq_quantize_weight(s)       <-> jang_tools/turboquant/linear.py:137-200
    TurboQuantLinear            <-> linear.py:24-60        (packed, norms, codebook, signs; y = x @ W^T)
    TurboQuantSwitchLinear      <-> linear.py:63-133       (stacked experts; module(x, idx))
    tq_fused_gate_up_swiglu     <-> jangtq_fused_gate_up_swiglu, JANGTQMatmul.metal:154-262
    tq_gather_matmul            <-> jangtq_gather_tq_matmul, JANGTQMatmul.metal:281-363

The reference multiplies by the de-rotated matrix; its Metal kernels (and these) rotate the activations once
instead, x_rot = H diag(signs) x, and multiply by norm * codebook[idx] -- the same product, since the
rotation is orthogonal.
"""
from __future__ import annotations

import functools
import math

import numpy as np
import torch
from torch import nn

from . import _lib, ops
from ._lib import JangqError

TQ_BITS = (2, 3, 4)


@functools.lru_cache(maxsize=64)
def compute_codebook(dim: int, bits: int, n_iter: int = 200) -> tuple:
    """2^bits sorted centroids of the post-rotation coordinate distribution: the density of one coordinate of a
    random unit vector in `dim` dimensions, (1 - x^2)^((dim - 3) / 2), quantized by Lloyd-Max iteration on a
    10000-point grid (conditional means by the trapezoid rule, start uniform on +-3/sqrt(dim), stop when the
    centroids move less than 1e-10).  The values are part of the storage format: a bundle quantized by the
    reference decodes with exactly these numbers."""
    if bits < 1:
        return (0.0,)
    n = 1 << bits
    x = np.linspace(-1.0, 1.0, 10000)
    if dim <= 2:
        f = np.full_like(x, 0.5)
    else:
        c = math.lgamma(dim / 2.0) - 0.5 * math.log(math.pi) - math.lgamma((dim - 1) / 2.0)
        f = np.exp(c + (dim - 3) / 2.0 * np.log(np.maximum(1.0 - x ** 2, 1e-30)))
    integrate = getattr(np, "trapezoid", None) or np.trapz
    area = integrate(f, x)
    if area > 0:
        f = f / area
    half_width = 3.0 / np.sqrt(max(dim, 1))
    cent = np.linspace(-half_width, half_width, n)
    for _ in range(n_iter):
        cuts = np.concatenate([[-1.0], (cent[:-1] + cent[1:]) / 2.0, [1.0]])
        nxt = cent.copy()
        for i in range(n):
            inside = (x >= cuts[i]) & ((x <= cuts[i + 1]) if i == n - 1 else (x < cuts[i + 1]))
            if inside.sum() > 1:
                nxt[i] = integrate(x[inside] * f[inside], x[inside]) / max(integrate(f[inside], x[inside]), 1e-10)
        done = np.allclose(cent, nxt, atol=1e-10)
        cent = nxt
        if done:
            break
    return tuple(sorted(cent.tolist()))


def codebook_tensor(dim: int, bits: int, device) -> torch.Tensor:
    return torch.tensor(compute_codebook(dim, bits), dtype=torch.float32, device=device)


def _check_bits(bits: int):
    if bits not in TQ_BITS:
        raise JangqError(_lib.JQ_EUNSUPPORTED, f"JANGTQ codebooks of {TQ_BITS} bits, got {bits}")


def tq_quantize_weight(weight: torch.Tensor, bits: int = 2, seed: int = 42) -> dict:
    """{"packed": int32 [.., out, words], "norms": float16 [.., out]} of a float CUDA matrix [out, in] or a stack
    [E, out, in]: rows rotated on the GPU (jq_hadamard_rotate, float32), then jq_tq_quantize."""
    _check_bits(bits)
    dev = _lib.require_cuda(weight)
    lib = _lib.load()
    K = weight.shape[-1]
    lead = tuple(weight.shape[:-1])
    w2 = weight.reshape(-1, K).float().contiguous()
    signs = ops.hadamard_signs(K, seed, dev)
    w_rot = ops.hadamard_rotate(w2, signs, dtype=torch.float32)
    cb = np.asarray(compute_codebook(K, bits), dtype=np.float32)
    edges = torch.from_numpy(((cb[:-1] + cb[1:]) / np.float32(2.0)).astype(np.float32)).to(dev)
    per = 32 // bits
    words = (K + per - 1) // per
    rows = w2.shape[0]
    packed = torch.empty((rows, words), dtype=torch.int32, device=dev)
    norms = torch.empty((rows,), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_tq_quantize(w_rot.data_ptr(), rows, K, bits, edges.data_ptr(), packed.data_ptr(),
                                      norms.data_ptr(), _lib.stream_ptr(dev)))
    return {"packed": packed.reshape(lead + (words,)), "norms": norms.reshape(lead)}


def tq_gather_matmul(x_rot: torch.Tensor, packed: torch.Tensor, norms: torch.Tensor, codebook: torch.Tensor,
                     rhs_indices: torch.Tensor | None, bits: int, x_div: int = 1) -> torch.Tensor:
    """out[p] = norms[e] * (codebook[idx[e]] . x_rot[p // x_div]) in float32; packed [E, N, words] (or [N, words]
    with rhs_indices None), x_rot float32 [rows, K]."""
    _check_bits(bits)
    dev = _lib.require_cuda(x_rot, packed, norms, codebook)
    lib = _lib.load()
    if packed.dim() == 2:
        packed, norms = packed.unsqueeze(0), norms.unsqueeze(0)
    E, N, _ = packed.shape
    x_rot = x_rot.float().contiguous()
    K = x_rot.shape[-1]
    if rhs_indices is None:
        pairs, rhs_ptr = x_rot.shape[0] * x_div, None
    else:
        rhs = rhs_indices.reshape(-1).to(torch.int32).contiguous()
        pairs, rhs_ptr = rhs.numel(), rhs.data_ptr()
    out = torch.empty((pairs, N), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_tq_gather_matmul(x_rot.data_ptr(), x_rot.stride(0), x_div, rhs_ptr, pairs,
                                           ops._as_i32(packed).contiguous().data_ptr(), norms.contiguous().data_ptr(),
                                           codebook.data_ptr(), E, N, K, bits, out.data_ptr(), out.stride(0),
                                           _lib.stream_ptr(dev)))
    return out


def tq_fused_gate_up_swiglu(x_rot: torch.Tensor, gate: "TurboQuantSwitchLinear", up: "TurboQuantSwitchLinear",
                            rhs_indices: torch.Tensor, swiglu_limit: float = 0.0) -> torch.Tensor:
    """act[t * k + j] = silu(gate_e x_t) * up_e x_t for e = rhs_indices[t, j] in one launch; x_rot float32 [T, K]
    already rotated with gate's signs; returns float32 [T * k, N]."""
    dev = _lib.require_cuda(x_rot, rhs_indices)
    lib = _lib.load()
    if (gate.bits, gate.in_features, gate.out_features, gate.num_experts) != (up.bits, up.in_features, up.out_features,
                                                                             up.num_experts):
        raise JangqError(_lib.JQ_EINVAL, "gate and up must share bits and shapes")
    x_rot = x_rot.float().contiguous()
    k = rhs_indices.shape[-1] if rhs_indices.dim() == 2 else 1
    rhs = rhs_indices.reshape(-1).to(torch.int32).contiguous()
    out = torch.empty((rhs.numel(), gate.out_features), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_tq_fused_gate_up_swiglu(x_rot.data_ptr(), x_rot.stride(0), k, rhs.data_ptr(), rhs.numel(),
                                                  gate.packed.data_ptr(), gate.norms.data_ptr(), up.packed.data_ptr(),
                                                  up.norms.data_ptr(), gate.codebook.data_ptr(), gate.num_experts,
                                                  gate.out_features, gate.in_features, gate.bits, float(swiglu_limit),
                                                  out.data_ptr(), out.stride(0), _lib.stream_ptr(dev)))
    return out


class TurboQuantLinear(nn.Module):
    """Linear layer over JANGTQ weights (linear.py:24-60): `packed` [out, words], `norms` [out] float16,
    `codebook` [2^bits] and `signs` [in] float32.  forward rotates x once and runs the codebook mat-vec."""

    def __init__(self, in_features: int, out_features: int, bits: int = 2, bias: bool = False, seed: int = 42,
                 device=None):
        super().__init__()
        _check_bits(bits)
        self.in_features, self.out_features, self.bits, self._seed = in_features, out_features, bits, seed
        per = 32 // bits
        self.register_buffer("packed", torch.zeros((out_features, (in_features + per - 1) // per), dtype=torch.int32,
                                                   device=device))
        self.register_buffer("norms", torch.zeros((out_features,), dtype=torch.float16, device=device))
        self.register_buffer("codebook", torch.tensor(compute_codebook(in_features, bits), dtype=torch.float32,
                                                      device=device))
        s = np.random.default_rng(seed).choice([-1.0, 1.0], size=in_features).astype(np.float32)
        self.register_buffer("signs", torch.from_numpy(s).to(device) if device is not None else torch.from_numpy(s))
        self.register_buffer("bias", torch.zeros((out_features,), dtype=torch.float32, device=device) if bias else None)

    @classmethod
    def from_float(cls, w: torch.Tensor, bits: int = 2, seed: int = 42):
        m = cls(w.shape[1], w.shape[0], bits, False, seed, device=w.device)
        q = tq_quantize_weight(w, bits, seed)
        m.packed, m.norms = q["packed"], q["norms"]
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = tuple(x.shape[:-1])
        x_rot = ops.hadamard_rotate(x.reshape(-1, self.in_features).float(), self.signs, dtype=torch.float32)
        y = tq_gather_matmul(x_rot, self.packed, self.norms, self.codebook, None, self.bits)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(lead + (self.out_features,)).to(x.dtype)


class TurboQuantSwitchLinear(nn.Module):
    """Stacked experts over JANGTQ weights (linear.py:63-133): `packed` [E, out, words], `norms` [E, out].
    module(x, idx): x [T, in] (or [T, 1, in]) with idx [T, k] -> [T, k, out]; rows already expanded per pair,
    x [R, in] with idx [R], -> [R, out].  Only the experts named by idx are read."""

    def __init__(self, in_features: int, out_features: int, num_experts: int, bits: int = 2, seed: int = 42,
                 device=None):
        super().__init__()
        _check_bits(bits)
        self.in_features, self.out_features, self.num_experts, self.bits = in_features, out_features, num_experts, bits
        per = 32 // bits
        self.register_buffer("packed", torch.zeros((num_experts, out_features, (in_features + per - 1) // per),
                                                   dtype=torch.int32, device=device))
        self.register_buffer("norms", torch.zeros((num_experts, out_features), dtype=torch.float16, device=device))
        self.register_buffer("codebook", torch.tensor(compute_codebook(in_features, bits), dtype=torch.float32,
                                                      device=device))
        s = np.random.default_rng(seed).choice([-1.0, 1.0], size=in_features).astype(np.float32)
        self.register_buffer("signs", torch.from_numpy(s).to(device) if device is not None else torch.from_numpy(s))

    @classmethod
    def from_float(cls, w: torch.Tensor, bits: int = 2, seed: int = 42):
        m = cls(w.shape[2], w.shape[1], w.shape[0], bits, seed, device=w.device)
        q = tq_quantize_weight(w, bits, seed)
        m.packed, m.norms = q["packed"], q["norms"]
        return m

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return ops.hadamard_rotate(x.reshape(-1, self.in_features).float(), self.signs, dtype=torch.float32)

    def forward(self, x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        x_rot = self.rotate(x)
        if idx.dim() == 2 and x_rot.shape[0] == idx.shape[0]:
            y = tq_gather_matmul(x_rot, self.packed, self.norms, self.codebook, idx, self.bits, x_div=idx.shape[1])
            return y.reshape(idx.shape[0], idx.shape[1], self.out_features).to(x.dtype)
        if x_rot.shape[0] != idx.numel():
            raise JangqError(_lib.JQ_EINVAL, f"cannot match {x_rot.shape[0]} rows of x with {idx.numel()} indices")
        y = tq_gather_matmul(x_rot, self.packed, self.norms, self.codebook, idx, self.bits, x_div=1)
        return y.reshape(tuple(idx.shape) + (self.out_features,)).to(x.dtype)
