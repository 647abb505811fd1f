"""Torch-facing ops with the signatures of the MLX calls the reference makes.

    quantize          <-> mx.quantize            (jang_tools/convert.py:602-645,1533-1554)
    dequantize        <-> mx.dequantize          (jang_tools/loader.py:469, affine.py:445-463)
    quantized_matmul  <-> mx.quantized_matmul    (jang_tools/jangrt/linear.py:41-45)

Tensors live on the current CUDA device; work is enqueued on the current
torch stream.  Packed codes are returned as torch.int32 holding the same bits
as MLX's uint32 (torch has few uint32 kernels); uint32 inputs are accepted.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import JangqError

ALLOWED_BITS = (2, 3, 4, 5, 6, 8)
ALLOWED_GROUP_SIZES = (32, 64, 128)


def _as_i32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.int32:
        return t
    if t.dtype == torch.uint32:
        return t.view(torch.int32)
    raise JangqError(_lib.JQ_EINVAL, f"packed codes must be uint32/int32, got {t.dtype}")


def _check_triple(wq, scales, biases, bits, group_size):
    if bits not in ALLOWED_BITS:
        raise JangqError(_lib.JQ_EUNSUPPORTED, f"unsupported bits={bits}")
    if group_size not in ALLOWED_GROUP_SIZES:
        raise JangqError(_lib.JQ_EUNSUPPORTED, f"unsupported group_size={group_size}")
    K = wq.shape[-1] * 32 // bits
    if wq.shape[-1] * 32 % bits or K % group_size:
        raise JangqError(_lib.JQ_EINVAL, f"packed width {wq.shape[-1]} does not match bits={bits}, "
                                         f"group_size={group_size}")
    if scales.shape != biases.shape or scales.dtype != biases.dtype:
        raise JangqError(_lib.JQ_EINVAL, "scales and biases must share shape and dtype")
    if tuple(scales.shape) != tuple(wq.shape[:-1]) + (K // group_size,):
        raise JangqError(_lib.JQ_EINVAL, f"scales shape {tuple(scales.shape)} does not match codes "
                                         f"{tuple(wq.shape)} at bits={bits}, group_size={group_size}")
    return K


def quantize(w: torch.Tensor, group_size: int = 64, bits: int = 4, *, sidecar_dtype: torch.dtype | None = None,
             f16_tiny_guard: bool = False, mode: str = "affine"):
    """Affine group quantization along the last axis -> (wq, scales, biases).

    The source dtype of `w` (float32/float16/bfloat16) is the arithmetic's input
    precision, exactly as for mx.quantize; the converter feeds float16
    (convert.py:1550).  Sidecars default to the source dtype.  mode="rtn" runs the
    converter's zero-point fallback instead (quantize.py:211-289, float16 sidecars);
    mode="mse" adds quantize_tensor's clip-ratio search (quantize.py:153-191);
    mode="mse_exhaustive" is the same search without the float32 screen, and
    mode="affine_ieee_div" / "rtn_ieee_div" the quantizers with a per-weight IEEE division (cross-checks).
    """
    dev = _lib.require_cuda(w)
    lib = _lib.load()
    if w.dim() < 2:
        raise JangqError(_lib.JQ_EINVAL, f"affine quantization expects a matrix, got {tuple(w.shape)}")
    K = w.shape[-1]
    if K == 0:
        raise JangqError(_lib.JQ_EINVAL, "affine quantization expects rows of at least one group")
    lead = tuple(w.shape[:-1])
    w2 = w.reshape(-1, K).contiguous()
    rows = w2.shape[0]
    if mode in ("rtn", "rtn_ieee_div", "mse", "mse_exhaustive") and sidecar_dtype is None:
        sidecar_dtype = torch.float16
    sdt = sidecar_dtype or w.dtype
    if bits not in ALLOWED_BITS or group_size not in ALLOWED_GROUP_SIZES or K % group_size or (K * bits) % 32:
        # let the library produce the precise message
        pass
    wq = torch.empty((rows, max(K * bits // 32, 0)), dtype=torch.int32, device=dev)
    G = K // group_size if group_size in ALLOWED_GROUP_SIZES else 0
    scales = torch.empty((rows, G), dtype=sdt, device=dev)
    biases = torch.empty((rows, G), dtype=sdt, device=dev)
    with torch.cuda.device(dev):
        if mode in ("affine", "affine_ieee_div"):
            flags = _lib.JQ_QUANT_F16_TINY_GUARD if f16_tiny_guard else 0
            if mode == "affine_ieee_div":
                flags |= _lib.JQ_QUANT_IEEE_DIV
            _lib.check(lib.jq_quantize(w2.data_ptr(), _lib.dtype_id(w2.dtype), rows, K, bits, group_size,
                                       _lib.dtype_id(sdt), flags, wq.data_ptr(), scales.data_ptr(),
                                       biases.data_ptr(), _lib.stream_ptr(dev)))
        elif mode in ("rtn", "rtn_ieee_div"):
            flags = _lib.JQ_QUANT_IEEE_DIV if mode == "rtn_ieee_div" else 0
            _lib.check(lib.jq_quantize_rtn(w2.data_ptr(), _lib.dtype_id(w2.dtype), rows, K, bits, group_size,
                                           _lib.dtype_id(sdt), flags, wq.data_ptr(), scales.data_ptr(),
                                           biases.data_ptr(), _lib.stream_ptr(dev)))
        elif mode in ("mse", "mse_exhaustive"):
            flags = _lib.JQ_QUANT_MSE_EXHAUSTIVE if mode == "mse_exhaustive" else 0
            _lib.check(lib.jq_quantize_mse(w2.data_ptr(), _lib.dtype_id(w2.dtype), rows, K, bits, group_size,
                                           _lib.dtype_id(sdt), flags, wq.data_ptr(), scales.data_ptr(),
                                           biases.data_ptr(), _lib.stream_ptr(dev)))
        else:
            raise JangqError(_lib.JQ_EINVAL, f"unknown quantize mode {mode!r}")
    return wq.reshape(lead + (wq.shape[-1],)), scales.reshape(lead + (G,)), biases.reshape(lead + (G,))


def dequantize(wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64, bits: int = 4,
               dtype: torch.dtype | None = None) -> torch.Tensor:
    """code*scale + bias -> [.., K] in `dtype` (default: the sidecar dtype, as mx.dequantize)."""
    dev = _lib.require_cuda(wq, scales, biases)
    lib = _lib.load()
    wq = _as_i32(wq)
    K = _check_triple(wq, scales, biases, bits, group_size)
    lead = tuple(wq.shape[:-1])
    wq2, s2, b2 = wq.reshape(-1, wq.shape[-1]).contiguous(), scales.reshape(-1, scales.shape[-1]).contiguous(), \
        biases.reshape(-1, biases.shape[-1]).contiguous()
    rows = wq2.shape[0]
    out = torch.empty((rows, K), dtype=dtype or scales.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_dequantize(wq2.data_ptr(), s2.data_ptr(), b2.data_ptr(), _lib.dtype_id(s2.dtype), rows, K,
                                     bits, group_size, out.data_ptr(), _lib.dtype_id(out.dtype),
                                     _lib.stream_ptr(dev)))
    return out.reshape(lead + (K,))


def quantize_imatrix(w: torch.Tensor, importance, group_size: int = 64, bits: int = 4, iterations: int = 6):
    """Activation-weighted affine fit (jang_tools/affine.py:279-399): importance[k] ~ E[x_k^2] of the input the
    matrix consumes.  w [rows, K] (or [E, rows, K]) on the GPU, any float dtype (read as float32); returns
    (wq uint32-as-int32, scales f16, biases f16) in the layout quantized_matmul / gather_qmm consume,
    bit-identical to the reference.  The importance floor (1e-4 of the median positive value) is applied here
    on the host."""
    import numpy as np
    dev = _lib.require_cuda(w)
    lib = _lib.load()
    if bits not in ALLOWED_BITS or group_size not in ALLOWED_GROUP_SIZES:
        raise JangqError(_lib.JQ_EUNSUPPORTED, f"bits={bits}, group_size={group_size} not supported")
    K = w.shape[-1]
    imp = np.asarray(importance.detach().float().cpu().numpy() if isinstance(importance, torch.Tensor) else importance,
                     dtype=np.float32)
    if imp.shape != (K,):
        raise JangqError(_lib.JQ_EINVAL, f"importance must have shape {(K,)}, got {imp.shape}")
    if not np.isfinite(imp).all() or np.any(imp < 0):
        raise JangqError(_lib.JQ_EINVAL, "importance values must be finite and nonnegative")
    positive = imp[imp > 0]
    floor = float(np.median(positive)) * 1e-4 if positive.size else 1.0
    imp = np.maximum(imp, max(floor, 1e-12)).astype(np.float32)
    lead = tuple(w.shape[:-1])
    w2 = w.reshape(-1, K).contiguous()
    rows = w2.shape[0]
    wq = torch.empty((rows, K * bits // 32), dtype=torch.int32, device=dev)
    s = torch.empty((rows, K // group_size), dtype=torch.float16, device=dev)
    b = torch.empty_like(s)
    impd = torch.from_numpy(imp).to(dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_quantize_imatrix(w2.data_ptr(), _lib.dtype_id(w2.dtype), impd.data_ptr(), rows, K, bits,
                                           group_size, iterations, wq.data_ptr(), s.data_ptr(), b.data_ptr(),
                                           _lib.stream_ptr(dev)))
    return wq.reshape(lead + (wq.shape[-1],)), s.reshape(lead + (s.shape[-1],)), b.reshape(lead + (b.shape[-1],))


_SIGNS_CACHE: dict = {}


def hadamard_signs(dim: int, seed: int = 42, device="cuda") -> torch.Tensor:
    """The +-1 vector of the randomized Hadamard transform (jang_tools/turboquant/rotation.py:43-59; the
    converter and the loader both use seed 42), float32 on `device`, cached."""
    import numpy as np
    key = (int(dim), int(seed), str(torch.device(device)))
    t = _SIGNS_CACHE.get(key)
    if t is None:
        s = np.random.default_rng(seed).choice([-1.0, 1.0], size=dim).astype(np.float32)
        t = _SIGNS_CACHE[key] = torch.from_numpy(s).to(device)
    return t


def hadamard_rotate(x: torch.Tensor, signs: torch.Tensor | None = None, seed: int = 42,
                    dtype: torch.dtype | None = None) -> torch.Tensor:
    """H * diag(signs) * x along the last axis, per power-of-two block (rotation.py:86-113).  The reference
    returns float32 (its signs are float32); `dtype` defaults to x's dtype so that the result can feed the
    decode mat-vec directly, pass torch.float32 for the reference's type."""
    dev = _lib.require_cuda(x)
    lib = _lib.load()
    K = x.shape[-1]
    if signs is None:
        signs = hadamard_signs(K, seed, dev)
    if signs.shape != (K,) or signs.dtype != torch.float32:
        raise JangqError(_lib.JQ_EINVAL, f"signs must be float32 [{K}], got {signs.dtype} {tuple(signs.shape)}")
    x2 = x.reshape(-1, K).contiguous()
    out = torch.empty((x2.shape[0], K), dtype=dtype or x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_hadamard_rotate(x2.data_ptr(), _lib.dtype_id(x2.dtype), K, x2.shape[0], K, signs.data_ptr(),
                                          out.data_ptr(), _lib.dtype_id(out.dtype), K, _lib.stream_ptr(dev)))
    return out.reshape(tuple(x.shape[:-1]) + (K,))


def embedding(ids: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64,
              bits: int = 4, dtype: torch.dtype | None = None) -> torch.Tensor:
    """Rows of a quantized table: out[.., :] = dequantize(wq[ids], scales[ids], biases[ids]) in one launch
    (nn.QuantizedEmbedding.__call__; jang-runtime/Metal/JANGEmbedding.metal:57-98).  ids: integer tensor of
    any shape on the table's device; ids outside the table give rows of zeros."""
    dev = _lib.require_cuda(wq, scales, biases, ids)
    lib = _lib.load()
    wq = _as_i32(wq)
    K = _check_triple(wq, scales, biases, bits, group_size)
    if wq.dim() != 2:
        raise JangqError(_lib.JQ_EINVAL, f"embedding table must be [rows, K*bits/32], got {tuple(wq.shape)}")
    wq, scales, biases = wq.contiguous(), scales.contiguous(), biases.contiguous()
    flat = ids.reshape(-1).to(torch.int32).contiguous()
    out = torch.empty((flat.numel(), K), dtype=dtype or scales.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_embedding(flat.data_ptr(), flat.numel(), wq.data_ptr(), scales.data_ptr(), biases.data_ptr(),
                                    _lib.dtype_id(scales.dtype), wq.shape[0], K, bits, group_size, out.data_ptr(),
                                    _lib.dtype_id(out.dtype), _lib.stream_ptr(dev)))
    return out.reshape(tuple(ids.shape) + (K,))


def _qgemv(x2: torch.Tensor, wq, scales, biases, K, bits, group_size, out: torch.Tensor, flags: int = 0):
    lib = _lib.load()
    dev = x2.device
    M, N = x2.shape[0], wq.shape[0]
    _lib.check(lib.jq_qgemv_ex(x2.data_ptr(), _lib.dtype_id(x2.dtype), M, x2.stride(0), wq.data_ptr(),
                               scales.data_ptr(), biases.data_ptr(), _lib.dtype_id(scales.dtype), N, K, bits,
                               group_size, out.data_ptr(), _lib.dtype_id(out.dtype), out.stride(0), flags,
                               _lib.stream_ptr(dev)))


def qgemv_fused(x2: torch.Tensor, linears, outs, flags: int = 0):
    """Mat-vecs of several weight matrices over the same activations x2 [M <= 16, K]: one C call, and
    one kernel launch for every run of up to four matrices that share K, the bit width and the group
    size (q/k/v, or gate/up, of a decoder layer).  `linears` are objects with weight/scales/biases/
    bits/group_size/in_features (JANGLinear), `outs` the output tensors [M, N_i]."""
    lib = _lib.load()
    n = len(linears)
    if n == 0:
        return
    if n > _lib.QGEMV_MAX_BATCH:
        for i in range(0, n, _lib.QGEMV_MAX_BATCH):
            qgemv_fused(x2, linears[i:i + _lib.QGEMV_MAX_BATCH], outs[i:i + _lib.QGEMV_MAX_BATCH], flags)
        return
    descs = (_lib.JqGemvDesc * n)()
    for d, lin, out in zip(descs, linears, outs):
        if lin.scales.dtype != linears[0].scales.dtype or out.dtype != x2.dtype:
            raise JangqError(_lib.JQ_EINVAL, "qgemv_fused: one sidecar dtype, outputs in the activation dtype")
        d.x, d.codes, d.scales, d.biases, d.y = (x2.data_ptr(), lin.weight.data_ptr(), lin.scales.data_ptr(),
                                                 lin.biases.data_ptr(), out.data_ptr())
        d.N, d.K, d.ldx, d.ldy = lin.weight.shape[0], lin.in_features, x2.stride(0), out.stride(0)
        d.bits, d.group_size = lin.bits, lin.group_size
    _lib.check(lib.jq_qgemv_batched_ex(descs, n, x2.shape[0], _lib.dtype_id(x2.dtype),
                                       _lib.dtype_id(linears[0].scales.dtype), flags, _lib.stream_ptr(x2.device)))


def qgemv_fused_norm(res: torch.Tensor, y: torch.Tensor, k: int, linears, outs, flags: int = 0,
                     eps: float | None = None) -> torch.Tensor:
    """x = rms_norm(res + sum of the k rows of y) (one token: res [1, K], y [k, K]) and the mat-vecs of `linears`
    over x in one launch (jq_qgemv_batched_norm); returns x [1, K]."""
    lib = _lib.load()
    n = len(linears)
    K = res.shape[-1]
    if res.shape[0] != 1 or tuple(y.shape) != (k, K) or n < 1 or n > _lib.QGEMV_MAX_BATCH:
        raise JangqError(_lib.JQ_EINVAL, f"qgemv_fused_norm: one token, y [{k}, {K}], 1..{_lib.QGEMV_MAX_BATCH} linears")
    if eps is None:
        eps = torch.finfo(res.dtype).eps
    res, y = res.contiguous(), y.contiguous()
    x = torch.empty_like(res)
    descs = (_lib.JqGemvDesc * n)()
    for d, lin, out in zip(descs, linears, outs):
        d.x, d.codes, d.scales, d.biases, d.y = (x.data_ptr(), lin.weight.data_ptr(), lin.scales.data_ptr(),
                                                 lin.biases.data_ptr(), out.data_ptr())
        d.N, d.K, d.ldx, d.ldy = lin.weight.shape[0], lin.in_features, x.stride(0), out.stride(0)
        d.bits, d.group_size = lin.bits, lin.group_size
    _lib.check(lib.jq_qgemv_batched_norm(res.data_ptr(), y.data_ptr(), y.stride(0), k, float(eps), x.data_ptr(), descs, n,
                                         _lib.dtype_id(res.dtype), _lib.dtype_id(linears[0].scales.dtype), flags,
                                         _lib.stream_ptr(res.device)))
    return x


def quantized_matmul(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                     transpose: bool = True, group_size: int = 64, bits: int = 4,
                     static_weights: bool = False) -> torch.Tensor:
    """y[.., N] = x[.., K] . deq(w)[N, K]^T with float32 accumulation, output in x's dtype.

    Few rows (decode) run the bandwidth-bound mat-vec kernel; many rows (prefill)
    run the tensor-core GEMM.  Only transpose=True (weights stored [N, K], the only
    form the reference uses) is provided.  static_weights=True promises that w/scales/biases are
    not written by earlier work on the stream, which lets the decode kernel overlap its predecessor.
    """
    if not transpose:
        raise JangqError(_lib.JQ_EUNSUPPORTED, "quantized_matmul: only transpose=True is provided")
    dev = _lib.require_cuda(x, w, scales, biases)
    w = _as_i32(w)
    if w.dim() != 2:
        raise JangqError(_lib.JQ_EINVAL, f"weight must be 2-D [N, K*bits/32], got {tuple(w.shape)}")
    K = _check_triple(w, scales, biases, bits, group_size)
    if x.shape[-1] != K:
        raise JangqError(_lib.JQ_EINVAL, f"x has {x.shape[-1]} features, weight expects {K}")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise JangqError(_lib.JQ_EINVAL, f"activations must be bfloat16 or float16, got {x.dtype}")
    lead = tuple(x.shape[:-1])
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M, N = x2.shape[0], w.shape[0]
    w, scales, biases = w.contiguous(), scales.contiguous(), biases.contiguous()
    out = torch.empty((M, N), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        if M <= _lib.QGEMV_MAX_M:
            if M > 0:
                _qgemv(x2, w, scales, biases, K, bits, group_size, out,
                       _lib.JQ_GEMV_STATIC_WEIGHTS if static_weights else 0)
        elif K % 64 == 0 and (K * bits // 8) % 16 == 0:
            from .gemm import qgemm
            qgemm(x2, w, scales, biases, K, bits, group_size, out)
        else:
            # row lengths the tensor-core kernel does not take (K not a multiple of 64, or packed
            # rows that are not a multiple of 16 bytes): the general mat-vec kernel, 16 rows at a time
            for m0 in range(0, M, _lib.QGEMV_MAX_M):
                _qgemv(x2[m0:m0 + _lib.QGEMV_MAX_M], w, scales, biases, K, bits, group_size,
                       out[m0:m0 + _lib.QGEMV_MAX_M])
    return out.reshape(lead + (N,))
