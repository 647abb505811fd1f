"""CPU oracle for the JANG affine quantized-inference path.

TEST INFRASTRUCTURE ONLY.  This module is a numpy restatement of the
reference's algorithm; it exists so that tests, the smoke check and the
bench's CPU-baseline leg can check (and time) the CUDA path against it.
The product package never imports it: the product path has no CPU fallback
and fails loudly when the CUDA library is missing.

Parity status: the quantizer, packer and dequantizer are pinned against
the reference's own numpy code (jang-tools/jang_tools/affine.py, pack.py,
quantize.py, imported when the reference tree is mounted) and against the
reference's MLX-generated golden vector
(jang-runtime/Tests/JANGCoreMetalTests/fixtures/matmul_4bit_64x128.safetensors);
see tests/golden/make_golden.py and tests/test_oracle_golden.py.  The
matmul and gather_qmm arithmetic lives in the un-vendored third-party
packages mlx 0.31.2 / mlx-lm 0.31.3 (jang-tools/uv.lock:910-962); it is
restated from the reference's decoder (affine.py:445-463), its in-repo
transcription of the MLX qmv order (dsv41/metal_decode.py:201-234) and the
golden vector's y_ref.  The plain softmax-top-k router lives in mlx-lm
only: parity unpinned for that one function.

Every function cites the reference lines it follows (paths are relative
to the reference project's root).
"""
from __future__ import annotations

import numpy as np

ALLOWED_BITS = (2, 3, 4, 5, 6, 8)          # jang_tools/affine.py:210
ALLOWED_GROUP_SIZES = (32, 64, 128)        # jang_tools/affine.py:27

# smallest normal float16, the mirror-only scale floor (affine.py:43)
_FP16_TINY = np.float32(np.finfo(np.float16).smallest_normal)


# --------------------------------------------------------------------------
# dtype helpers (bf16 by hand so that the oracle needs numpy only)
# --------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (round-to-nearest-even), return uint16 bits."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    rounded = np.where(nan, (u >> 16) | 0x0040, rounded)
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Return float32 values rounded to `dtype` ('f32' | 'f16' | 'bf16')."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "f16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(x.shape)
    raise ValueError(f"unknown dtype {dtype!r}")


# --------------------------------------------------------------------------
# a1: bit packing  (jang_tools/pack.py:12-82 pack, :85-149 unpack)
# --------------------------------------------------------------------------
def pack_rows(codes: np.ndarray, bits: int) -> np.ndarray:
    """LSB-first bitstream per row, viewed as little-endian uint32 words.

    Code j of a row occupies bits [j*bits, j*bits+bits) of that row's stream
    (pack.py:28-82); rows are packed independently and the stream is re-viewed
    as uint32 [rows, K*bits/32] (affine.py:256-265).
    """
    codes = np.asarray(codes, dtype=np.uint8)
    rows, K = codes.shape
    if (K * bits) % 32:
        raise ValueError(f"packed row is not uint32-aligned: columns={K}, bits={bits}")
    shifts = np.arange(bits, dtype=np.uint8)
    bitplane = ((codes[:, :, None] >> shifts) & 1).astype(np.uint8)
    stream = np.packbits(bitplane.reshape(rows, K * bits), axis=1, bitorder="little")
    return np.ascontiguousarray(stream).view("<u4").reshape(rows, K * bits // 32)


def unpack_rows(packed: np.ndarray, bits: int, K: int | None = None) -> np.ndarray:
    """Inverse of pack_rows -> uint8 [rows, K] (pack.py:85-149), vectorised for every width: the stream is
    cut into units of lcm(bits, 8) bits (1 byte for 2/4/8-bit codes, 3 bytes for 3/6-bit, 5 bytes for 5-bit),
    each unit is read as one little-endian integer and its codes are shifted out.  (The reference's own
    3/5/6-bit branch is a per-element loop.)"""
    packed = np.ascontiguousarray(packed, dtype="<u4")
    rows, words = packed.shape
    if K is None:
        K = words * 32 // bits
    unit_bytes = {2: 1, 4: 1, 8: 1, 3: 3, 6: 3, 5: 5}[bits]
    per_unit = unit_bytes * 8 // bits
    if K % per_unit:
        raise ValueError(f"K={K} is not a multiple of {per_unit} codes")
    stream = packed.view(np.uint8).reshape(rows, words * 4)[:, : K * bits // 8].reshape(rows, -1, unit_bytes)
    if unit_bytes == 1:
        unit = stream[:, :, 0]
    else:
        unit = np.zeros(stream.shape[:2], dtype=np.uint64)
        for i in range(unit_bytes):
            unit |= stream[:, :, i].astype(np.uint64) << np.uint64(8 * i)
    shifts = (np.arange(per_unit) * bits).astype(unit.dtype)
    codes = (unit[:, :, None] >> shifts) & unit.dtype.type((1 << bits) - 1)
    return codes.astype(np.uint8).reshape(rows, K)


# --------------------------------------------------------------------------
# a2: affine group quantizer (jang_tools/affine.py:193-276, mirror of MLX
#     affine_quantize; converter call sites convert.py:602-645,1533-1554)
# --------------------------------------------------------------------------
def quantize_affine_codes(w: np.ndarray, bits: int, group_size: int, src_dtype: str = "f16",
                          sidecar_dtype: str | None = None, f16_tiny_guard: bool = False):
    """Return (codes uint8 [rows,K], scales f32 [rows,K/gs], biases f32 [rows,K/gs]).

    Scales/biases are float32 arrays holding values already rounded to
    `sidecar_dtype` (default: the source dtype, affine.py:254-255).  The source
    is first rounded to `src_dtype` (affine.py:212 casts to float16; the MLX
    kernel itself takes f32/f16/bf16 and the golden vector was made from f32).
    `f16_tiny_guard` reproduces the numpy mirror's `_to_f16_nonzero`
    (affine.py:46-51), which MLX does not do; it only matters for f16 sidecars.
    """
    if bits not in ALLOWED_BITS:
        raise ValueError(f"unsupported native affine bits={bits}")
    if group_size not in ALLOWED_GROUP_SIZES:
        raise ValueError(f"unsupported affine group_size={group_size}")
    w = np.asarray(w)
    if w.ndim != 2:
        raise ValueError(f"affine quantization expects a 2D matrix, got {w.shape}")
    rows, K = w.shape
    if K % group_size:
        raise ValueError(f"input dimension {K} is not divisible by group_size={group_size}")
    if (K * bits) % 32:
        raise ValueError(f"packed row is not uint32-aligned: columns={K}, bits={bits}")
    sidecar_dtype = sidecar_dtype or src_dtype
    G = K // group_size
    bins = np.float32((1 << bits) - 1)
    g = round_to(w, src_dtype).reshape(rows, G, group_size)          # affine.py:212,227-229
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        lo = g.min(axis=-1)                                          # :230
        hi = np.maximum(g.max(axis=-1), np.float32(0.0))             # :233 (max seeded with 0)
        scale = np.maximum((hi - lo) / bins, np.float32(1e-7))       # :234
        dom_lo = np.abs(lo) > np.abs(hi)                             # :235
        scale = np.where(dom_lo, scale, -scale)                      # :236
        edge = np.where(dom_lo, lo, hi)                              # :237
        q0 = np.rint(edge / scale)                                   # :238 (half-to-even)
        at_zero = q0 == 0                                            # :239
        refined = np.where(at_zero, scale, edge / np.where(at_zero, np.float32(1), q0))
        scale = refined.astype(np.float32)                           # :240-246
        bias = np.where(at_zero, np.float32(0.0), edge).astype(np.float32)   # :247
        q = np.minimum(np.rint((g - bias[..., None]) / scale[..., None]), bins)  # :248-250
    codes = np.nan_to_num(q, nan=0.0).clip(0, float(bins)).astype(np.uint8)
    s = scale
    if f16_tiny_guard and sidecar_dtype == "f16":                    # affine.py:46-51
        s = np.where(np.abs(s) < _FP16_TINY,
                     np.copysign(_FP16_TINY, np.where(s == 0, np.float32(1.0), s)), s)
    return (codes.reshape(rows, K), round_to(s, sidecar_dtype).reshape(rows, G),
            round_to(bias, sidecar_dtype).reshape(rows, G))


def quantize_affine(w, bits, group_size, src_dtype="f16", sidecar_dtype=None, f16_tiny_guard=False):
    """(packed uint32 [rows, K*bits/32], scales, biases) — see quantize_affine_codes."""
    codes, s, b = quantize_affine_codes(w, bits, group_size, src_dtype, sidecar_dtype, f16_tiny_guard)
    return pack_rows(codes, bits), s, b


# --------------------------------------------------------------------------
# a3: RTN zero-point quantizer, the converter's no-MLX fallback
#     (jang_tools/quantize.py:127-208 else-branch, :211-289; convert.py:1564-1592)
# --------------------------------------------------------------------------
def quantize_rtn_codes(w: np.ndarray, bits: int, group_size: int = 64):
    """Return (codes, scales, biases) with f16-rounded sidecars held in float32.

    Blocks are consecutive `group_size` runs of the flattened [rows, K] tensor
    (quantize.py:238-256), identical to per-row groups when K % group_size == 0.
    """
    w = np.asarray(w, dtype=np.float32)
    rows, K = w.shape
    if K % group_size:
        raise ValueError("K must be a multiple of group_size")
    L = np.float32((1 << bits) - 1)
    blk = w.reshape(-1, group_size)
    wmin = blk.min(axis=1)                                           # quantize.py:148-149
    wmax = blk.max(axis=1)
    const = wmax == wmin                                             # :152
    rng = wmax - wmin                                                # :193-194
    rng[const] = 1.0
    scale = (rng / L).astype(np.float32)                             # :196
    zero = np.clip(np.round(-wmin / scale), 0, L)                    # :197-198
    q = np.clip(np.round(blk / scale[:, None] + zero[:, None]), 0, L).astype(np.uint8)  # :200-201
    scale[const] = 1.0                                               # :203-205
    zero[const] = 0.0
    q[const] = 0
    scales = round_to(scale, "f16")                                  # :278
    biases = round_to((-scale * zero).astype(np.float32), "f16")     # :279
    G = K // group_size
    return q.reshape(rows, K), scales.reshape(rows, G), biases.reshape(rows, G)


def quantize_rtn(w, bits, group_size=64):
    codes, s, b = quantize_rtn_codes(w, bits, group_size)
    return pack_rows(codes, bits), s, b


# --------------------------------------------------------------------------
# f3: clip-ratio search, quantize_tensor's default method="mse"
#     (jang_tools/quantize.py:153-191; bits > 4 take the RTN branch, :153,:192)
# --------------------------------------------------------------------------
MSE_CLIP_RATIOS = np.linspace(0.7, 1.0, 20)                          # quantize.py:163


def _sum_like_numpy(sq: np.ndarray) -> np.ndarray:
    """Row sums of a float64 [n, gs] array (gs in 8..128) in the order numpy's
    add.reduce uses along a contiguous axis: eight running sums over the
    elements i = j (mod 8), folded as ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7))."""
    n, gs = sq.shape
    r = sq[:, 0:8].copy()
    for i in range(8, gs, 8):
        r = r + sq[:, i:i + 8]
    return ((r[:, 0] + r[:, 1]) + (r[:, 2] + r[:, 3])) + ((r[:, 4] + r[:, 5]) + (r[:, 6] + r[:, 7]))


def quantize_mse_codes(w: np.ndarray, bits: int, group_size: int = 64):
    """Return (codes, scales, biases), f16-rounded sidecars held in float32.

    The reference multiplies float32 block minima by float64 clip ratios, so
    under NumPy >= 2 promotion rules the whole search (scale, zero point, codes,
    squared error) runs in float64 and only the winning scale is rounded to
    float32 (quantize.py:159,184).  This restatement follows that arithmetic,
    with the error sum written out in numpy's reduction order.
    """
    if bits > 4:
        return quantize_rtn_codes(w, bits, group_size)
    w = np.asarray(w, dtype=np.float32)
    rows, K = w.shape
    if K % group_size:
        raise ValueError("K must be a multiple of group_size")
    L = (1 << bits) - 1
    blk = w.reshape(-1, group_size)
    nb = blk.shape[0]
    wmin = blk.min(axis=1)
    wmax = blk.max(axis=1)
    const = wmax == wmin
    x = blk.astype(np.float64)
    best_q = np.zeros((nb, group_size), dtype=np.uint8)                  # :158-161
    best_scale = np.ones(nb, dtype=np.float32)
    best_zero = np.zeros(nb, dtype=np.float32)
    best_mse = np.full(nb, np.inf, dtype=np.float64)
    for ratio in MSE_CLIP_RATIOS:
        c_min = wmin.astype(np.float64) * ratio                          # :164-165
        c_max = wmax.astype(np.float64) * ratio
        c_range = c_max - c_min                                          # :167-168
        c_range[c_range == 0] = 1.0
        scale = c_range / L                                              # :170
        zero = np.clip(np.round(-c_min / scale), 0, L)                   # :171-172
        q = np.clip(np.round(x / scale[:, None] + zero[:, None]), 0, L)  # :174-175
        err = x - (q - zero[:, None]) * scale[:, None]                   # :176
        mse = _sum_like_numpy(err * err) / group_size                    # :178
        better = mse < best_mse                                          # :181-185
        best_mse[better] = mse[better]
        best_q[better] = q[better].astype(np.uint8)
        best_scale[better] = scale[better]
        best_zero[better] = zero[better]
    best_scale[const] = 1.0                                              # :187-189
    best_zero[const] = 0.0
    best_q[const] = 0
    scales = round_to(best_scale, "f16")                                 # :281
    biases = round_to((-best_scale * best_zero).astype(np.float32), "f16")  # :282
    G = K // group_size
    return best_q.reshape(rows, K), scales.reshape(rows, G), biases.reshape(rows, G)


def quantize_mse(w, bits, group_size=64):
    codes, s, b = quantize_mse_codes(w, bits, group_size)
    return pack_rows(codes, bits), s, b


# --------------------------------------------------------------------------
# a4: dequantizer (jang_tools/affine.py:445-463; docs/adoption/PORTING.md:80-116)
# --------------------------------------------------------------------------
def dequantize_affine(packed, scales, biases, bits: int, group_size: int) -> np.ndarray:
    """W[i,j] = code[i,j]*scales[i,j//gs] + biases[i,j//gs] in float32, the
    product and the sum rounded separately (numpy: two float32 operations)."""
    packed = np.asarray(packed)
    rows = packed.shape[0]
    K = packed.shape[1] * 32 // bits
    codes = unpack_rows(packed, bits, K).astype(np.float32).reshape(rows, K // group_size, group_size)
    s = np.asarray(scales, dtype=np.float32)[..., None]
    b = np.asarray(biases, dtype=np.float32)[..., None]
    return (codes * s + b).reshape(rows, K)


# --------------------------------------------------------------------------
# a5/a6: quantized matmul  y = x . deq(W)^T
#   arithmetic: affine.py:457-463 + JangV2QuantMatmul.metal:50-70 (dequant then
#   f32 dot); MLX qmv order transcribed at dsv41/metal_decode.py:201-234
# --------------------------------------------------------------------------
def qmatmul(x, packed, scales, biases, bits: int, group_size: int, acc=np.float64) -> np.ndarray:
    """Y[M,N] = X[M,K] . deq(W)[N,K]^T, accumulated in `acc`, returned as f32."""
    W = dequantize_affine(packed, scales, biases, bits, group_size)
    x = np.atleast_2d(np.asarray(x, dtype=np.float32))
    return (x.astype(acc) @ W.astype(acc).T).astype(np.float32)


def qmatmul_group_order(x, packed, scales, biases, bits: int, group_size: int) -> np.ndarray:
    """Same product in the MLX qmv order: per group s*sum(q*x) + b*sum(x), f32
    (dsv41/metal_decode.py:201-234).  Small shapes only."""
    packed = np.asarray(packed)
    N = packed.shape[0]
    K = packed.shape[1] * 32 // bits
    G = K // group_size
    q = unpack_rows(packed, bits, K).astype(np.float32).reshape(N, G, group_size)
    x = np.atleast_2d(np.asarray(x, dtype=np.float32)).reshape(-1, G, group_size)
    qx = np.einsum("ngk,mgk->mng", q, x).astype(np.float32)
    sx = x.sum(axis=-1, dtype=np.float32)
    s = np.asarray(scales, dtype=np.float32)
    b = np.asarray(biases, dtype=np.float32)
    return (qx * s[None] + sx[:, None, :] * b[None]).sum(axis=-1, dtype=np.float32)


# --------------------------------------------------------------------------
# a9: router.  Plain softmax top-k lives in mlx-lm (un-vendored): parity
#     unpinned.  The normalisation form follows dots3/ops.py:159-162.
# --------------------------------------------------------------------------
def route_softmax_topk(logits: np.ndarray, k: int, renorm: bool = True, scale: float = 1.0):
    """(idx int32 [T,k], w f32 [T,k]); ties go to the lower expert id
    (dsv41/metal_decode.py:1141), experts are listed by descending score."""
    z = np.asarray(logits, dtype=np.float32)
    z = z - z.max(axis=-1, keepdims=True)
    p = np.exp(z)
    p = p / p.sum(axis=-1, keepdims=True, dtype=np.float32)
    idx = np.argsort(-p, axis=-1, kind="stable")[:, :k]
    w = np.take_along_axis(p, idx, axis=-1)
    if renorm:
        w = w / (w.sum(axis=-1, keepdims=True, dtype=np.float32) + np.float32(1e-20))
    return idx.astype(np.int32), (w * np.float32(scale)).astype(np.float32)


# --------------------------------------------------------------------------
# a7: routed MoE (gather_qmm semantics)
#   naive loop: dots3/ops_selftest.py:18-27; layer logic dsv41/model.py:1206-1245
#   and dots3/ops.py:195-223
# --------------------------------------------------------------------------
def moe_sort(idx: np.ndarray, num_experts: int):
    """order = stable argsort of the flat expert ids, inv = argsort(order),
    offsets[e] = first sorted row of expert e (dsv41/model.py:1207-1212)."""
    flat = np.asarray(idx).reshape(-1)
    order = np.argsort(flat, kind="stable").astype(np.int32)
    inv = np.argsort(order, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=num_experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return order, inv, offsets


def gather_qmm(x, packed, scales, biases, rhs_indices, bits, group_size, lhs_indices=None):
    """y[r] = x[lhs[r]] . deq(W[rhs[r]])^T  (dots3/ops.py:168-192 call shape).
    x [R0,K]; packed [E,N,Kp]; rhs_indices [R]; lhs_indices [R] or None (identity)."""
    x = np.asarray(x, dtype=np.float32)
    rhs = np.asarray(rhs_indices).reshape(-1)
    lhs = np.arange(rhs.size) if lhs_indices is None else np.asarray(lhs_indices).reshape(-1)
    E, N, _ = np.asarray(packed).shape
    out = np.zeros((rhs.size, N), np.float32)
    for e in np.unique(rhs):
        rowsel = np.nonzero(rhs == e)[0]
        W = dequantize_affine(packed[e], scales[e], biases[e], bits, group_size)
        out[rowsel] = (x[lhs[rowsel]].astype(np.float64) @ W.astype(np.float64).T).astype(np.float32)
    return out


def _silu(g):
    return g / (1.0 + np.exp(-g))


def moe_layer(x, idx, w, gate, up, down, *, swiglu_limit: float = 0.0, act_dtype: str = "bf16",
              shared=None) -> np.ndarray:
    """Routed-expert SwiGLU layer, float32 result [T,D].

    gate/up/down are tuples (packed[E,N,Kp], scales, biases, bits, group_size).
    Follows dsv41/model.py:1214-1245: gate/up in the activation dtype -> f32,
    optional clamp, h = silu(g)*u*w[t,k] (weight applied before down), h cast to
    the activation dtype, down, f32 sum over the k slots, plus an optional shared
    expert `shared` = (gate, up, down) of 2-D triples (model.py:1237-1245).
    """
    x = round_to(x, act_dtype)
    T, D = x.shape
    k = idx.shape[1]
    flat = np.asarray(idx).reshape(-1)
    lhs = np.repeat(np.arange(T), k)
    g = round_to(gather_qmm(x, *gate[:3], flat, gate[3], gate[4], lhs), act_dtype)
    u = round_to(gather_qmm(x, *up[:3], flat, up[3], up[4], lhs), act_dtype)
    if swiglu_limit > 0:
        u = np.clip(u, -swiglu_limit, swiglu_limit)
        g = np.minimum(g, swiglu_limit)
    h = (_silu(g.astype(np.float32)) * u).astype(np.float32)
    h = h * np.asarray(w, dtype=np.float32).reshape(-1)[:, None]
    h = round_to(h, act_dtype)
    y = round_to(gather_qmm(h, *down[:3], flat, down[3], down[4]), act_dtype)
    out = y.reshape(T, k, D).sum(axis=1, dtype=np.float32)
    if shared is not None:
        sg, su, sd = shared
        g2 = round_to(qmatmul(x, *sg), act_dtype)
        u2 = round_to(qmatmul(x, *su), act_dtype)
        if swiglu_limit > 0:
            u2 = np.clip(u2, -swiglu_limit, swiglu_limit)
            g2 = np.minimum(g2, swiglu_limit)
        h2 = round_to((_silu(g2) * u2).astype(np.float32), act_dtype)
        out = out + round_to(qmatmul(h2, *sd), act_dtype)
    return out.astype(np.float32)


# ---- importance-weighted affine fit (jang_tools/affine.py:279-399) ---------------------------------------------
F16_TINY = np.float32(np.finfo(np.float16).smallest_normal)


def to_f16_nonzero(scale: np.ndarray) -> np.ndarray:
    """float16 cast of a scale that must not become zero (jang_tools/affine.py:44-51): magnitudes below the
    smallest normal float16 become +-that value (a zero counts as positive)."""
    scale = np.asarray(scale)
    safe = np.where(np.abs(scale) < F16_TINY, np.copysign(F16_TINY, np.where(scale == 0, 1.0, scale)), scale)
    return safe.astype(np.float16)


def floor_importance(importance: np.ndarray) -> np.ndarray:
    """jang_tools/affine.py:310-312: importance below 1e-4 of the median positive value (and below 1e-12) is
    raised to that floor, so that no column is ignored entirely."""
    imp = np.asarray(importance, dtype=np.float32)
    positive = imp[imp > 0]
    floor = float(np.median(positive)) * 1e-4 if positive.size else 1.0
    return np.maximum(imp, max(floor, 1e-12))


def quantize_imatrix_affine_codes(w: np.ndarray, importance: np.ndarray, bits: int, group_size: int,
                                  iterations: int = 6):
    """Activation-weighted affine fit, jang_tools/affine.py:279-399: per group, start from the min/max grid,
    then `iterations` rounds of (weighted least squares for scale and bias given the codes; re-round the
    codes), all in float64 with sums over the group in numpy's order; store float16 sidecars (scale kept
    non-zero) and derive the final codes from the STORED sidecars in float32.  Returns (codes uint8 [rows, K],
    scales f16 [rows, G], biases f16 [rows, G], relative weighted error)."""
    matrix = np.asarray(w, dtype=np.float32)
    rows, K = matrix.shape
    G = K // group_size
    imp = floor_importance(importance)
    h = imp.reshape(1, G, group_size).astype(np.float64)
    bins = float((1 << bits) - 1)
    grouped = matrix.reshape(rows, G, group_size)
    low = grouped.min(axis=-1).astype(np.float64)
    high = grouped.max(axis=-1).astype(np.float64)
    scale = np.maximum((high - low) / bins, 1e-8)
    bias = low
    codes = np.clip(np.rint((grouped - bias[..., None]) / scale[..., None]), 0, bins).astype(np.float64)
    values = grouped.astype(np.float64)
    sum_h = np.sum(h, axis=-1)
    sum_hw = np.sum(h * values, axis=-1)
    for _ in range(iterations):
        sum_hq = np.sum(h * codes, axis=-1)
        sum_hq2 = np.sum(h * codes * codes, axis=-1)
        sum_hqw = np.sum(h * codes * values, axis=-1)
        det = sum_h * sum_hq2 - sum_hq * sum_hq
        fitted_scale = np.divide(sum_h * sum_hqw - sum_hq * sum_hw, det, out=scale.copy(), where=np.abs(det) > 1e-20)
        fitted_bias = (sum_hw - fitted_scale * sum_hq) / sum_h
        valid = np.isfinite(fitted_scale) & (np.abs(fitted_scale) >= 1e-8)
        scale = np.where(valid, fitted_scale, scale)
        bias = np.where(valid, fitted_bias, bias)
        codes = np.clip(np.rint((values - bias[..., None]) / scale[..., None]), 0, bins)
    scale_f16 = to_f16_nonzero(scale)
    bias_f16 = bias.astype(np.float16)
    ss, sb = scale_f16.astype(np.float32), bias_f16.astype(np.float32)
    codes_u8 = np.clip(np.rint((grouped - sb[..., None]) / ss[..., None]), 0, bins).astype(np.uint8)
    rec = codes_u8.astype(np.float32) * ss[..., None] + sb[..., None]
    err = float(np.sum(h * np.square(rec - grouped), dtype=np.float64))
    ref = float(np.sum(h * np.square(grouped), dtype=np.float64))
    return codes_u8.reshape(rows, K), scale_f16, bias_f16, float(np.sqrt(err / max(ref, 1e-30)))


def quantize_imatrix_affine(w, importance, bits, group_size, iterations: int = 6):
    """Packed form: (uint32 [rows, K*bits/32], scales f16, biases f16, relative weighted error)."""
    codes, s, b, e = quantize_imatrix_affine_codes(w, importance, bits, group_size, iterations)
    return pack_rows(codes, bits), s, b, e


# ---- randomized Hadamard rotation (jang_tools/turboquant/rotation.py:17-113) ----------------------------------
# The reference module needs MLX to import, so this restatement is checked against an explicit Hadamard matrix
# (scipy) and the rotation's defining property instead of reference outputs: parity unpinned for the bit
# pattern of the float32 results, pinned for the mathematics.
def pow2_blocks(dim: int) -> list[int]:
    """dim as a sum of distinct powers of two, largest first (rotation.py:26-40): 192 -> [128, 64]."""
    blocks, rem = [], int(dim)
    while rem > 0:
        p = 1 << (rem.bit_length() - 1)
        blocks.append(p)
        rem -= p
    return blocks


def hadamard_signs(dim: int, seed: int = 0) -> np.ndarray:
    """+-1 signs of the randomized transform (rotation.py:43-59): numpy's default_rng(seed).choice."""
    return np.random.default_rng(seed).choice([-1.0, 1.0], size=dim).astype(np.float32)


def _fwht_f32(x: np.ndarray) -> np.ndarray:
    """Unnormalised Walsh-Hadamard butterflies along the last axis in float32, block size h = 1, 2, 4, ...:
    (a, b) -> (a + b, a - b) for the two halves of every run of 2h elements, then * float32(1/sqrt(d))
    (rotation.py:62-83)."""
    x = np.array(x, dtype=np.float32)
    d = x.shape[-1]
    h = 1
    while h < d:
        y = x.reshape(x.shape[:-1] + (d // (2 * h), 2, h))
        a, b = y[..., 0, :], y[..., 1, :]
        x = np.concatenate([a + b, a - b], axis=-1).reshape(x.shape[:-1] + (d,))
        h *= 2
    return x * np.float32(1.0 / (d ** 0.5))


def hadamard_rotate(x: np.ndarray, signs: np.ndarray) -> np.ndarray:
    """H * diag(signs) * x per power-of-two block of the last axis (rotation.py:86-113), float32."""
    x = np.asarray(x, dtype=np.float32)
    parts, off = [], 0
    for b in pow2_blocks(x.shape[-1]):
        parts.append(_fwht_f32(x[..., off:off + b] * signs[off:off + b]))
        off += b
    return np.concatenate(parts, axis=-1)


def hadamard_inverse(y: np.ndarray, signs: np.ndarray) -> np.ndarray:
    """signs * H * y per block (rotation.py:116-140)."""
    y = np.asarray(y, dtype=np.float32)
    parts, off = [], 0
    for b in pow2_blocks(y.shape[-1]):
        parts.append(_fwht_f32(y[..., off:off + b]) * signs[off:off + b])
        off += b
    return np.concatenate(parts, axis=-1)


# ---- JANGTQ: rotated codebook weights (jang_tools/turboquant/linear.py:24-60,137-200, codebook.py:27-102,
#      pipeline.py:32-53; kernels jang-runtime/Sources/JANGCoreMetal/JANGTQMatmul.metal:154-363) -------------
# Storage: packed uint32 [.., out, in / (32 // bits)] holding 32 // bits codebook indices per word, LSB first
# (3-bit: 10 per word, the top 2 bits unused -- NOT the affine codec's continuous bitstream), one float16 norm
# per row, one codebook of 2^bits float32 centroids per (in_features, bits), one +-1 sign vector per
# in_features.  y[out] = norm[out] * sum_i codebook[idx[out, i]] * rot(x)[i],  rot = H * diag(signs).
# Parity unpinned for everything that runs through MLX in the reference (rotation, norms, index choice);
# compute_codebook is plain numpy there and is pinned by tests/golden/tq_codebooks.json.
def tq_codebook(dim: int, bits: int, n_iter: int = 200) -> np.ndarray:
    """Lloyd-Max centroids for a coordinate of a random unit vector in `dim` dimensions
    (codebook.py:27-102): density (1 - x^2)^((dim - 3) / 2) on a 10000-point grid over [-1, 1], centroids
    started uniformly on +-3/sqrt(dim), conditional means by the trapezoid rule until they move < 1e-10."""
    import math
    if bits < 1:
        return np.array([0.0])
    n = 1 << bits
    grid = np.linspace(-1.0, 1.0, 10000)
    if dim <= 2:
        pdf = np.ones_like(grid) * 0.5
    else:
        logc = math.lgamma(dim / 2.0) - 0.5 * math.log(math.pi) - math.lgamma((dim - 1) / 2.0)
        pdf = np.exp(logc + (dim - 3) / 2.0 * np.log(np.maximum(1.0 - grid ** 2, 1e-30)))
    trap = getattr(np, "trapezoid", getattr(np, "trapz", None))
    total = trap(pdf, grid)
    if total > 0:
        pdf = pdf / total
    cent = np.linspace(-3.0 / np.sqrt(max(dim, 1)), 3.0 / np.sqrt(max(dim, 1)), n)
    for _ in range(n_iter):
        edges = np.concatenate([[-1.0], (cent[:-1] + cent[1:]) / 2.0, [1.0]])
        new = np.zeros(n)
        for i in range(n):
            m = (grid >= edges[i]) & ((grid <= edges[i + 1]) if i == n - 1 else (grid < edges[i + 1]))
            if m.sum() <= 1:
                new[i] = cent[i]
                continue
            new[i] = trap(grid[m] * pdf[m], grid[m]) / max(trap(pdf[m], grid[m]), 1e-10)
        if np.allclose(cent, new, atol=1e-10):
            break
        cent = new
    return np.array(sorted(cent.tolist()))


def tq_pack(idx: np.ndarray, bits: int) -> np.ndarray:
    """[rows, K] indices -> uint32 [rows, K / (32 // bits)] (pipeline.py:32-53; K a multiple of 32 // bits)."""
    per = 32 // bits
    rows, K = idx.shape
    v = idx.astype(np.uint32).reshape(rows, K // per, per)
    out = np.zeros((rows, K // per), np.uint32)
    for i in range(per):
        out |= v[:, :, i] << np.uint32(i * bits)
    return out


def tq_unpack(packed: np.ndarray, bits: int, K: int) -> np.ndarray:
    per = 32 // bits
    p = np.asarray(packed, dtype=np.uint32)
    shifts = (np.arange(per) * bits).astype(np.uint32)
    idx = (p[..., None] >> shifts) & np.uint32((1 << bits) - 1)
    return idx.reshape(p.shape[:-1] + (-1,))[..., :K].astype(np.uint8)


def tq_quantize(w: np.ndarray, bits: int, seed: int = 42):
    """(packed, norms float16, codebook float32, signs float32) of a [out, in] matrix
    (linear.py:137-178): rotate the rows, take their L2 norms (floored at 1e-10), normalise, and count for every
    element the boundaries (midpoints of neighbouring centroids) it exceeds.  float32 throughout."""
    w = np.asarray(w, dtype=np.float32)
    K = w.shape[1]
    signs = np.random.default_rng(seed).choice([-1.0, 1.0], size=K).astype(np.float32)
    wr = hadamard_rotate(w, signs)
    norms = np.sqrt((wr * wr).sum(axis=1, keepdims=True, dtype=np.float32))
    wn = wr / np.maximum(norms, np.float32(1e-10))
    cb = tq_codebook(K, bits).astype(np.float32)
    edges = ((cb[:-1] + cb[1:]) / np.float32(2.0)).astype(np.float32)
    idx = np.zeros(wn.shape, np.uint8)
    for e in edges:
        idx += (wn > e).astype(np.uint8)
    return tq_pack(idx, bits), norms[:, 0].astype(np.float16), cb, signs


def tq_dequantize(packed, norms, codebook, signs, bits: int) -> np.ndarray:
    """The float32 matrix TurboQuantLinear multiplies by (linear.py:51-56): codebook[idx] * norm, rotated back."""
    K = signs.shape[0]
    w = np.asarray(codebook, np.float32)[tq_unpack(packed, bits, K)] * np.asarray(norms, np.float32)[:, None]
    return hadamard_inverse(w, signs)


def tq_matmul_rotated(x_rot, packed, norms, codebook, bits: int) -> np.ndarray:
    """y[m, out] = norm[out] * sum_i codebook[idx[out, i]] * x_rot[m, i] in float64 (JANGTQMatmul.metal:18-30)."""
    x_rot = np.atleast_2d(np.asarray(x_rot, np.float64))
    K = x_rot.shape[1]
    W = np.asarray(codebook, np.float64)[tq_unpack(packed, bits, K)]
    return ((x_rot @ W.T) * np.asarray(norms, np.float64)[None, :]).astype(np.float32)


def tq_gather_matmul(x_rot, packed, norms, codebook, rhs, bits: int, x_div: int = 1) -> np.ndarray:
    """out[p] = tq_matmul_rotated(x_rot[p // x_div], expert rhs[p]) (jangtq_gather_tq_matmul, metal:281-363)."""
    rhs = np.asarray(rhs).reshape(-1)
    return np.stack([tq_matmul_rotated(x_rot[p // x_div], packed[e], norms[e], codebook, bits)[0]
                     for p, e in enumerate(rhs)])


def tq_fused_gate_up_swiglu(x_rot, packed_g, norms_g, packed_u, norms_u, codebook, rhs, bits: int, topk: int,
                            swiglu_limit: float = 0.0) -> np.ndarray:
    """out[t * k + j] = silu(min(g, lim)) * clip(u, +-lim) with g, u the gate / up products of token t and its
    j-th expert (jangtq_fused_gate_up_swiglu, metal:154-262)."""
    g = tq_gather_matmul(x_rot, packed_g, norms_g, codebook, rhs, bits, topk).astype(np.float32)
    u = tq_gather_matmul(x_rot, packed_u, norms_u, codebook, rhs, bits, topk).astype(np.float32)
    if swiglu_limit > 0:
        g = np.minimum(g, np.float32(swiglu_limit))
        u = np.clip(u, -np.float32(swiglu_limit), np.float32(swiglu_limit))
    return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
