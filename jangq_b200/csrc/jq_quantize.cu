// K1: affine group quantizer, its zero-point RTN sibling, and the dequantizer.
//
// All three are streaming kernels bounded by HBM bandwidth: the quantizer reads
// sizeof(T) bytes and writes bits/8 + 2*sizeof(S)/group_size bytes per weight.
// Because K % group_size == 0 and K*bits % 32 == 0, groups and packed words
// never straddle a row, so the kernels walk the tensor as one flat array.
//
// Mapping: one thread owns 16 consecutive weights (one or two 16-byte loads per
// 8 of them), so a group of 32/64/128 weights is 2/4/8 adjacent lanes and the
// min/max reduction is 1-3 xor-shuffles.  16 codes of `bits` bits are 2*bits
// bytes: whole words for 2/4/6/8 bits; for 3/5 bits two adjacent lanes exchange
// 16 bits so that every store is a whole 32-bit word.
//
// Arithmetic follows the reference line by line with IEEE round-to-nearest
// intrinsics so that no FMA contraction or approximate division can change a
// code (jang_tools/affine.py:227-252).  The per-weight division has a fast
// path: t*rcp(scale) differs from the correctly rounded quotient by less than
// 2^-23*|q| <= 3.1e-5 for |q| <= 257, so rint() of both agree unless the
// quotient lies within that distance of a half-integer; values within 1e-3 of one
// (1 in 500; one warp instruction in 16 has such a lane) are recomputed with the
// exact division.
#include "jq_common.cuh"

namespace jq {

enum { MODE_AFFINE = 0, MODE_RTN = 1 };

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 f = __ldg(q + i);
        v[4 * i + 0] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
}
template <>
__device__ __forceinline__ void load16<__half>(const __half* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 u = __ldg(q + i);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            v[8 * i + 2 * j] = f.x; v[8 * i + 2 * j + 1] = f.y;
        }
    }
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 u = __ldg(q + i);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
}

// Store the 16 codes of one lane (2*BITS bytes) as whole words.  `chunk` is the
// lane's flat 16-weight chunk index; lanes of an even/odd pair cooperate for odd
// widths.  All lanes of the warp must call this (it shuffles).
template <int BITS>
__device__ __forceinline__ void store_codes(uint32_t* __restrict__ codes, int64_t chunk, const uint32_t (&q)[16],
                                            bool valid) {
    uint32_t out[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int pos = j * BITS, wd = pos >> 5, sh = pos & 31;
        out[wd] |= q[j] << sh;
        if (sh + BITS > 32) out[wd + 1] |= q[j] >> (32 - sh);
    }
    if constexpr (BITS == 2) {
        if (valid) codes[chunk] = out[0];
    } else if constexpr (BITS == 4) {
        if (valid) *reinterpret_cast<uint2*>(codes + 2 * chunk) = make_uint2(out[0], out[1]);
    } else if constexpr (BITS == 8) {
        if (valid) *reinterpret_cast<uint4*>(codes + 4 * chunk) = make_uint4(out[0], out[1], out[2], out[3]);
    } else if constexpr (BITS == 6) {
        if (valid) {
            uint32_t* p = codes + 3 * chunk;
            p[0] = out[0]; p[1] = out[1]; p[2] = out[2];
        }
    } else if constexpr (BITS == 3) {
        // 48 bits per lane; an (even, odd) lane pair makes 3 words
        const uint32_t partner_lo = __shfl_down_sync(0xFFFFFFFFu, out[0], 1);
        if (valid) {
            uint32_t* p = codes + 3 * (chunk >> 1);
            if ((chunk & 1) == 0) {
                p[0] = out[0];
                p[1] = (out[1] & 0xFFFFu) | (partner_lo << 16);
            } else {
                p[2] = (out[0] >> 16) | (out[1] << 16);
            }
        }
    } else {  // BITS == 5: 80 bits per lane; a lane pair makes 5 words
        const uint32_t partner_lo = __shfl_down_sync(0xFFFFFFFFu, out[0], 1);
        if (valid) {
            uint32_t* p = codes + 5 * (chunk >> 1);
            if ((chunk & 1) == 0) {
                p[0] = out[0];
                p[1] = out[1];
                p[2] = (out[2] & 0xFFFFu) | (partner_lo << 16);
            } else {
                p[3] = (out[0] >> 16) | (out[1] << 16);
                p[4] = (out[1] >> 16) | (out[2] << 16);
            }
        }
    }
}

template <typename T, typename S, int BITS, int MODE>
__global__ void __launch_bounds__(256)
quantize_kernel(const T* __restrict__ w, uint32_t* __restrict__ codes, S* __restrict__ scales,
                S* __restrict__ biases, int64_t n_chunks, int lanes_per_group, int flags) {
    const int64_t chunk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = chunk < n_chunks;
    float v[16];
    if (valid) {
        load16<T>(w + chunk * 16, v);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
    }
    float lo = v[0], hi = v[0];
#pragma unroll
    for (int j = 1; j < 16; ++j) { lo = fminf(lo, v[j]); hi = fmaxf(hi, v[j]); }
    for (int d = 1; d < lanes_per_group; d <<= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
        hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
    }
    constexpr float bins = (float)((1 << BITS) - 1);
    uint32_t q[16];
    float scale, bias;
    if constexpr (MODE == MODE_AFFINE) {
        // jang_tools/affine.py:230-250
        hi = fmaxf(hi, 0.0f);
        scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), bins), 1e-7f);
        const bool dom_lo = fabsf(lo) > fabsf(hi);
        scale = dom_lo ? scale : -scale;
        const float edge = dom_lo ? lo : hi;
        const float q0 = rintf(__fdiv_rn(edge, scale));
        bias = 0.0f;
        if (q0 != 0.0f) { scale = __fdiv_rn(edge, q0); bias = edge; }
        const float rcp = __frcp_rn(scale);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float t = __fsub_rn(v[j], bias);
            const float qa = __fmul_rn(t, rcp);
            // rint() and the float->int conversion as one full-rate add: qa + 1.5*2^23 rounds qa to the nearest
            // even-on-ties integer in the low mantissa bits (|qa| < 2^22)
            const float shifted = __fadd_rn(qa, 12582912.0f);
            const float ra = __fsub_rn(shifted, 12582912.0f);
            if (fabsf(qa - ra) < 0.499f) {
                const int qi = __float_as_int(shifted) - 0x4B400000;
                q[j] = (uint32_t)min(max(qi, 0), (int)bins);
            } else {
                float r = rintf(__fdiv_rn(t, scale));
                r = fmaxf(fminf(r, bins), 0.0f);  // NaN -> 0
                q[j] = (uint32_t)(int)r;
            }
        }
        if ((flags & JQ_QUANT_F16_TINY_GUARD) && Elt<S>::id == JQ_F16) {
            const float tiny = 6.103515625e-05f;  // smallest normal float16 (affine.py:43)
            if (fabsf(scale) < tiny) scale = copysignf(tiny, scale == 0.0f ? 1.0f : scale);
        }
    } else {
        // jang_tools/quantize.py:148-205 (standard min/max RTN branch)
        const bool is_const = (hi == lo);
        const float range = is_const ? 1.0f : __fsub_rn(hi, lo);
        scale = __fdiv_rn(range, bins);
        float zero = fminf(fmaxf(rintf(__fdiv_rn(-lo, scale)), 0.0f), bins);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float r = rintf(__fadd_rn(__fdiv_rn(v[j], scale), zero));
            r = fmaxf(fminf(r, bins), 0.0f);
            q[j] = is_const ? 0u : (uint32_t)(int)r;
        }
        if (is_const) { scale = 1.0f; zero = 0.0f; }
        bias = __fmul_rn(-scale, zero);           // quantize.py:279
    }
    store_codes<BITS>(codes, chunk, q, valid);
    if (valid && (threadIdx.x & (lanes_per_group - 1)) == 0) {
        const int64_t g = chunk / lanes_per_group;
        scales[g] = Elt<S>::from_f32(scale);
        biases[g] = Elt<S>::from_f32(bias);
    }
}

template <int MODE>
static int launch_quantize(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int gs, int sidecar_dtype,
                           int flags, uint32_t* codes, void* scales, void* biases, cudaStream_t st) {
    int rc = check_quant_shape(rows, K, bits, gs);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(w_dtype) && valid_dtype(sidecar_dtype), JQ_EINVAL, "bad dtype");
    const int64_t n = rows * K;
    if (n == 0) return JQ_OK;
    JQ_REQUIRE(w && codes && scales && biases, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(aligned(w, 16) && aligned(codes, 16), JQ_EINVAL, "w and codes must be 16-byte aligned");
    const int64_t n_chunks = n / 16;
    const int threads = 256;
    const int64_t blocks = (n_chunks + threads - 1) / threads;
    JQ_REQUIRE(blocks < (1ll << 31), JQ_EUNSUPPORTED, "tensor too large for one launch (%lld weights)", (long long)n);
    const int lpg = gs / 16;
    JQ_DISPATCH_DTYPE(w_dtype, T,
        JQ_DISPATCH_DTYPE(sidecar_dtype, S,
            JQ_DISPATCH_BITS(bits, B,
                (quantize_kernel<T, S, B, MODE><<<(unsigned)blocks, threads, 0, st>>>(
                    (const T*)w, codes, (S*)scales, (S*)biases, n_chunks, lpg, flags)))))
    return check_launch("quantize");
}

// ---- dequantizer ---------------------------------------------------------------
// One thread produces 8 consecutive weights (BITS bytes of codes, at most 3 words).
template <typename S, typename O, int BITS>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint32_t* __restrict__ codes, const S* __restrict__ scales, const S* __restrict__ biases,
                  O* __restrict__ out, int64_t n_oct, int64_t n_words, int gs_shift /* log2(gs/8) */) {
    const int64_t oct = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (oct >= n_oct) return;
    const int64_t byte0 = oct * BITS;
    const int64_t w0 = byte0 >> 2;
    const int sh = (int)(byte0 & 3) * 8;
    const uint32_t a = __ldg(codes + w0);
    const uint32_t b = (w0 + 1 < n_words) ? __ldg(codes + w0 + 1) : 0u;
    const uint32_t c = (BITS > 4 && w0 + 2 < n_words) ? __ldg(codes + w0 + 2) : 0u;
    // 64 bits of the stream starting at this thread's first code
    const uint32_t lo = __funnelshift_r(a, b, sh);
    const uint32_t hi = __funnelshift_r(b, c, sh);
    const unsigned long long bitsv = ((unsigned long long)hi << 32) | lo;
    const int64_t g = oct >> gs_shift;
    const float s = Elt<S>::to_f32(scales[g]);
    const float bs = Elt<S>::to_f32(biases[g]);
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t qv = (uint32_t)(bitsv >> (j * BITS)) & ((1u << BITS) - 1u);
        r[j] = __fadd_rn(__fmul_rn((float)qv, s), bs);   // affine.py:457-463: two roundings
    }
    O* o = out + oct * 8;
    if constexpr (sizeof(O) == 4) {
        float4* o4 = reinterpret_cast<float4*>(o);
        o4[0] = make_float4(r[0], r[1], r[2], r[3]);
        o4[1] = make_float4(r[4], r[5], r[6], r[7]);
    } else {
        O tmp[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) tmp[j] = Elt<O>::from_f32(r[j]);
        *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(tmp);
    }
}

// Quantized embedding lookup: out[t] = dequantize(row ids[t]).  Same arithmetic and thread mapping as
// dequantize_kernel, rows taken through ids; an id outside [0, rows) gives a row of zeros.
template <typename S, typename O, int BITS>
__global__ void __launch_bounds__(256)
embedding_kernel(const uint32_t* __restrict__ codes, const S* __restrict__ scales, const S* __restrict__ biases,
                 const int32_t* __restrict__ ids, O* __restrict__ out, int64_t n_oct, int oct_per_row, int words_per_row,
                 int groups_per_row, int64_t rows, int gs_shift) {
    const int64_t oct = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (oct >= n_oct) return;
    const int64_t t = oct / oct_per_row;
    const int o = (int)(oct - t * oct_per_row);
    const int64_t row = ids[t];
    float r[8];
    if (row < 0 || row >= rows) {
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = 0.f;
    } else {
        const uint32_t* cr = codes + row * words_per_row;
        const int byte0 = o * BITS;
        const int w0 = byte0 >> 2;
        const int sh = (byte0 & 3) * 8;
        const uint32_t a = __ldg(cr + w0);
        const uint32_t b = (w0 + 1 < words_per_row) ? __ldg(cr + w0 + 1) : 0u;
        const uint32_t c = (BITS > 4 && w0 + 2 < words_per_row) ? __ldg(cr + w0 + 2) : 0u;
        const uint32_t lo = __funnelshift_r(a, b, sh);
        const uint32_t hi = __funnelshift_r(b, c, sh);
        const unsigned long long bitsv = ((unsigned long long)hi << 32) | lo;
        const int64_t g = row * groups_per_row + (o >> gs_shift);
        const float s = Elt<S>::to_f32(scales[g]);
        const float bs = Elt<S>::to_f32(biases[g]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t qv = (uint32_t)(bitsv >> (j * BITS)) & ((1u << BITS) - 1u);
            r[j] = __fadd_rn(__fmul_rn((float)qv, s), bs);
        }
    }
    O* op = out + oct * 8;
    if constexpr (sizeof(O) == 4) {
        float4* o4 = reinterpret_cast<float4*>(op);
        o4[0] = make_float4(r[0], r[1], r[2], r[3]);
        o4[1] = make_float4(r[4], r[5], r[6], r[7]);
    } else {
        O tmp[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) tmp[j] = Elt<O>::from_f32(r[j]);
        *reinterpret_cast<uint4*>(op) = *reinterpret_cast<const uint4*>(tmp);
    }
}

}  // namespace jq

extern "C" {

int jq_quantize(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int group_size, int sidecar_dtype,
                int flags, uint32_t* codes, void* scales, void* biases, jq_stream_t stream) {
    return jq::launch_quantize<jq::MODE_AFFINE>(w, w_dtype, rows, K, bits, group_size, sidecar_dtype, flags, codes,
                                                scales, biases, (cudaStream_t)stream);
}

int jq_quantize_rtn(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int group_size, int sidecar_dtype,
                    uint32_t* codes, void* scales, void* biases, jq_stream_t stream) {
    return jq::launch_quantize<jq::MODE_RTN>(w, w_dtype, rows, K, bits, group_size, sidecar_dtype, 0, codes, scales,
                                             biases, (cudaStream_t)stream);
}

int jq_dequantize(const uint32_t* codes, const void* scales, const void* biases, int sidecar_dtype, int64_t rows,
                  int64_t K, int bits, int group_size, void* out, int out_dtype, jq_stream_t stream) {
    using namespace jq;
    int rc = check_quant_shape(rows, K, bits, group_size);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(sidecar_dtype) && valid_dtype(out_dtype), JQ_EINVAL, "bad dtype");
    const int64_t n = rows * K;
    if (n == 0) return JQ_OK;
    JQ_REQUIRE(codes && scales && biases && out, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(aligned(out, 16) && aligned(codes, 4), JQ_EINVAL, "out must be 16-byte aligned");
    const int64_t n_oct = n / 8, n_words = n * bits / 32;
    const int threads = 256;
    const int64_t blocks = (n_oct + threads - 1) / threads;
    JQ_REQUIRE(blocks < (1ll << 31), JQ_EUNSUPPORTED, "tensor too large for one launch");
    const int gs_shift = group_size == 32 ? 2 : group_size == 64 ? 3 : 4;
    cudaStream_t st = (cudaStream_t)stream;
    JQ_DISPATCH_DTYPE(sidecar_dtype, S,
        JQ_DISPATCH_DTYPE(out_dtype, O,
            JQ_DISPATCH_BITS(bits, B,
                (dequantize_kernel<S, O, B><<<(unsigned)blocks, threads, 0, st>>>(
                    codes, (const S*)scales, (const S*)biases, (O*)out, n_oct, n_words, gs_shift)))))
    return check_launch("dequantize");
}

int jq_embedding(const int32_t* ids, int64_t T, const uint32_t* codes, const void* scales, const void* biases,
                 int sidecar_dtype, int64_t rows, int64_t K, int bits, int group_size, void* out, int out_dtype,
                 jq_stream_t stream) {
    using namespace jq;
    int rc = check_quant_shape(rows, K, bits, group_size);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(sidecar_dtype) && valid_dtype(out_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(T >= 0, JQ_EINVAL, "bad token count");
    if (T == 0 || K == 0) return JQ_OK;
    JQ_REQUIRE(ids && codes && scales && biases && out, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(aligned(out, 16) && aligned(codes, 4) && K < (1ll << 31), JQ_EINVAL, "out must be 16-byte aligned");
    const int64_t n_oct = T * (K / 8);
    const int threads = 256;
    const int64_t blocks = (n_oct + threads - 1) / threads;
    JQ_REQUIRE(blocks < (1ll << 31), JQ_EUNSUPPORTED, "too many tokens for one launch");
    const int gs_shift = group_size == 32 ? 2 : group_size == 64 ? 3 : 4;
    cudaStream_t st = (cudaStream_t)stream;
    JQ_DISPATCH_DTYPE(sidecar_dtype, S,
        JQ_DISPATCH_DTYPE(out_dtype, O,
            JQ_DISPATCH_BITS(bits, B,
                (embedding_kernel<S, O, B><<<(unsigned)blocks, threads, 0, st>>>(
                    codes, (const S*)scales, (const S*)biases, ids, (O*)out, n_oct, (int)(K / 8), (int)(K * bits / 32),
                    (int)(K / group_size), rows, gs_shift)))))
    return check_launch("embedding");
}

}  // extern "C"
