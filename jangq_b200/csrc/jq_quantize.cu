// K1: affine group quantizer, its zero-point RTN sibling with and without the clip-ratio search, and the
// dequantizer.
//
// Bytes per weight: the quantizers read sizeof(T) and write bits/8 + 2*sizeof(S)/group_size.  Because
// K % group_size == 0 and K*bits % 32 == 0, groups and packed words never straddle a row, so the kernels walk the
// tensor as one flat array.  Arithmetic follows the reference line by line with IEEE round-to-nearest intrinsics so
// that no FMA contraction or approximate division can change a code (jang_tools/affine.py:227-252).
//
// quantize_group_kernel is the product path.  quantize_kernel is the earlier form, selected by JQ_QUANT_IEEE_DIV
// for cross-checks: one thread owns 16 consecutive weights, a group is 2/4/8 adjacent lanes, and the per-weight
// quotient is t*rcp(scale) with a fallback to the IEEE division within 1e-3 of a rounding tie.
#include <type_traits>

#include "jq_common.cuh"
#include "jq_mma.cuh"

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
__device__ __forceinline__ void store_words(uint32_t* __restrict__ codes, int64_t chunk, const uint32_t (&out)[4],
                                            bool valid);

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
    store_words<BITS>(codes, chunk, out, valid);
}

// The 2*BITS bytes of one lane, already packed LSB-first into out[0..], to memory as whole words.
template <int BITS>
__device__ __forceinline__ void store_words(uint32_t* __restrict__ codes, int64_t chunk, const uint32_t (&out)[4],
                                            bool valid) {
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
                r = fmaxf(fminf(r, bins), 0.0f);  // NaN -> bins (fminf returns its other operand)
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

// ---- affine and RTN quantizers: one thread per group, branch-free exact quotient -------------------------------
// The arithmetic of quantize_kernel (above: the form that divides per weight, kept as a cross-check behind
// JQ_QUANT_IEEE_DIV) in half the instructions; the quantizers are bound by instruction issue, not by HBM.
//   * y = RN(t/scale) from the correctly rounded reciprocal in three instructions: y0 = RN(t*r), then
//     y = RN(y0 + RN(t - y0*scale) * r).  The residual is exact in an fma, and with r = RN(1/scale) and y0 within one
//     ulp of the quotient the corrected value is the correctly rounded quotient (Markstein's theorem).  No guard and
//     no branch: with 16-bit sources exact rounding ties are common (weights and group edge sit on a coarse grid, so
//     (w - edge) * q0 / edge is often exactly k + 1/2) and a guarded reciprocal takes its exact-division branch in a
//     large share of warp steps.  Groups whose scale is outside [1e-25, 1e25], where the reciprocal or a residual may
//     leave the normal float32 range, divide per weight instead;
//   * y * 2^-149 is a subnormal whose bit pattern is rint(y) (ties to even) as an integer, negative for negative y;
//     for 2-, 4- and 8-bit codes one cvt.pack.sat then clamps two of them and shifts them into the word being built;
//   * a thread owns a whole group, so the per-group scalars (three IEEE divisions, the reciprocal) are issued once per
//     group and need no shuffles; with 16 weights per lane they were a third of all instructions, computed by each of
//     the 2/4/8 lanes sharing a group.  A CTA of 128 threads copies its 128 consecutive groups into shared memory with
//     coalesced 16-byte asynchronous copies (row pitch = group bytes + 16, an odd number of 16-byte slots, so the
//     per-thread row reads are conflict-free), then every thread walks its own row twice: min/max (on bf16x2 / half2
//     pairs for 16-bit sources: exact), then codes in runs of 32 weights (= BITS whole words);
//   * sidecars leave as consecutive elements of consecutive lanes.
// NaN weights give code `bins`, as the dividing kernel does.
// rint(y), ties to even, as an integer: y * 2^-149 lands on the subnormal grid, whose bit pattern is the integer
// itself (sign in bit 31, so a negative y reads as a negative integer; y >= 2^23 and NaN read as large positive
// ones).  mul.rn.f32 without .ftz keeps subnormal results whatever the compile flags.
__device__ __forceinline__ int rint_bits(float y) {
    int r;
    asm("{\n\t.reg .f32 t;\n\tmul.rn.f32 t, %1, 0f00000001;\n\tmov.b32 %0, t;\n\t}" : "=r"(r) : "f"(y));
    return r;
}

// d = (c << 2*BITS) | sat(a) << BITS | sat(b), each saturated to [0, 2^BITS - 1]
template <int BITS>
__device__ __forceinline__ uint32_t pack_sat2(int a, int b, uint32_t c) {
    uint32_t d;
    if constexpr (BITS == 8) asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else if constexpr (BITS == 4) asm("cvt.pack.sat.u4.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else asm("cvt.pack.sat.u2.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <typename T> struct Vec16;      // 16 bytes of weights
template <> struct Vec16<float> {
    static constexpr int N = 4;
    template <int E> static __device__ __forceinline__ float get(const uint4& u) {
        return __uint_as_float(E == 0 ? u.x : E == 1 ? u.y : E == 2 ? u.z : u.w);
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    template <int E> static __device__ __forceinline__ float get(const uint4& u) {
        const uint32_t wd = (E >> 1) == 0 ? u.x : (E >> 1) == 1 ? u.y : (E >> 1) == 2 ? u.z : u.w;
        return __uint_as_float((E & 1) ? (wd & 0xFFFF0000u) : (wd << 16));
    }
};
template <> struct Vec16<__half> {
    static constexpr int N = 8;
    template <int E> static __device__ __forceinline__ float get(const uint4& u) {
        const uint32_t wd = (E >> 1) == 0 ? u.x : (E >> 1) == 1 ? u.y : (E >> 1) == 2 ? u.z : u.w;
        const __half2 h = *reinterpret_cast<const __half2*>(&wd);
        return (E & 1) ? __high2float(h) : __low2float(h);
    }
};

template <typename T>
__device__ __forceinline__ void row_minmax(const uint8_t* row, int vectors, float& lo, float& hi) {
    if constexpr (sizeof(T) == 4) {
        const float4 f0 = *reinterpret_cast<const float4*>(row);
        lo = fminf(fminf(f0.x, f0.y), fminf(f0.z, f0.w));
        hi = fmaxf(fmaxf(f0.x, f0.y), fmaxf(f0.z, f0.w));
#pragma unroll 4
        for (int i = 1; i < vectors; ++i) {
            const float4 f = *reinterpret_cast<const float4*>(row + 16 * i);
            lo = fminf(fminf(lo, f.x), fminf(fminf(f.y, f.z), f.w));
            hi = fmaxf(fmaxf(hi, f.x), fmaxf(fmaxf(f.y, f.z), f.w));
        }
    } else {
        using P = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
        uint4 u = *reinterpret_cast<const uint4*>(row);
        P l = __hmin2(__hmin2(*reinterpret_cast<P*>(&u.x), *reinterpret_cast<P*>(&u.y)),
                      __hmin2(*reinterpret_cast<P*>(&u.z), *reinterpret_cast<P*>(&u.w)));
        P h = __hmax2(__hmax2(*reinterpret_cast<P*>(&u.x), *reinterpret_cast<P*>(&u.y)),
                      __hmax2(*reinterpret_cast<P*>(&u.z), *reinterpret_cast<P*>(&u.w)));
#pragma unroll 4
        for (int i = 1; i < vectors; ++i) {
            u = *reinterpret_cast<const uint4*>(row + 16 * i);
            l = __hmin2(__hmin2(l, *reinterpret_cast<P*>(&u.x)),
                        __hmin2(__hmin2(*reinterpret_cast<P*>(&u.y), *reinterpret_cast<P*>(&u.z)), *reinterpret_cast<P*>(&u.w)));
            h = __hmax2(__hmax2(h, *reinterpret_cast<P*>(&u.x)),
                        __hmax2(__hmax2(*reinterpret_cast<P*>(&u.y), *reinterpret_cast<P*>(&u.z)), *reinterpret_cast<P*>(&u.w)));
        }
        lo = fminf(__low2float(l), __high2float(l));
        hi = fmaxf(__low2float(h), __high2float(h));
    }
}

template <typename S>
__device__ __forceinline__ void put_sidecar(void* p, int64_t i, float v) {
    reinterpret_cast<S*>(p)[i] = Elt<S>::from_f32(v);
}

// One group: `row` is its GS weights in shared memory, `grp` its index.
template <typename T, int BITS, int GS, int MODE>
__device__ __forceinline__ void quantize_one_group(const uint8_t* row, int64_t grp, uint32_t* __restrict__ codes,
                                                   void* __restrict__ scales, void* __restrict__ biases,
                                                   int sidecar_dtype, int flags) {
    constexpr int ROW = GS * (int)sizeof(T);
    constexpr int VPG = ROW / 16;
    constexpr int WPV = Vec16<T>::N;                  // weights per vector
    constexpr int VPR = 32 / WPV;                     // vectors per run of 32 weights
    constexpr int BINS = (1 << BITS) - 1;

    float lo, hi;
    row_minmax<T>(row, VPG, lo, hi);

    // AFFINE: code = clamp(rint((w - bias) / scale));  RTN: code = clamp(rint(w / scale + zero))
    float scale, bias, zero = 0.0f;
    bool is_const = false;
    if constexpr (MODE == MODE_AFFINE) {
        // jang_tools/affine.py:230-250
        hi = fmaxf(hi, 0.0f);
        scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), (float)BINS), 1e-7f);
        const bool dom_lo = fabsf(lo) > fabsf(hi);
        scale = dom_lo ? scale : -scale;
        const float edge = dom_lo ? lo : hi;
        const float q0 = rintf(__fdiv_rn(edge, scale));
        bias = 0.0f;
        if (q0 != 0.0f) { scale = __fdiv_rn(edge, q0); bias = edge; }
    } else {
        // jang_tools/quantize.py:148-205 (standard min/max branch)
        is_const = (hi == lo);
        scale = __fdiv_rn(is_const ? 1.0f : __fsub_rn(hi, lo), (float)BINS);
        zero = fminf(fmaxf(rintf(__fdiv_rn(-lo, scale)), 0.0f), (float)BINS);
        bias = 0.0f;
    }
    const float rcp = __frcp_rn(scale);
    uint32_t* dst = codes + grp * (GS * BITS / 32);

    if (!(fabsf(scale) > 1e-25f && fabsf(scale) < 1e25f)) {
        // Near the ends of the float32 range the reciprocal or the residual can be subnormal, which is outside
        // what the residual form guarantees: divide per weight, emit words from a bit queue.
        unsigned long long acc = 0ull;
        int fill = 0;
        const T* rw = reinterpret_cast<const T*>(row);
#pragma unroll 1
        for (int j = 0; j < GS; ++j) {
            const float v = Elt<T>::to_f32(rw[j]);
            float r = MODE == MODE_AFFINE ? rintf(__fdiv_rn(__fsub_rn(v, bias), scale))
                                          : rintf(__fadd_rn(__fdiv_rn(v, scale), zero));
            r = fmaxf(fminf(r, (float)BINS), 0.0f);
            acc |= (unsigned long long)(is_const ? 0u : (uint32_t)(int)r) << fill;
            fill += BITS;
            if (fill >= 32) { *dst++ = (uint32_t)acc; acc >>= 32; fill -= 32; }
        }
    } else {
#pragma unroll
        for (int run = 0; run < GS / 32; ++run) {
            uint32_t out[BITS];
#pragma unroll
            for (int i = 0; i < BITS; ++i) out[i] = 0u;
#pragma unroll
            for (int vv = 0; vv < VPR; ++vv) {
                const uint4 u = *reinterpret_cast<const uint4*>(row + (run * VPR + vv) * 16);
                int si[WPV];
                auto one = [&](float val, int e) {
                    const float t = MODE == MODE_AFFINE ? __fsub_rn(val, bias) : val;
                    const float y0 = __fmul_rn(t, rcp);
                    float y = __fmaf_rn(__fmaf_rn(-y0, scale, t), rcp, y0);       // = RN(t / scale)
                    if constexpr (MODE == MODE_RTN) y = __fadd_rn(y, zero);
                    si[e] = rint_bits(y);
                };
                one(Vec16<T>::template get<0>(u), 0);
                one(Vec16<T>::template get<1>(u), 1);
                one(Vec16<T>::template get<2>(u), 2);
                one(Vec16<T>::template get<3>(u), 3);
                if constexpr (WPV == 8) {
                    one(Vec16<T>::template get<4>(u), 4);
                    one(Vec16<T>::template get<5>(u), 5);
                    one(Vec16<T>::template get<6>(u), 6);
                    one(Vec16<T>::template get<7>(u), 7);
                }
                if constexpr (BITS == 2 || BITS == 4 || BITS == 8) {
                    // two codes per instruction, clamped by its saturation; the last pair goes in first
                    uint32_t part = 0u;
#pragma unroll
                    for (int e = WPV - 2; e >= 0; e -= 2) {
                        part = pack_sat2<BITS>(si[e + 1], si[e], part);
                        if (BITS == 8 && (e & 3) == 0) {         // four 8-bit codes fill a word
                            out[(vv * WPV + e) / 4] = part;
                            part = 0u;
                        }
                    }
                    if constexpr (BITS != 8) {
                        constexpr int span = WPV * BITS;         // bits of this vector: 8, 16 or 32
                        const int pos = vv * span, wd = pos >> 5, sh = pos & 31;
                        out[wd] |= part << sh;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < WPV; ++e) {
                        const uint32_t x = (uint32_t)min(max(si[e], 0), BINS);
                        const int pos = (vv * WPV + e) * BITS, wd = pos >> 5, sh = pos & 31;
                        out[wd] += x << sh;              // disjoint fields: the sum is the OR, in one shift-add
                        if (sh + BITS > 32) out[wd + 1] += x >> (32 - sh);
                    }
                }
            }
            if (is_const) {
#pragma unroll
                for (int i = 0; i < BITS; ++i) out[i] = 0u;
            }
            uint32_t* p = dst + run * BITS;
            if constexpr (BITS == 4) {
                *reinterpret_cast<uint4*>(p) = make_uint4(out[0], out[1], out[2], out[3]);
            } else if constexpr (BITS == 8) {
                reinterpret_cast<uint4*>(p)[0] = make_uint4(out[0], out[1], out[2], out[3]);
                reinterpret_cast<uint4*>(p)[1] = make_uint4(out[4], out[5], out[6], out[7]);
            } else if constexpr (BITS == 2 || BITS == 6) {
#pragma unroll
                for (int i = 0; i < BITS / 2; ++i) reinterpret_cast<uint2*>(p)[i] = make_uint2(out[2 * i], out[2 * i + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < BITS; ++i) p[i] = out[i];
            }
        }
    }
    if constexpr (MODE == MODE_AFFINE) {
        if ((flags & JQ_QUANT_F16_TINY_GUARD) && sidecar_dtype == JQ_F16) {
            const float tiny = 6.103515625e-05f;  // smallest normal float16 (affine.py:43)
            if (fabsf(scale) < tiny) scale = copysignf(tiny, scale == 0.0f ? 1.0f : scale);
        }
    } else {
        if (is_const) { scale = 1.0f; zero = 0.0f; }  // quantize.py:203-205
        bias = __fmul_rn(-scale, zero);               // quantize.py:279
    }
    if (sidecar_dtype == JQ_F16) { put_sidecar<__half>(scales, grp, scale); put_sidecar<__half>(biases, grp, bias); }
    else if (sidecar_dtype == JQ_BF16) { put_sidecar<__nv_bfloat16>(scales, grp, scale); put_sidecar<__nv_bfloat16>(biases, grp, bias); }
    else { put_sidecar<float>(scales, grp, scale); put_sidecar<float>(biases, grp, bias); }
}

// NT tiles of 128 groups per CTA, all requested up front, one commit group each: with two, the second tile is still
// arriving while the first is quantized (a grid of a single wave would otherwise load everywhere, then compute
// everywhere).
template <typename T, int BITS, int GS, int MODE, int NT>
__global__ void __launch_bounds__(128)
quantize_group_kernel(const T* __restrict__ w, uint32_t* __restrict__ codes, void* __restrict__ scales,
                      void* __restrict__ biases, int sidecar_dtype, int64_t n_groups, int flags) {
    constexpr int THREADS = 128;
    constexpr int ROW = GS * (int)sizeof(T);          // bytes of one group
    constexpr int VPG = ROW / 16;                     // 16-byte vectors per group (a power of two)
    constexpr int PITCH = ROW + 16;
    extern __shared__ __align__(16) uint8_t tile[];
    const int tid = threadIdx.x;
    const int64_t g0 = (int64_t)blockIdx.x * (THREADS * NT);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int64_t gt = g0 + t * THREADS;
        const int n_here = (int)max((int64_t)0, min((int64_t)THREADS, n_groups - gt));
        const uint8_t* src = reinterpret_cast<const uint8_t*>(w) + gt * ROW;
        uint8_t* dstt = tile + t * (THREADS * PITCH);
#pragma unroll
        for (int i = 0; i < VPG; ++i) {
            const int v = i * THREADS + tid;
            const int g = v / VPG, c = v % VPG;
            if (g < n_here) cp_async16(dstt + g * PITCH + c * 16, src + (size_t)v * 16);
        }
        cp_async_commit();
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (t == NT - 1) cp_async_wait<0>(); else cp_async_wait<NT - 1>();
        __syncthreads();
        const int64_t grp = g0 + t * THREADS + tid;
        if (grp < n_groups)
            quantize_one_group<T, BITS, GS, MODE>(tile + t * (THREADS * PITCH) + tid * PITCH, grp, codes, scales, biases,
                                                  sidecar_dtype, flags);
    }
}

template <typename T, int BITS, int GS, int MODE, int NT>
static int launch_group_nt(const void* w, uint32_t* codes, void* scales, void* biases, int sidecar_dtype,
                           int64_t n_groups, int flags, cudaStream_t st) {
    constexpr int smem = NT * 128 * (GS * (int)sizeof(T) + 16);
    auto kern = quantize_group_kernel<T, BITS, GS, MODE, NT>;
    if (smem > 48 * 1024) JQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int64_t ctas = (n_groups + 128 * NT - 1) / (128 * NT);
    JQ_REQUIRE(ctas < (1ll << 31), JQ_EUNSUPPORTED, "tensor too large for one launch");
    kern<<<(unsigned)ctas, 128, smem, st>>>((const T*)w, codes, scales, biases, sidecar_dtype, n_groups, flags);
    return JQ_OK;
}

// Two tiles per CTA where both fit 48 KB (>= 6 CTAs per SM) and the grid still fills the GPU twice over; measured on
// bf16 sources at 4 bits: 8192x8192 31.7 -> 30.9 us, group size 32 37.8 -> 32.7 us, but 4096x4096 10.5 -> 11.0 us.
template <typename T, int BITS, int GS, int MODE>
static int launch_group(const void* w, uint32_t* codes, void* scales, void* biases, int sidecar_dtype, int64_t n_groups,
                        int flags, cudaStream_t st) {
    constexpr int tile_bytes = 128 * (GS * (int)sizeof(T) + 16);
    if constexpr (2 * tile_bytes <= 48 * 1024) {
        if (n_groups >= (int64_t)256 * 12 * sm_count())
            return launch_group_nt<T, BITS, GS, MODE, 2>(w, codes, scales, biases, sidecar_dtype, n_groups, flags, st);
    }
    return launch_group_nt<T, BITS, GS, MODE, 1>(w, codes, scales, biases, sidecar_dtype, n_groups, flags, st);
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
    if (!(flags & JQ_QUANT_IEEE_DIV)) {
        const int64_t n_groups = n / gs;
        int rc2 = JQ_OK;
        JQ_DISPATCH_DTYPE(w_dtype, T,
            JQ_DISPATCH_BITS(bits, B,
                (rc2 = gs == 32 ? launch_group<T, B, 32, MODE>(w, codes, scales, biases, sidecar_dtype, n_groups, flags, st)
                     : gs == 64 ? launch_group<T, B, 64, MODE>(w, codes, scales, biases, sidecar_dtype, n_groups, flags, st)
                                : launch_group<T, B, 128, MODE>(w, codes, scales, biases, sidecar_dtype, n_groups, flags, st))))
        if (rc2 != JQ_OK) return rc2;
        return check_launch("quantize");
    }
    JQ_DISPATCH_DTYPE(w_dtype, T,
        JQ_DISPATCH_DTYPE(sidecar_dtype, S,
            JQ_DISPATCH_BITS(bits, B,
                (quantize_kernel<T, S, B, MODE><<<(unsigned)blocks, threads, 0, st>>>(
                    (const T*)w, codes, (S*)scales, (S*)biases, n_chunks, lpg, flags)))))
    return check_launch("quantize");
}

// ---- clip-ratio search (quantize_tensor(method="mse"), jang_tools/quantize.py:153-191) ------------
// For each block the reference tries 20 clip ratios, quantizes the block against the shrunken
// range and keeps the ratio with the least mean squared error.  Its float32 minima are multiplied
// by float64 ratios, so (NumPy >= 2 promotion) every step of the search is float64; this kernel
// does the same arithmetic in the same order, including the order of the error sum, so the winner
// is the reference's winner bit for bit.
//
// Evaluated for all 20 ratios the search is bound by the FP64 pipe (20 x ~10 double operations per
// weight, 384 us for 4096x4096), so a float32 pass first narrows the ratios to those that can still win
// (see the bound at the screening pass) and only those are evaluated in float64.
// Mapping: eight lanes per block, lane k owning the weights i = k (mod 8).  numpy's add.reduce over
// a contiguous row keeps eight running sums over exactly those residue classes and folds them as
// ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)), which is a three-step xor butterfly over the eight lanes.
// The per-ratio scalars (scale, its reciprocal, zero point) are computed once
// per block, ratio r by lane r % 8, and handed round by shuffle.  Every quotient (x/scale per weight, the scale and
// the zero point per ratio) is the correctly rounded one, formed from the correctly rounded reciprocal and one exact
// residual (div_by_rcp) instead of a division.
// linspace(0.7, 1.0, 20) as numpy produces it (start + i*step, last element set to stop)
__constant__ double MSE_RATIOS[20] = {
    0x1.6666666666666p-1, 0x1.6e7bf53896e7cp-1, 0x1.7691840ac7691p-1, 0x1.7ea712dcf7ea7p-1, 0x1.86bca1af286bcp-1,
    0x1.8ed2308158ed2p-1, 0x1.96e7bf53896e8p-1, 0x1.9efd4e25b9efdp-1, 0x1.a712dcf7ea713p-1, 0x1.af286bca1af28p-1,
    0x1.b73dfa9c4b73ep-1, 0x1.bf53896e7bf54p-1, 0x1.c7691840ac769p-1, 0x1.cf7ea712dcf7fp-1, 0x1.d79435e50d794p-1,
    0x1.dfa9c4b73dfaap-1, 0x1.e7bf53896e7c0p-1, 0x1.efd4e25b9efd5p-1, 0x1.f7ea712dcf7eap-1, 0x1.0000000000000p+0};

// RN(a / b) from r = RN(1 / b): y0 = RN(a*r) is within one ulp of the quotient, the residual a - y0*b is exact in an
// fma, and the corrected value rounds to the correctly rounded quotient (Markstein's theorem; no overflow or underflow
// for the magnitudes here: b >= 1e-46, |a| < 2^129).
__device__ __forceinline__ double div_by_rcp(double a, double b, double r) {
    const double y0 = __dmul_rn(a, r);
    return __fma_rn(__fma_rn(-y0, b, a), r, y0);
}

template <typename T, typename S, int BITS, int GS>
__global__ void __launch_bounds__(256)
quantize_mse_kernel(const T* __restrict__ w, uint32_t* __restrict__ codes, S* __restrict__ scales,
                    S* __restrict__ biases, int64_t n_blocks, int64_t n_words, bool screen) {
    constexpr int EPL = GS / 8;                       // weights per lane
    constexpr int L = (1 << BITS) - 1;
    constexpr int WORDS_PER_WARP = 4 * GS * BITS / 32;
    constexpr int NC = 32 / BITS + 2;                 // codes that can touch one 32-bit word
    __shared__ __align__(16) uint8_t stage[8][4 * GS + 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane >> 3, k = lane & 7;
    const int64_t warp_blk = ((int64_t)blockIdx.x * 8 + warp) * 4;
    const int64_t qb = warp_blk + sub;
    const bool valid = qb < n_blocks;

    float xf[EPL];
#pragma unroll
    for (int t = 0; t < EPL; ++t) xf[t] = valid ? Elt<T>::to_f32(w[qb * GS + t * 8 + k]) : 0.0f;
    float lo = xf[0], hi = xf[0];
#pragma unroll
    for (int t = 1; t < EPL; ++t) { lo = fminf(lo, xf[t]); hi = fmaxf(hi, xf[t]); }
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
        hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
    }
    const bool is_const = (hi == lo);                 // quantize.py:151

    // scalars of ratios k, k+8, k+16 (quantize.py:164-172)
    double sc[3], rc[3];
    int zp[3];
#pragma unroll
    for (int s = 0; s < 3; ++s) {
        const int r = s * 8 + k;
        sc[s] = 1.0; rc[s] = 1.0; zp[s] = 0;
        if (r < 20) {
            const double ratio = MSE_RATIOS[r];
            const double c_min = __dmul_rn((double)lo, ratio);
            const double c_max = __dmul_rn((double)hi, ratio);
            double c_range = __dsub_rn(c_max, c_min);
            if (c_range == 0.0) c_range = 1.0;
            sc[s] = div_by_rcp(c_range, (double)L, 1.0 / L);
            rc[s] = __drcp_rn(sc[s]);
            zp[s] = min(max(__double2int_rn(div_by_rcp(-c_min, sc[s], rc[s])), 0), L);
        }
    }

    // Screening pass in float32.  With d = 2^-17 * max|x| the float32 root-mean-square error of a ratio
    // is within d of the float64 one: the reconstruction (q-z)*scale is at most 2*max|x| and carries three
    // float32 roundings (2^-21.7 * max|x| together); a code can differ from the float64 code only where the
    // quotient is within 2^-20 of a tie, which moves |error| by less than 2^-19.5 * max|x|.  So the float64
    // winner has a float32 rms no larger than the float32 minimum plus 2d, and only ratios inside that
    // window (plus 1e-4 relative for the float32 summation) need the exact evaluation below; they are
    // taken in ascending order with the reference's strict comparison.  Blocks whose magnitude would
    // push float32 squares out of range, or that hold a NaN, skip the screen and evaluate all 20.
    unsigned cand = is_const ? 0u : 0xFFFFFu;                  // a constant block's result is fixed (:187-189)
    const float amax = fmaxf(fabsf(lo), fabsf(hi));
    if (screen) {   // warp-uniform: every lane runs the pass (it shuffles), whether or not its block uses the outcome
        float scf[3], rcf[3], m32[3];
#pragma unroll
        for (int s = 0; s < 3; ++s) { scf[s] = (float)sc[s]; rcf[s] = (float)rc[s]; m32[s] = 0.0f; }
#pragma unroll
        for (int s = 0; s < 3; ++s) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                if (s * 8 + kk >= 20) break;
                const int src = (lane & 24) | kk;
                const float scale = __shfl_sync(0xFFFFFFFFu, scf[s], src);
                const float rcp = __shfl_sync(0xFFFFFFFFu, rcf[s], src);
                const float z = (float)__shfl_sync(0xFFFFFFFFu, zp[s], src);
                const float cl = -z, ch = (float)L - z;
                float acc = 0.0f;
#pragma unroll
                for (int t = 0; t < EPL; ++t) {
                    // rint(x/scale) through the 1.5*2^23 add; quotients too large for it clamp correctly anyway
                    const float r = __fsub_rn(fmaf(xf[t], rcp, 12582912.0f), 12582912.0f);
                    const float c = fminf(fmaxf(r, cl), ch);
                    const float e = fmaf(-c, scale, xf[t]);
                    acc = fmaf(e, e, acc);
                }
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 4);
                if (kk == k) m32[s] = acc * (1.0f / GS);
            }
        }
        float mn = fminf(m32[0], m32[1]);
        if (16 + k < 20) mn = fminf(mn, m32[2]);
#pragma unroll
        for (int d = 1; d < 8; d <<= 1) mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, d));
        const float lim = fmaf(sqrtf(mn), 1.0001f, amax * 1.52587890625e-05f);   // rms_min*(1+1e-4) + 2^-16*max|x|
        const float thr = lim * lim * 1.00001f;
        unsigned narrowed = 0u;
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            const unsigned b = __ballot_sync(0xFFFFFFFFu, (s * 8 + k < 20) && (m32[s] <= thr));
            narrowed |= ((b >> (lane & 24)) & 0xFFu) << (8 * s);
        }
        if (!is_const && amax > 1e-15f && amax < 1e15f) cand = narrowed;
    }

    double best = __longlong_as_double(0x7FF0000000000000ll);   // +inf
    double best_scale = 1.0, best_rcp = 1.0;
    int best_zero = 0;
    bool found = false;
    while (__any_sync(0xFFFFFFFFu, cand != 0u)) {
        // each group of eight lanes takes its own next candidate; the loop runs for the longest list
        const bool active = cand != 0u;
        const int r = active ? __ffs(cand) - 1 : 0;
        cand &= cand - 1u;
        const int s = r >> 3, src = (lane & 24) | (r & 7);
        const double scale = __shfl_sync(0xFFFFFFFFu, s == 0 ? sc[0] : s == 1 ? sc[1] : sc[2], src);
        const double rcp = __shfl_sync(0xFFFFFFFFu, s == 0 ? rc[0] : s == 1 ? rc[1] : rc[2], src);
        const int z = __shfl_sync(0xFFFFFFFFu, s == 0 ? zp[0] : s == 1 ? zp[1] : zp[2], src);
        const double zd = (double)z;
        double acc = 0.0;
#pragma unroll
        for (int t = 0; t < EPL; ++t) {
            const double x = (double)xf[t];
            const double v = __dadd_rn(div_by_rcp(x, scale, rcp), zd);   // quantize.py:174
            const int qi = min(max(__double2int_rn(v), 0), L);           // :175
            const double e = __dsub_rn(x, __dmul_rn((double)(qi - z), scale));   // :176
            acc = __dadd_rn(acc, __dmul_rn(e, e));
        }
        acc = __dadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 1));
        acc = __dadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 2));
        acc = __dadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 4));
        const double mse = __dmul_rn(acc, 1.0 / GS);          // :178 (division by a power of two)
        if (active && mse < best) { best = mse; best_scale = scale; best_rcp = rcp; best_zero = z; found = true; }   // :181-185
    }
    if (is_const || !found) { best_scale = 1.0; best_rcp = 1.0; best_zero = 0; }   // :187-189, and the initial values of :158-160

    // codes of the winning ratio, staged so that each lane can assemble whole words
    uint8_t* st = stage[warp];
#pragma unroll
    for (int t = 0; t < EPL; ++t) {
        int qi = 0;
        if (!is_const && found) {
            const double v = __dadd_rn(div_by_rcp((double)xf[t], best_scale, best_rcp), (double)best_zero);
            qi = min(max(__double2int_rn(v), 0), L);
        }
        st[sub * GS + t * 8 + k] = (uint8_t)qi;
    }
    __syncwarp();
    const int64_t word0 = warp_blk * (GS * BITS / 32);
    for (int wi = lane; wi < WORDS_PER_WARP; wi += 32) {
        if (word0 + wi >= n_words) break;
        const int p = 32 * wi, c = p / BITS, o = p - c * BITS;
        unsigned long long acc = 0ull;
#pragma unroll
        for (int j = 0; j < NC; ++j) acc |= (unsigned long long)st[c + j] << (j * BITS);   // bits past o+32 are dropped
        codes[word0 + wi] = (uint32_t)(acc >> o);
    }
    if (valid && k == 0) {
        const float sf = __double2float_rn(best_scale);           // :184 (float32 array)
        scales[qb] = Elt<S>::from_f32(sf);                        // :281-282
        biases[qb] = Elt<S>::from_f32(__fmul_rn(-sf, (float)best_zero));
    }
}

static int launch_quantize_mse(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int gs, int sidecar_dtype,
                               int flags, uint32_t* codes, void* scales, void* biases, cudaStream_t st) {
    int rc = check_quant_shape(rows, K, bits, gs);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(w_dtype) && valid_dtype(sidecar_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(bits <= 4, JQ_EINVAL, "the clip-ratio search covers 2, 3 and 4 bits");
    const int64_t n = rows * K;
    if (n == 0) return JQ_OK;
    JQ_REQUIRE(w && codes && scales && biases, JQ_EINVAL, "null pointer");
    const int64_t n_blocks = n / gs, n_words = n * bits / 32;
    const int64_t ctas = (n_blocks + 31) / 32;
    JQ_REQUIRE(ctas < (1ll << 31), JQ_EUNSUPPORTED, "tensor too large for one launch (%lld weights)", (long long)n);
#define JQ_MSE_GS(G)                                                                                        \
    JQ_DISPATCH_DTYPE(w_dtype, T,                                                                           \
        JQ_DISPATCH_DTYPE(sidecar_dtype, S,                                                                 \
            JQ_DISPATCH_BITS(bits, B,                                                                       \
                if constexpr (B <= 4) {                                                                     \
                    quantize_mse_kernel<T, S, B, G><<<(unsigned)ctas, 256, 0, st>>>(                        \
                        (const T*)w, codes, (S*)scales, (S*)biases, n_blocks, n_words,                      \
                        !(flags & JQ_QUANT_MSE_EXHAUSTIVE));                                                \
                })))
    if (gs == 32) { JQ_MSE_GS(32); }
    else if (gs == 64) { JQ_MSE_GS(64); }
    else { JQ_MSE_GS(128); }
#undef JQ_MSE_GS
    return check_launch("quantize_mse");
}

// ---- dequantizer ---------------------------------------------------------------
// One thread produces four runs of 8 consecutive weights (BITS bytes of codes, inside two words), 256 runs
// apart, and issues the loads of all four before it converts any: a thread that reads 4 bytes of codes per
// 16 bytes it writes keeps too little in flight to cover the read latency (8 KB per SM at full occupancy).
constexpr int DEQ_UNROLL = 4;

template <typename S, typename O, int BITS>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint32_t* __restrict__ codes, const S* __restrict__ scales, const S* __restrict__ biases,
                  O* __restrict__ out, int64_t n_oct, int64_t n_words, int gs_shift /* log2(gs/8) */) {
    const int64_t oct0 = (int64_t)blockIdx.x * (256 * DEQ_UNROLL) + threadIdx.x;
    uint32_t a[DEQ_UNROLL], b[DEQ_UNROLL];
    float s[DEQ_UNROLL], bs[DEQ_UNROLL];
#pragma unroll
    for (int u = 0; u < DEQ_UNROLL; ++u) {
        const int64_t oct = oct0 + u * 256;
        a[u] = b[u] = 0u;
        s[u] = bs[u] = 0.f;
        if (oct < n_oct) {
            const int64_t w0 = (oct * BITS) >> 2;
            a[u] = __ldg(codes + w0);
            // the run starts at byte (oct * BITS) & 3 of a[u]; its 8 * BITS bits end inside a[u] for 2 and 4 bits
            // (start 0 or 2, 16 or 32 bits) and inside b[u] for every other width (at most 24 + 40 bits)
            if (BITS != 2 && BITS != 4 && w0 + 1 < n_words) b[u] = __ldg(codes + w0 + 1);
            const int64_t g = oct >> gs_shift;
            s[u] = Elt<S>::to_f32(scales[g]);
            bs[u] = Elt<S>::to_f32(biases[g]);
        }
    }
#pragma unroll
    for (int u = 0; u < DEQ_UNROLL; ++u) {
        const int64_t oct = oct0 + u * 256;
        if (oct >= n_oct) continue;
        const int sh = (int)((oct * BITS) & 3) * 8;
        // 64 bits of the stream starting at this run's first code
        const uint32_t lo = __funnelshift_r(a[u], b[u], sh);
        const uint32_t hi = b[u] >> sh;
        const unsigned long long bitsv = ((unsigned long long)hi << 32) | lo;
        float r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t qv = (uint32_t)(bitsv >> (j * BITS)) & ((1u << BITS) - 1u);
            r[j] = __fadd_rn(__fmul_rn((float)qv, s[u]), bs[u]);   // affine.py:457-463: two roundings
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
                    int flags, uint32_t* codes, void* scales, void* biases, jq_stream_t stream) {
    return jq::launch_quantize<jq::MODE_RTN>(w, w_dtype, rows, K, bits, group_size, sidecar_dtype, flags, codes, scales,
                                             biases, (cudaStream_t)stream);
}

int jq_quantize_mse(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int group_size, int sidecar_dtype,
                    int flags, uint32_t* codes, void* scales, void* biases, jq_stream_t stream) {
    // quantize.py:153: widths above 4 bits skip the search and take the min/max branch
    if (bits > 4)
        return jq::launch_quantize<jq::MODE_RTN>(w, w_dtype, rows, K, bits, group_size, sidecar_dtype, flags, codes, scales,
                                                 biases, (cudaStream_t)stream);
    return jq::launch_quantize_mse(w, w_dtype, rows, K, bits, group_size, sidecar_dtype, flags, codes, scales, biases,
                                   (cudaStream_t)stream);
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
    const int64_t blocks = (n_oct + threads * jq::DEQ_UNROLL - 1) / (threads * jq::DEQ_UNROLL);
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
