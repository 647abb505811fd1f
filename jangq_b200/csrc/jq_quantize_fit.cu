// K1 variant: activation-weighted affine fit (jang_tools/affine.py:279-399, quantize_imatrix_affine_numpy).
//
// Per quantization group: start from the min/max grid, then `iterations` rounds of
//   weighted least squares for (scale, bias) given the codes  ->  re-round the codes,
// all in float64, then float16 sidecars (scale kept non-zero) and final codes derived from the STORED
// sidecars in float32.  The result is bit-identical to the numpy reference, which pins three things:
//   * every float64 operation is an explicit round-to-nearest intrinsic (no FMA contraction);
//   * a sum over the group follows numpy's order for a contiguous axis of at most 128 elements: eight
//     running sums over the elements i mod 8, combined as ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)).  Eight lanes
//     own one group, lane j the elements j, j+8, ...; the combine is an xor-shuffle tree over 1, 2, 4;
//   * float64 -> float16 is one rounding (__double2half).
// Bound: float64 arithmetic (about 20 operations per weight and iteration), not HBM: algorithmic bytes are
// rows*K*sizeof(src) read + rows*K*bits/8 + rows*(K/gs)*4 written.
#include <cuda_fp16.h>

#include "jq_common.cuh"

namespace jq {

constexpr int FIT_GROUPS_PER_BLOCK = 32;                 // 256 threads, 8 lanes per group

__device__ __forceinline__ double fit_gsum(double acc) { // acc: this lane's running sum
    acc = __dadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 1));
    acc = __dadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 2));
    acc = __dadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 4));
    return acc;
}

template <typename W, int GS>
__global__ void __launch_bounds__(256)
quantize_fit_kernel(const W* __restrict__ w, const float* __restrict__ importance, int64_t n_groups, int G, int bits,
                    int iterations, uint8_t* __restrict__ codes_bytes, __half* __restrict__ scales,
                    __half* __restrict__ biases) {
    constexpr int PER = GS / 8;
    __shared__ uint8_t sc[FIT_GROUPS_PER_BLOCK * GS];
    const int lg = threadIdx.x >> 3, j = threadIdx.x & 7;
    const int64_t group = (int64_t)blockIdx.x * FIT_GROUPS_PER_BLOCK + lg;
    const bool live = group < n_groups;
    const int64_t gsafe = live ? group : n_groups - 1;   // idle lanes shadow the last group: shuffles stay full-warp
    const int gcol = (int)(gsafe % G);
    const W* wp = w + gsafe * GS;
    const float* hp = importance + (int64_t)gcol * GS;
    const double bins = (double)((1 << bits) - 1);

    float v[PER], h[PER];
    float lo = 3.4028235e38f, hi = -3.4028235e38f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        v[i] = Elt<W>::to_f32(wp[j + 8 * i]);
        h[i] = hp[j + 8 * i];
        lo = fminf(lo, v[i]);
        hi = fmaxf(hi, v[i]);
    }
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
        hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
    }
    double scale = fmax(__ddiv_rn(__dsub_rn((double)hi, (double)lo), bins), 1e-8);
    double bias = (double)lo;
    double c[PER];
    // (v - bias) / scale, correctly rounded, in three operations from the correctly rounded reciprocal r: y0 = RN(t*r),
    // y = RN(y0 + RN(t - y0*scale)*r); the residual is exact in an fma and y0 is within one ulp of the quotient, so y is
    // the rounded quotient (Markstein's theorem; |scale| >= 1e-8 and |t| < 2^129: no overflow or underflow).  rint by
    // adding and removing 1.5 * 2^52 (beyond 2^51 the result is still far outside [0, bins] on the right side).
    auto round_codes = [&]() {
        const double r = __drcp_rn(scale);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const double t = __dsub_rn((double)v[i], bias);
            const double y0 = __dmul_rn(t, r);
            const double y = __fma_rn(__fma_rn(-y0, scale, t), r, y0);
            const double rq = __dsub_rn(__dadd_rn(y, 6755399441055744.0), 6755399441055744.0);
            c[i] = fmin(fmax(rq, 0.0), bins);
        }
    };
    round_codes();
    double a0 = (double)h[0], a1 = __dmul_rn((double)h[0], (double)v[0]);
#pragma unroll
    for (int i = 1; i < PER; ++i) {
        a0 = __dadd_rn(a0, (double)h[i]);
        a1 = __dadd_rn(a1, __dmul_rn((double)h[i], (double)v[i]));
    }
    const double sum_h = fit_gsum(a0), sum_hw = fit_gsum(a1);
    for (int it = 0; it < iterations; ++it) {
        double q0, q1, q2;
        {
            const double t = __dmul_rn((double)h[0], c[0]);
            q0 = t; q1 = __dmul_rn(t, c[0]); q2 = __dmul_rn(t, (double)v[0]);
        }
#pragma unroll
        for (int i = 1; i < PER; ++i) {
            const double t = __dmul_rn((double)h[i], c[i]);
            q0 = __dadd_rn(q0, t);
            q1 = __dadd_rn(q1, __dmul_rn(t, c[i]));
            q2 = __dadd_rn(q2, __dmul_rn(t, (double)v[i]));
        }
        const double sum_hq = fit_gsum(q0), sum_hq2 = fit_gsum(q1), sum_hqw = fit_gsum(q2);
        const double det = __dsub_rn(__dmul_rn(sum_h, sum_hq2), __dmul_rn(sum_hq, sum_hq));
        double fs = scale;
        if (fabs(det) > 1e-20) fs = __ddiv_rn(__dsub_rn(__dmul_rn(sum_h, sum_hqw), __dmul_rn(sum_hq, sum_hw)), det);
        const double fb = __ddiv_rn(__dsub_rn(sum_hw, __dmul_rn(fs, sum_hq)), sum_h);
        if (isfinite(fs) && fabs(fs) >= 1e-8) { scale = fs; bias = fb; }
        round_codes();
    }
    // float16 sidecars; a scale below the smallest normal float16 becomes +-that value (zero counts as positive)
    const double tiny = 6.103515625e-05;
    double sd = scale;
    if (fabs(sd) < tiny) sd = scale < 0.0 ? -tiny : tiny;
    const __half s16 = __double2half(sd), b16 = __double2half(bias);
    const float ss = __half2float(s16), sb = __half2float(b16);
    const float fbins = (float)bins;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const float q = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v[i], sb), ss)), 0.f), fbins);
        sc[lg * GS + j + 8 * i] = (uint8_t)q;
    }
    if (live && j == 0) { scales[group] = s16; biases[group] = b16; }
    __syncthreads();
    // pack: one thread per 8 consecutive codes -> `bits` bytes
    const int octs_block = FIT_GROUPS_PER_BLOCK * GS / 8;
    for (int o = threadIdx.x; o < octs_block; o += blockDim.x) {
        const int64_t goct = (int64_t)blockIdx.x * octs_block + o;
        if (goct * 8 >= n_groups * GS) break;
        unsigned long long word = 0ull;
#pragma unroll
        for (int e = 0; e < 8; ++e) word |= (unsigned long long)sc[o * 8 + e] << (e * bits);
        uint8_t* dst = codes_bytes + goct * bits;
        for (int bte = 0; bte < bits; ++bte) dst[bte] = (uint8_t)(word >> (8 * bte));
    }
}

}  // namespace jq

extern "C" {

int jq_quantize_imatrix(const void* w, int w_dtype, const float* importance, int64_t rows, int64_t K, int bits,
                        int group_size, int iterations, uint32_t* codes, void* scales_f16, void* biases_f16,
                        jq_stream_t stream) {
    using namespace jq;
    int rc = check_quant_shape(rows, K, bits, group_size);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(w_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(iterations > 0 && iterations <= 64, JQ_EINVAL, "iterations must be in 1..64");
    if (rows == 0 || K == 0) return JQ_OK;
    JQ_REQUIRE(w && importance && codes && scales_f16 && biases_f16, JQ_EINVAL, "null pointer");
    const int G = (int)(K / group_size);
    const int64_t n_groups = rows * G;
    const int64_t blocks = (n_groups + FIT_GROUPS_PER_BLOCK - 1) / FIT_GROUPS_PER_BLOCK;
    JQ_REQUIRE(blocks < (1ll << 31), JQ_EUNSUPPORTED, "tensor too large for one launch");
    cudaStream_t st = (cudaStream_t)stream;
#define JQ_FIT_LAUNCH(GSZ)                                                                                    \
    JQ_DISPATCH_DTYPE(w_dtype, W,                                                                             \
        (quantize_fit_kernel<W, GSZ><<<(unsigned)blocks, 256, 0, st>>>((const W*)w, importance, n_groups, G, bits, \
            iterations, (uint8_t*)codes, (__half*)scales_f16, (__half*)biases_f16)))
    if (group_size == 32) { JQ_FIT_LAUNCH(32) }
    else if (group_size == 64) { JQ_FIT_LAUNCH(64) }
    else { JQ_FIT_LAUNCH(128) }
#undef JQ_FIT_LAUNCH
    return check_launch("quantize_imatrix");
}

}  // extern "C"
