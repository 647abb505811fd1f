// JANGTQ: rotated codebook weights as an alternate dequantization functor of the gather mat-vec
// (jang-runtime/Sources/JANGCoreMetal/JANGTQMatmul.metal:154-363, jang_tools/turboquant/linear.py:24-200).
//
//     y[p, out] = norm[e_p, out] * sum_i codebook[idx[e_p, out, i]] * x_rot[row(p), i]
//
// with x_rot = H * diag(signs) * x (jq_hadamard_rotate), idx packed 32 / bits per uint32 word (LSB first; 3-bit
// words hold 10 indices and leave 2 bits unused), norms float16, codebook 2^bits float32 centroids.
// Three entry points: the gather mat-vec (down projection: every pair has its own activation row), the
// fused gate/up + SwiGLU of the routed experts, and the weight quantizer (row norms, boundary counts, packing).
//
// Bound: HBM bandwidth on paper (bits / 8 bytes per weight); this first form is a SIMT look-up kernel
// (extract, table load, FMA per weight and row: about 4 instructions per weight), i.e. instruction-bound at
// roughly a tenth of the HBM rate for 2-bit codes.  A warp owns four output rows so that every activation
// read from shared memory is used four times (eight in the fused form: gate and up).
#include "jq_common.cuh"

namespace jq {
namespace tq {

constexpr int WARPS = 8;
constexpr int RPW = 4;                // output rows per warp
constexpr int ROWS = WARPS * RPW;     // output rows per CTA

// x of one pair in shared memory, word-major with one float of padding per packed word, so that the lanes
// of a warp (consecutive words) read position k of their words from distinct banks
__device__ __forceinline__ int xs_index(int word, int k, int per) { return word * (per + 1) + k; }

template <int BITS, bool FUSED>
__global__ void __launch_bounds__(WARPS * 32)
tq_matvec_kernel(const float* __restrict__ x_rot, int64_t ldx, int x_div, const int32_t* __restrict__ rhs,
                 const uint32_t* __restrict__ packed_a, const __half* __restrict__ norms_a,
                 const uint32_t* __restrict__ packed_b, const __half* __restrict__ norms_b,
                 const float* __restrict__ codebook, int num_experts, int N, int K, int words, float limit,
                 float* __restrict__ out, int64_t ldo) {
    constexpr int PER = 32 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    extern __shared__ float sm[];
    float* cb = sm;                               // [2^BITS]
    float* xs = sm + (1 << BITS);                 // [words * (PER + 1)]
    const int p = blockIdx.y;
    const int e = rhs ? rhs[p] : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * ROWS + warp * RPW;
    if (e < 0 || e >= num_experts) {              // an expert outside the bank: zero rows, as the affine gather does
        for (int r = 0; r < RPW; ++r)
            if (lane == 0 && row0 + r < N) out[(int64_t)p * ldo + row0 + r] = 0.f;
        return;
    }
    for (int i = threadIdx.x; i < (1 << BITS); i += WARPS * 32) cb[i] = codebook[i];
    const float* xr = x_rot + (int64_t)(p / x_div) * ldx;
    for (int i = threadIdx.x; i < K; i += WARPS * 32) xs[xs_index(i / PER, i % PER, PER)] = xr[i];
    for (int i = K + threadIdx.x; i < words * PER; i += WARPS * 32) xs[xs_index(i / PER, i % PER, PER)] = 0.f;
    __syncthreads();
    if (row0 >= N) return;
    const uint32_t* pa = packed_a + ((int64_t)e * N + row0) * words;
    const uint32_t* pb = FUSED ? packed_b + ((int64_t)e * N + row0) * words : nullptr;
    float acc_a[RPW], acc_b[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) { acc_a[r] = 0.f; acc_b[r] = 0.f; }
    for (int w = lane; w < words; w += 32) {
        uint32_t va[RPW], vb[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const bool live = row0 + r < N;
            va[r] = live ? pa[(int64_t)r * words + w] : 0u;
            if constexpr (FUSED) vb[r] = live ? pb[(int64_t)r * words + w] : 0u;
        }
        const float* xw = xs + w * (PER + 1);
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const float xv = xw[k];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                acc_a[r] = fmaf(xv, cb[(va[r] >> (k * BITS)) & MASK], acc_a[r]);
                if constexpr (FUSED) acc_b[r] = fmaf(xv, cb[(vb[r] >> (k * BITS)) & MASK], acc_b[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            acc_a[r] += __shfl_xor_sync(0xFFFFFFFFu, acc_a[r], d);
            if constexpr (FUSED) acc_b[r] += __shfl_xor_sync(0xFFFFFFFFu, acc_b[r], d);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int row = row0 + r;
            if (row >= N) break;
            float v = acc_a[r] * __half2float(norms_a[(int64_t)e * N + row]);
            if constexpr (FUSED) {
                float u = acc_b[r] * __half2float(norms_b[(int64_t)e * N + row]);
                if (limit > 0.f) {
                    v = fminf(v, limit);
                    u = fmaxf(fminf(u, limit), -limit);
                }
                v = (v / (1.0f + __expf(-v))) * u;
            }
            out[(int64_t)p * ldo + row] = v;
        }
    }
}

// One warp per row of the rotated float32 matrix: L2 norm (floored at 1e-10), then for every element the
// number of boundaries it exceeds after normalisation, packed 32 / BITS per word.
template <int BITS>
__global__ void __launch_bounds__(256)
tq_quantize_kernel(const float* __restrict__ w_rot, int64_t rows, int K, int words, const float* __restrict__ edges,
                   uint32_t* __restrict__ packed, __half* __restrict__ norms) {
    constexpr int PER = 32 / BITS;
    constexpr int NE = (1 << BITS) - 1;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* wr = w_rot + row * K;
    float ss = 0.f;
    for (int i = lane; i < K; i += 32) ss = fmaf(wr[i], wr[i], ss);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
    const float nrm = sqrtf(ss);
    const float safe = fmaxf(nrm, 1e-10f);
    if (lane == 0) norms[row] = __float2half_rn(nrm);
    float ed[NE];
#pragma unroll
    for (int i = 0; i < NE; ++i) ed[i] = edges[i];
    for (int w = lane; w < words; w += 32) {
        uint32_t v = 0u;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = w * PER + k;
            if (i < K) {
                const float x = __fdiv_rn(wr[i], safe);
                uint32_t q = 0u;
#pragma unroll
                for (int j = 0; j < NE; ++j) q += x > ed[j] ? 1u : 0u;
                v |= q << (k * BITS);
            }
        }
        packed[row * words + w] = v;
    }
}

static int check_common(int bits, int64_t N, int64_t K) {
    JQ_REQUIRE(bits == 2 || bits == 3 || bits == 4, JQ_EUNSUPPORTED, "JANGTQ codebooks of 2, 3 or 4 bits, got %d", bits);
    JQ_REQUIRE(N >= 0 && K > 0 && N < (1ll << 31) && K < (1 << 20), JQ_EINVAL, "bad shape");
    return JQ_OK;
}

template <bool FUSED>
static int launch_matvec(const float* x_rot, int64_t ldx, int x_div, const int32_t* rhs, int64_t pairs,
                         const uint32_t* pa, const void* na, const uint32_t* pb, const void* nb, const float* codebook,
                         int num_experts, int64_t N, int64_t K, int bits, float limit, float* out, int64_t ldo,
                         cudaStream_t st) {
    int rc = check_common(bits, N, K);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(pairs >= 0 && pairs < 65536, JQ_EINVAL, "fewer than 65536 (token, expert) pairs per call");
    if (pairs == 0 || N == 0) return JQ_OK;
    JQ_REQUIRE(x_rot && pa && na && codebook && out && (!FUSED || (pb && nb)), JQ_EINVAL, "null pointer");
    JQ_REQUIRE(x_div >= 1 && num_experts >= 1 && ldx >= K && ldo >= N, JQ_EINVAL, "bad argument");
    const int per = 32 / bits;
    const int words = (int)((K + per - 1) / per);
    const size_t smem = ((size_t)(1 << bits) + (size_t)words * (per + 1)) * sizeof(float);
    JQ_REQUIRE(smem <= 200 * 1024, JQ_EUNSUPPORTED, "in_features too large for one activation row in shared memory");
    const dim3 grid((unsigned)((N + ROWS - 1) / ROWS), (unsigned)pairs);
#define JQ_TQ_LAUNCH(B)                                                                                          \
    if (bits == B) {                                                                                             \
        if (smem > 48 * 1024)                                                                                    \
            JQ_CUDA_OK(cudaFuncSetAttribute(tq_matvec_kernel<B, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                            200 * 1024));                                                        \
        tq_matvec_kernel<B, FUSED><<<grid, WARPS * 32, smem, st>>>(x_rot, ldx, x_div, rhs, pa, (const __half*)na, pb, \
                                                                   (const __half*)nb, codebook, num_experts, (int)N,  \
                                                                   (int)K, words, limit, out, ldo);              \
    }
    JQ_TQ_LAUNCH(2) JQ_TQ_LAUNCH(3) JQ_TQ_LAUNCH(4)
#undef JQ_TQ_LAUNCH
    return check_launch("tq mat-vec");
}

}  // namespace tq
}  // namespace jq

extern "C" {

int jq_tq_gather_matmul(const float* x_rot, int64_t ldx, int x_div, const int32_t* rhs_indices, int64_t pairs,
                        const uint32_t* packed, const void* norms, const float* codebook, int num_experts, int64_t N,
                        int64_t K, int bits, float* out, int64_t ldo, jq_stream_t stream) {
    return jq::tq::launch_matvec<false>(x_rot, ldx, x_div, rhs_indices, pairs, packed, norms, nullptr, nullptr, codebook,
                                        num_experts, N, K, bits, 0.f, out, ldo, (cudaStream_t)stream);
}

int jq_tq_fused_gate_up_swiglu(const float* x_rot, int64_t ldx, int x_div, const int32_t* rhs_indices, int64_t pairs,
                               const uint32_t* packed_gate, const void* norms_gate, const uint32_t* packed_up,
                               const void* norms_up, const float* codebook, int num_experts, int64_t N, int64_t K,
                               int bits, float swiglu_limit, float* out_act, int64_t ldo, jq_stream_t stream) {
    return jq::tq::launch_matvec<true>(x_rot, ldx, x_div, rhs_indices, pairs, packed_gate, norms_gate, packed_up, norms_up,
                                       codebook, num_experts, N, K, bits, swiglu_limit, out_act, ldo,
                                       (cudaStream_t)stream);
}

int jq_tq_quantize(const float* w_rot, int64_t rows, int64_t K, int bits, const float* boundaries, uint32_t* packed,
                   void* norms, jq_stream_t stream) {
    using namespace jq;
    int rc = tq::check_common(bits, rows, K);
    if (rc != JQ_OK) return rc;
    if (rows == 0) return JQ_OK;
    JQ_REQUIRE(w_rot && boundaries && packed && norms, JQ_EINVAL, "null pointer");
    const int per = 32 / bits;
    const int words = (int)((K + per - 1) / per);
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (bits == 2) tq::tq_quantize_kernel<2><<<grid, 256, 0, (cudaStream_t)stream>>>(w_rot, rows, (int)K, words, boundaries, packed, (__half*)norms);
    if (bits == 3) tq::tq_quantize_kernel<3><<<grid, 256, 0, (cudaStream_t)stream>>>(w_rot, rows, (int)K, words, boundaries, packed, (__half*)norms);
    if (bits == 4) tq::tq_quantize_kernel<4><<<grid, 256, 0, (cudaStream_t)stream>>>(w_rot, rows, (int)K, words, boundaries, packed, (__half*)norms);
    return check_launch("tq quantize");
}

}  // extern "C"
