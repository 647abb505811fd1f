// K2: decode-shaped quantized mat-vec  y[M,N] = x[M,K] . deq(W)[N,K]^T,  M <= 8 per launch.
//
// Bound: HBM bandwidth.  Algorithmic bytes per launch =
//     N*K*bits/8 (codes) + N*(K/gs)*2*sizeof(sidecar) + M*K*2 + M*N*2.
//
// Structure (one CTA = 16 weight rows x all of K, 4 warps):
//   * every warp is its own producer: it bulk-copies (cp.async.bulk + mbarrier
//     complete_tx) 16 row segments of KT codes into private shared-memory buffers,
//     2-3 stages deep, and consumes them itself, so no cross-warp handshake exists
//     until the final reduction; warp w owns stages w, w+4, ...;
//   * codes are dequantized in registers straight into m16n8k16 MMA A operands
//     (jq_mma.cuh: one shift + one LOP3 per two codes); the activations are the B
//     operand (column n of the MMA = activation row m), so M = 1..8 cost the same;
//   * the MMA accumulates one quantization group, then  acc += scale * C  in f32;
//   * the bias term sum_g b[n,g]*X[m,g] and the offset term of the register
//     dequantizer, with X[m,g] = sum of x over the group, are themselves tiny MMAs
//     over the [16 x K/gs] sidecar tiles, X split into hi+lo halves of the 16-bit
//     type so that the f32 sum is kept to ~2^-17;
//   * X[m,g] is computed once per CTA with an all-ones A operand.
// The general fallback kernel (any alignment, group size 32, mixed dtypes) is a
// plain one-warp-per-row SIMT loop with a shuffle reduction.
#include <cstdlib>

#include "jq_mma.cuh"

namespace jq {

__device__ int g_timeout_flag = 0;   // set when a bounded mbarrier wait ran out

struct GemvArgs {
    const void* x;
    const uint32_t* codes;
    const void* scales;
    const void* biases;
    void* y;
    int64_t N, K, ldx, ldy;
    int M, kt, G;
};

constexpr int GEMV_WARPS = 4;

template <int BITS> struct GemvCfg {
    static constexpr int KT_MAX = (BITS <= 4) ? 1024 : 512;
    static constexpr int SEGW_MAX = KT_MAX * BITS / 32;
    static constexpr int STAGE_WORDS = 16 * (SEGW_MAX + 4);
    static constexpr int NBUF = (STAGE_WORDS * 4 > 6000) ? 2 : 3;
};

__host__ __device__ inline int align_up(int v, int a) { return (v + a - 1) / a * a; }

template <typename AT, int BITS, int GS>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
qgemv_mma_kernel(const GemvArgs a) {
    using A = Act<AT>;
    using F = Fields<AT, BITS>;
    using Cfg = GemvCfg<BITS>;
    constexpr int NW = GEMV_WARPS, NBUF = Cfg::NBUF, STAGE = Cfg::STAGE_WORDS;
    static_assert(NW == 4, "the final reduction maps the 4 warps onto the 4 accumulator slots");
    constexpr int BPG = GS / 64;            // 64-code k-blocks per quantization group
    constexpr int UW = Unit<BITS>::WORDS;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    float* Xs = reinterpret_cast<float*>(smem + 128);
    uint32_t* bufs = reinterpret_cast<uint32_t*>(smem + 128 + align_up(a.G * 8 * 4, 128));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int64_t n0 = (int64_t)blockIdx.x * 16;
    const int rows_valid = (int)min((int64_t)16, a.N - n0);
    const int K = (int)a.K, kt = a.kt, G = a.G, M = a.M;
    const int nst = (K + kt - 1) / kt;
    const int RS = kt * BITS / 32 + 4;       // row stride in words (16-byte pad against bank conflicts)
    const int64_t rowwords = a.K * BITS / 32;
    uint32_t* mybuf = bufs + warp * NBUF * STAGE;
    uint64_t* mybar = bars + warp * NBUF;
    const uint16_t* xs16 = reinterpret_cast<const uint16_t*>(a.x);
    const uint16_t* sc16 = reinterpret_cast<const uint16_t*>(a.scales);
    const uint16_t* bi16 = reinterpret_cast<const uint16_t*>(a.biases);

    if (threadIdx.x == 0) {
        for (int i = 0; i < NW * NBUF; ++i) mbar_init(bars + i, 1);
        mbar_fence_init();
    }
    __syncthreads();

    auto issue = [&](int st, int b) {
        const int k0 = st * kt;
        const int kc = min(kt, K - k0);
        const uint32_t segbytes = (uint32_t)(kc * BITS / 8);
        if (lane == 0) mbar_expect_tx(mybar + b, segbytes * (uint32_t)rows_valid);
        __syncwarp();
        if (lane < rows_valid)
            bulk_g2s(mybuf + b * STAGE + lane * RS, a.codes + (n0 + lane) * rowwords + (int64_t)k0 * BITS / 32,
                     segbytes, mybar + b);
    };

    // start streaming weights before anything else
#pragma unroll
    for (int i = 0; i < NBUF; ++i) {
        const int st = warp + i * NW;
        if (st < nst) issue(st, i);
    }

    // X[m][grp] = sum of x over the group, via an all-ones A operand
    {
        const uint32_t ones[4] = {A::ONES, A::ONES, A::ONES, A::ONES};
        for (int grp = warp; grp < G; grp += NW) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint16_t* xr = xs16 + (int64_t)g * a.ldx + (int64_t)grp * GS + tig * 8;
#pragma unroll
            for (int i = 0; i < GS / 32; ++i) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (g < M) v = __ldg(reinterpret_cast<const uint4*>(xr + i * 32));
                A::mma(c, ones, v.x, v.y);
                A::mma(c, ones, v.z, v.w);
            }
            if (g == 0) {
                Xs[grp * 8 + 2 * tig] = c[0];
                Xs[grp * 8 + 2 * tig + 1] = c[1];
            }
        }
    }
    __syncthreads();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int64_t r_lo = min(n0 + g, a.N - 1), r_hi = min(n0 + g + 8, a.N - 1);
    bool ok = true;

    int it = 0;
    for (int st = warp; st < nst && ok; st += NW, ++it) {
        const int b = it % NBUF;
        const uint32_t parity = (uint32_t)(it / NBUF) & 1u;
        const int k0 = st * kt;
        const int kc = min(kt, K - k0);
        const int nblk = kc >> 6;
        if (!mbar_wait(mybar + b, parity)) {
            ok = false;
            atomicExch(&g_timeout_flag, 1);
            break;
        }
        const uint32_t* row_lo = mybuf + b * STAGE + g * RS;
        const uint32_t* row_hi = row_lo + 8 * RS;
        float cg[F::PASSES][4];
#pragma unroll
        for (int p = 0; p < F::PASSES; ++p) cg[p][0] = cg[p][1] = cg[p][2] = cg[p][3] = 0.f;
        float s_lo = 0.f, s_hi = 0.f;
        for (int blk = 0; blk < nblk; ++blk) {
            const int kb = k0 + blk * 64;
            uint32_t xr[8];
            {
                uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
                if (g < M) {
                    const uint4* xp = reinterpret_cast<const uint4*>(xs16 + (int64_t)g * a.ldx + kb + tig * 16);
                    v0 = __ldg(xp);
                    v1 = __ldg(xp + 1);
                }
                xr[0] = v0.x; xr[1] = v0.y; xr[2] = v0.z; xr[3] = v0.w;
                xr[4] = v1.x; xr[5] = v1.y; xr[6] = v1.z; xr[7] = v1.w;
            }
            if (blk % BPG == 0) {
                const int grp = kb / GS;
                s_lo = A::to_f32(__ldg(sc16 + r_lo * G + grp));
                s_hi = A::to_f32(__ldg(sc16 + r_hi * G + grp));
            }
            uint32_t ulo[UW], uhi[UW];
            load_unit<BITS>(row_lo, blk, tig, ulo);
            load_unit<BITS>(row_hi, blk, tig, uhi);
#define JQ_STEP(T)                                                                     \
    {                                                                                  \
        const uint32_t b0 = make_b<BITS, T, 0>(xr), b1 = make_b<BITS, T, 1>(xr);       \
        {                                                                              \
            const uint32_t af[4] = {make_a<AT, BITS, T, 0, 0>(ulo), make_a<AT, BITS, T, 0, 0>(uhi), \
                                    make_a<AT, BITS, T, 1, 0>(ulo), make_a<AT, BITS, T, 1, 0>(uhi)}; \
            A::mma(cg[0], af, b0, b1);                                                 \
        }                                                                              \
        if constexpr (F::PASSES == 2) {                                                \
            const uint32_t af[4] = {make_a<AT, BITS, T, 0, 1>(ulo), make_a<AT, BITS, T, 0, 1>(uhi), \
                                    make_a<AT, BITS, T, 1, 1>(ulo), make_a<AT, BITS, T, 1, 1>(uhi)}; \
            A::mma(cg[F::PASSES - 1], af, b0, b1);                                     \
        }                                                                              \
    }
            JQ_STEP(0) JQ_STEP(1) JQ_STEP(2) JQ_STEP(3)
#undef JQ_STEP
            if (blk % BPG == BPG - 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float c = cg[0][i];
                    if constexpr (F::PASSES == 2) c = fmaf(16.f, cg[F::PASSES - 1][i], c);
                    acc[i] = fmaf(i < 2 ? s_lo : s_hi, c, acc[i]);
                }
#pragma unroll
                for (int p = 0; p < F::PASSES; ++p) cg[p][0] = cg[p][1] = cg[p][2] = cg[p][3] = 0.f;
            }
        }
        __syncwarp();
        const int nxt = st + NBUF * NW;
        if (nxt < nst) issue(nxt, b);
    }

    // bias and offset terms: sum_g (b - OFFSET*s)[n,g] * X[m,g] as MMAs over the sidecars
    float sx[4] = {0.f, 0.f, 0.f, 0.f}, bx[4] = {0.f, 0.f, 0.f, 0.f};
    for (int gb = warp; gb * 16 < G; gb += NW) {
        const int g0 = gb * 16 + 2 * tig;
        auto ld2 = [&](const uint16_t* base, int64_t row, int grp) -> uint32_t {
            const uint32_t v0 = (grp < G) ? (uint32_t)__ldg(base + row * G + grp) : 0u;
            const uint32_t v1 = (grp + 1 < G) ? (uint32_t)__ldg(base + row * G + grp + 1) : 0u;
            return v0 | (v1 << 16);
        };
        const uint32_t as[4] = {ld2(sc16, r_lo, g0), ld2(sc16, r_hi, g0), ld2(sc16, r_lo, g0 + 8),
                                ld2(sc16, r_hi, g0 + 8)};
        const uint32_t ab[4] = {ld2(bi16, r_lo, g0), ld2(bi16, r_hi, g0), ld2(bi16, r_lo, g0 + 8),
                                ld2(bi16, r_hi, g0 + 8)};
        auto ldX = [&](int grp) -> float { return grp < G ? Xs[grp * 8 + g] : 0.f; };
        const float x0 = ldX(g0), x1 = ldX(g0 + 1), x2 = ldX(g0 + 8), x3 = ldX(g0 + 9);
        const uint32_t h0 = A::pack_hi(x0, x1), h1 = A::pack_hi(x2, x3);
        const uint32_t l0 = A::pack_hi(x0 - A::lo_f32(h0), x1 - A::hi_f32(h0));
        const uint32_t l1 = A::pack_hi(x2 - A::lo_f32(h1), x3 - A::hi_f32(h1));
        A::mma(sx, as, h0, h1);
        A::mma(sx, as, l0, l1);
        A::mma(bx, ab, h0, h1);
        A::mma(bx, ab, l0, l1);
    }

    __syncthreads();   // every warp is done with its buffers and with Xs
    float* red = reinterpret_cast<float*>(bufs);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        red[(warp * 4 + i) * 32 + lane] = fmaf(acc[i], F::POST, fmaf(-F::OFFSET, sx[i], bx[i]));
    __syncthreads();
    {
        const int i = threadIdx.x >> 5;    // 4 warps <-> the 4 accumulator slots
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[(w * 4 + i) * 32 + lane];
        const int row = g + ((i & 2) ? 8 : 0), m = 2 * tig + (i & 1);
        if (row < rows_valid && m < M)
            reinterpret_cast<uint16_t*>(a.y)[(int64_t)m * a.ldy + n0 + row] = A::from_f32(v);
    }
}

// ---- general fallback: one warp per weight row, SIMT -----------------------------------
__device__ __forceinline__ float ld_any(const void* p, int64_t i, int dtype) {
    if (dtype == JQ_F32) return reinterpret_cast<const float*>(p)[i];
    if (dtype == JQ_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_any(void* p, int64_t i, int dtype, float v) {
    if (dtype == JQ_F32) reinterpret_cast<float*>(p)[i] = v;
    else if (dtype == JQ_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

template <int BITS>
__global__ void __launch_bounds__(128)
qgemv_simple_kernel(const GemvArgs a, int x_dtype, int sc_dtype, int y_dtype, int gs) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * 4 + warp;
    if (n >= a.N) return;
    const int64_t rowwords = a.K * BITS / 32;
    const uint32_t* row = a.codes + n * rowwords;
    const int64_t n_oct = a.K / 8;
    float acc[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m] = 0.f;
    for (int64_t oct = lane; oct < n_oct; oct += 32) {
        const int64_t byte0 = oct * BITS;
        const int64_t w0 = byte0 >> 2;
        const int sh = (int)(byte0 & 3) * 8;
        const uint32_t c0 = row[w0];
        const uint32_t c1 = (w0 + 1 < rowwords) ? row[w0 + 1] : 0u;
        const uint32_t c2 = (BITS > 4 && w0 + 2 < rowwords) ? row[w0 + 2] : 0u;
        const unsigned long long bitsv =
            ((unsigned long long)__funnelshift_r(c1, c2, sh) << 32) | __funnelshift_r(c0, c1, sh);
        const int64_t grp = (oct * 8) / gs;
        const float s = ld_any(a.scales, n * a.G + grp, sc_dtype);
        const float bs = ld_any(a.biases, n * a.G + grp, sc_dtype);
        float q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = (float)((uint32_t)(bitsv >> (j * BITS)) & ((1u << BITS) - 1u));
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            if (m < a.M) {
                float qx = 0.f, sx = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float xv = ld_any(a.x, (int64_t)m * a.ldx + oct * 8 + j, x_dtype);
                    qx = fmaf(q[j], xv, qx);
                    sx += xv;
                }
                acc[m] = fmaf(s, qx, fmaf(bs, sx, acc[m]));    // dsv41/metal_decode.py:233 order
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        float v = acc[m];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, d);
        if (lane == 0 && m < a.M) st_any(a.y, (int64_t)m * a.ldy + n, y_dtype, v);
    }
}

static bool force_simple() {
    const char* e = getenv("JANGQ_FORCE_SIMPLE_GEMV");
    return e && e[0] == '1';
}

template <typename AT, int BITS, int GS>
static int launch_mma(const GemvArgs& a, cudaStream_t st, bool* launched) {
    using Cfg = GemvCfg<BITS>;
    const size_t smem = 128 + align_up(a.G * 8 * 4, 128) + (size_t)GEMV_WARPS * Cfg::NBUF * Cfg::STAGE_WORDS * 4;
    *launched = false;
    if (smem > 200 * 1024) return JQ_OK;   // very long rows: fallback
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_mma_kernel<AT, BITS, GS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        200 * 1024));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    const unsigned grid = (unsigned)((a.N + 15) / 16);
    qgemv_mma_kernel<AT, BITS, GS><<<grid, GEMV_WARPS * 32, smem, st>>>(a);
    *launched = true;
    return check_launch("qgemv");
}

int qgemv_dispatch(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
                   const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int gs, void* y,
                   int y_dtype, int64_t ldy, cudaStream_t st) {
    int rc = check_quant_shape(N, K, bits, gs);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(x_dtype) && valid_dtype(sidecar_dtype) && valid_dtype(y_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(M >= 0 && M <= JQ_QGEMV_MAX_M, JQ_EINVAL, "qgemv takes 0 <= M <= %d rows, got %lld", JQ_QGEMV_MAX_M,
               (long long)M);
    if (M == 0 || N == 0) return JQ_OK;
    JQ_REQUIRE(K > 0, JQ_EINVAL, "K must be positive");
    JQ_REQUIRE(x && codes && scales && biases && y, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(ldx >= K && ldy >= N, JQ_EINVAL, "leading dimension too small");
    JQ_REQUIRE(N < (1ll << 31) && K < (1ll << 31), JQ_EUNSUPPORTED, "dimension too large");

    const bool fast = !force_simple() && (gs == 64 || gs == 128) && x_dtype != JQ_F32 && sidecar_dtype == x_dtype &&
                      y_dtype == x_dtype && aligned(codes, 16) && ((K * bits / 8) % 16 == 0) && aligned(x, 16) &&
                      (ldx % 8 == 0) && aligned(scales, 2) && aligned(biases, 2);
    for (int64_t m0 = 0; m0 < M; m0 += 8) {
        GemvArgs a;
        a.x = (const char*)x + m0 * ldx * dtype_size(x_dtype);
        a.codes = codes; a.scales = scales; a.biases = biases;
        a.y = (char*)y + m0 * ldy * dtype_size(y_dtype);
        a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy;
        a.M = (int)((M - m0) < 8 ? (M - m0) : 8);
        a.G = (int)(K / gs);
        bool launched = false;
        if (fast) {
            // stage length: as long as possible while every warp still gets a stage
            int kt = (bits <= 4) ? 1024 : 512;
            while (K / kt < GEMV_WARPS && kt * bits / 8 > 128) kt >>= 1;
            a.kt = kt;
#define JQ_GEMV_CASE(B, GSZ)                                                                     \
    if (bits == B && gs == GSZ) {                                                                \
        rc = (x_dtype == JQ_BF16) ? launch_mma<__nv_bfloat16, B, GSZ>(a, st, &launched)          \
                                  : launch_mma<__half, B, GSZ>(a, st, &launched);                \
        if (rc != JQ_OK) return rc;                                                              \
    }
            JQ_GEMV_CASE(2, 64) JQ_GEMV_CASE(3, 64) JQ_GEMV_CASE(4, 64) JQ_GEMV_CASE(5, 64) JQ_GEMV_CASE(6, 64)
            JQ_GEMV_CASE(8, 64) JQ_GEMV_CASE(2, 128) JQ_GEMV_CASE(3, 128) JQ_GEMV_CASE(4, 128)
            JQ_GEMV_CASE(5, 128) JQ_GEMV_CASE(6, 128) JQ_GEMV_CASE(8, 128)
#undef JQ_GEMV_CASE
        }
        if (!launched) {
            a.kt = 0;
            const unsigned grid = (unsigned)((N + 3) / 4);
            JQ_DISPATCH_BITS(bits, B,
                (qgemv_simple_kernel<B><<<grid, 128, 0, st>>>(a, x_dtype, sidecar_dtype, y_dtype, gs)))
            rc = check_launch("qgemv (general)");
            if (rc != JQ_OK) return rc;
        }
    }
    return JQ_OK;
}

}  // namespace jq

extern "C" {

int jq_qgemv(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
             const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y,
             int y_dtype, int64_t ldy, jq_stream_t stream) {
    return jq::qgemv_dispatch(x, x_dtype, M, ldx, codes, scales, biases, sidecar_dtype, N, K, bits, group_size, y,
                              y_dtype, ldy, (cudaStream_t)stream);
}

int jq_qgemv_batched(const JqGemvDesc* descs, int count, int64_t M, int act_dtype, int sidecar_dtype,
                     jq_stream_t stream) {
    JQ_REQUIRE(count >= 0 && count <= JQ_QGEMV_MAX_BATCH, JQ_EINVAL, "count must be in [0, %d]", JQ_QGEMV_MAX_BATCH);
    JQ_REQUIRE(count == 0 || descs, JQ_EINVAL, "null descriptor table");
    for (int i = 0; i < count; ++i) {
        const JqGemvDesc& d = descs[i];
        int rc = jq::qgemv_dispatch(d.x, act_dtype, M, d.ldx, d.codes, d.scales, d.biases, sidecar_dtype, d.N, d.K,
                                    d.bits, d.group_size, d.y, act_dtype, d.ldy, (cudaStream_t)stream);
        if (rc != JQ_OK) return rc;
    }
    return JQ_OK;
}

int jq_device_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, jq::g_timeout_flag, sizeof(int)) != cudaSuccess)
        return jq::fail(JQ_ECUDA, "could not read the device status word");
    if (v != 0) return jq::fail(JQ_ETIMEOUT, "a bounded device-side wait ran out");
    return JQ_OK;
}

}  // extern "C"
