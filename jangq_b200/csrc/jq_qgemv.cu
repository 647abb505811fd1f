// K2: decode-shaped quantized mat-vec  y[M,N] = x[M,K] . deq(W)[N,K]^T,  M <= 8 per launch.
//
// Bound: HBM bandwidth.  Algorithmic bytes per launch =
//     N*K*bits/8 (codes) + N*(K/gs)*2*sizeof(sidecar) + M*K*2 + M*N*2.
//
// Structure (one CTA = 16*MT weight rows x all of K, 4 warps):
//   * every warp is its own producer and consumer: with 128-bit cp.async copies
//     (every lane one 16-byte chunk, 8 lanes per 128-byte row segment) it streams a
//     stage = 16*MT row segments of `kt` codes plus the M activation row segments of
//     the same k-range into private shared-memory buffers, 2-3 stages deep, so no
//     cross-warp handshake exists until the final reduction; warp w owns stages
//     w, w+4, ...  (one bulk-copy instruction moves a single row segment and is
//     issued by one lane at a time, which made ~33 of them per stage cost more
//     issue slots than the stage's arithmetic; per-lane cp.async costs ~10
//     instructions per stage);  scales/biases of a stage are
//     fetched one stage ahead with 8-byte loads and parked in shared memory as the
//     f32 pair (s*POST, b - OFFSET*s);
//   * codes are dequantized in registers straight into m16n8k16 MMA A operands
//     (jq_mma.cuh: one shift + one LOP3 per two codes); the activations are the B
//     operand (column n of the MMA = activation row m), so M = 1..8 cost the same;
//   * per quantization group the MMA accumulates C = sum (2^FB + q) x (scaled) and,
//     with X = sum of x over the group,   acc += (s*POST) * C + (b - OFFSET*s) * X ;
//     X comes from a per-stage SIMT pre-pass when M <= 2 and from an extra MMA with
//     an all-ones A operand otherwise;
//   * the four warps' partial sums are added through shared memory;
//   * a launch may cover several matrices that share x (GemvBatch): the grid is the concatenation of
//     their row tiles.
// The general fallback kernel (any alignment, group size 32, 5-bit, mixed dtypes)
// is a plain one-warp-per-row SIMT loop with a shuffle reduction.
#include <cstdlib>

#include "jq_mma.cuh"
#include "jq_qgemv.cuh"

namespace jq {

__device__ int g_timeout_flag = 0;   // set by any kernel whose bounded wait ran out

__host__ __device__ inline int align_up(int v, int a) { return (v + a - 1) / a * a; }

// Compile-time geometry of one stage buffer (per warp, per pipeline slot).
template <int BITS, int GS, int MT> struct GemvGeom {
    static constexpr int KT = (BITS <= 4 || GS == 128) ? 512 : 256;   // codes per row and stage
    static constexpr int ROWS = 16 * MT;
    // row padding (words) that keeps the per-lane unit loads free of bank conflicts
    static constexpr int PAD = BITS == 2 ? 4 : BITS == 6 ? 12 : BITS == 8 ? 16 : 8;
    static constexpr int RS = KT * BITS / 32 + PAD;      // code row stride, words
    static constexpr int XS = KT + 8;                    // activation row stride, elements
    static constexpr int NG = KT / GS;                   // groups per stage (4 or 8)
    static constexpr int NQ = NG / 4;                    // 8-byte sidecar quads per row
    static constexpr int NGP = NG + 1;                   // padded sidecar row stride, float2
    static constexpr int Z_OFF = ROWS * RS * 4;          // 32 zero bytes (B operand of lanes g >= M)
    static constexpr int SC_OFF = Z_OFF + 32;            // float2 (s*POST, b - OFFSET*s) [ROWS][NGP]
    static constexpr int XSUM_OFF = SC_OFF + ROWS * NGP * 8;   // float X[NG][8]
    static constexpr int X_OFF = XSUM_OFF + NG * 8 * 4;  // activations [M][XS]
    __host__ __device__ static constexpr int stage_bytes(int M) { return X_OFF + M * XS * 2; }
};

template <typename AT, int BITS, int GS, int MT, int NW>
__global__ void __launch_bounds__(NW * 32)
qgemv_mma_kernel(const GemvArgs a, const GemvBatch bt) {
    using A = Act<AT>;
    using F = Fields<AT, BITS>;
    using Geo = GemvGeom<BITS, GS, MT>;
    static_assert(NW == 4 || NW == 8, "4 or 8 warps split K");
    constexpr int ROWS = Geo::ROWS, KT = Geo::KT, RS = Geo::RS, XS = Geo::XS, NG = Geo::NG, NQ = Geo::NQ,
                  NGP = Geo::NGP;

    extern __shared__ __align__(128) uint8_t smem[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int K = (int)a.K, G = a.G, M = a.M, nbuf = a.nbuf;
    const int nst = (K + KT - 1) / KT;
    const int stage_bytes = Geo::stage_bytes(M);
    const int64_t rowbytes = a.K * BITS / 8;
    uint8_t* mybuf = smem + (size_t)warp * nbuf * stage_bytes;
    const uint16_t* xs16 = reinterpret_cast<const uint16_t*>(a.x);
    // which matrix of the fused launch this block belongs to (gather mode: always the tables below)
    int mi = 0, blk0 = 0;
    while (mi + 1 < bt.count && (int)blockIdx.x >= bt.blk_end[mi]) { blk0 = bt.blk_end[mi]; ++mi; }
    const int64_t N = bt.N[mi], ldy = bt.ldy[mi];
    const int64_t n0 = (int64_t)((int)blockIdx.x - blk0) * ROWS;
    const int rows_valid = (int)min((int64_t)ROWS, N - n0);
    const uint16_t* sc16 = reinterpret_cast<const uint16_t*>(bt.scales[mi]);
    const uint16_t* bi16 = reinterpret_cast<const uint16_t*>(bt.biases[mi]);
    const uint32_t* codes_g = bt.codes[mi];
    uint16_t* y16 = reinterpret_cast<uint16_t*>(bt.y[mi]);
    if (a.pair_expert) {
        // the pair list is itself an output of the predecessor (the router): nothing is read before it is done
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int p = blockIdx.y;
        const int e = a.pair_expert[p] - a.expert_base;
        const bool second = blockIdx.z != 0;                         // gate | up in one launch
        if (e < 0 || e >= a.num_experts) {                            // expert of another rank: the pair's row is zero
            uint16_t* yz = reinterpret_cast<uint16_t*>(second ? a.y2 : bt.y[0]) + (int64_t)p * ldy + n0;
            for (int r = threadIdx.x; r < rows_valid; r += blockDim.x) yz[r] = 0;
            return;
        }
        if (a.bits_tab && a.bits_tab[e] != BITS) return;              // handled by the launch of its own width
        codes_g = (second ? a.codes_tab2 : a.codes_tab)[e];
        sc16 = reinterpret_cast<const uint16_t*>((second ? a.scales_tab2 : a.scales_tab)[e]);
        bi16 = reinterpret_cast<const uint16_t*>((second ? a.biases_tab2 : a.biases_tab)[e]);
        xs16 += (int64_t)(p / a.x_div) * a.ldx;
        if (second) y16 = reinterpret_cast<uint16_t*>(a.y2);
        y16 += (int64_t)p * ldy;
    }

    if (lane < 8)
        for (int b = 0; b < nbuf; ++b)
            reinterpret_cast<uint32_t*>(mybuf + (size_t)b * stage_bytes + Geo::Z_OFF)[lane] = 0u;

    // ---- stage copies: 16 bytes per lane and instruction -------------------------------------
    // LPR lanes share a code row (the smallest power of two covering its chunks), so one
    // instruction covers 32/LPR rows and the per-iteration address update is two adds.
    const uint8_t* code_base = reinterpret_cast<const uint8_t*>(codes_g) + n0 * rowbytes;
    auto issue_codes = [&](int st, int b) {
        if (st < nst) {
            const int k0 = st * KT;
            const int kc = min(KT, K - k0);
            uint8_t* buf = mybuf + (size_t)b * stage_bytes;
            const int cpr = kc * BITS / 128;                          // 16-byte chunks per code row
            const int lpr = cpr <= 4 ? 4 : cpr <= 8 ? 8 : cpr <= 16 ? 16 : 32;
            const int col = lane & (lpr - 1), rpi = 32 / lpr;
            if (col < cpr) {
                int row = lane / lpr;
                const uint8_t* src = code_base + (int64_t)row * rowbytes + (int64_t)k0 * BITS / 8 + col * 16;
                uint8_t* dst = buf + row * (RS * 4) + col * 16;
                for (; row < rows_valid; row += rpi) {
                    cp_async16(dst, src);
                    src += (int64_t)rpi * rowbytes;
                    dst += rpi * (RS * 4);
                }
            }
        }
    };
    auto issue_x = [&](int st, int b) {
        if (st < nst) {
            const int k0 = st * KT;
            const int kc = min(KT, K - k0);
            uint8_t* buf = mybuf + (size_t)b * stage_bytes;
            const int cpx = kc / 8;                                    // chunks per activation row (32 or 64)
            for (int m = 0; m < M; ++m)
                for (int c = lane; c < cpx; c += 32)
                    cp_async16(buf + Geo::X_OFF + (m * XS + c * 8) * 2, xs16 + (int64_t)m * a.ldx + k0 + c * 8);
        }
    };

    // ---- sidecars of a stage: pair index -> (row, quad of 4 groups), one 8-byte load each -----
    constexpr int SCP = (ROWS * NQ + 31) / 32;     // pairs per lane
    uint2 sv[SCP], bv[SCP];
    auto fetch_sc = [&](int st) {
#pragma unroll
        for (int i = 0; i < SCP; ++i) {
            const int pr = lane + 32 * i;
            const int row = pr / NQ, quad = pr % NQ;
            const int grp = st * NG + quad * 4;
            sv[i] = make_uint2(0u, 0u);
            bv[i] = make_uint2(0u, 0u);
            if (pr < ROWS * NQ && grp < G) {
                const int64_t off = min(n0 + row, N - 1) * G + grp;
                sv[i] = __ldg(reinterpret_cast<const uint2*>(sc16 + off));
                bv[i] = __ldg(reinterpret_cast<const uint2*>(bi16 + off));
            }
        }
    };
    auto store_sc = [&](uint8_t* buf) {
#pragma unroll
        for (int i = 0; i < SCP; ++i) {
            const int pr = lane + 32 * i;
            const int row = pr / NQ, quad = pr % NQ;
            if (pr < ROWS * NQ) {
                float2* dst = reinterpret_cast<float2*>(buf + Geo::SC_OFF) + row * NGP + quad * 4;
                const float s0 = A::lo_f32(sv[i].x), s1 = A::hi_f32(sv[i].x), s2 = A::lo_f32(sv[i].y),
                            s3 = A::hi_f32(sv[i].y);
                dst[0] = make_float2(s0 * F::POST, fmaf(-F::OFFSET, s0, A::lo_f32(bv[i].x)));
                dst[1] = make_float2(s1 * F::POST, fmaf(-F::OFFSET, s1, A::hi_f32(bv[i].x)));
                dst[2] = make_float2(s2 * F::POST, fmaf(-F::OFFSET, s2, A::lo_f32(bv[i].y)));
                dst[3] = make_float2(s3 * F::POST, fmaf(-F::OFFSET, s3, A::hi_f32(bv[i].y)));
            }
        }
    };

    // Start streaming the weights before anything else.  Under programmatic dependent launch
    // this kernel may begin while its predecessor in the stream still runs: weights and
    // sidecars (static by contract) are prefetched at once, the activations only after
    // griddepcontrol.wait, and the successor is allowed to start launching immediately.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
    for (int i = 0; i < GEMV_MAX_NBUF; ++i)
        if (i < nbuf) issue_codes(warp + i * NW, i);
    fetch_sc(warp);
    asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
    for (int i = 0; i < GEMV_MAX_NBUF; ++i)
        if (i < nbuf) {
            issue_x(warp + i * NW, i);
            cp_async_commit();
        }

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

    int it = 0;
    for (int st = warp; st < nst; st += NW, ++it) {
        const int b = it % nbuf;
        const int kc = min(KT, K - st * KT);
        const int nblk = kc >> 6;
        uint8_t* buf = mybuf + (size_t)b * stage_bytes;
        store_sc(buf);
        if (st + NW < nst) fetch_sc(st + NW);
        if (nbuf == 3) cp_async_wait<2>(); else cp_async_wait<1>();   // this stage's copies have landed
        __syncwarp();

        // ---- X[grp][m] = sum of the group's activations -----------------------------------------
        float* Xs = reinterpret_cast<float*>(buf + Geo::XSUM_OFF);
        if (M <= 2) {
            // SIMT: lane l sums the 16 activations of chunk l; GS/16 adjacent lanes make a group
            for (int m = 0; m < M; ++m) {
                float sum = 0.f;
                if (lane * 16 < kc) {
                    const uint4* xp = reinterpret_cast<const uint4*>(buf + Geo::X_OFF + (m * XS + lane * 16) * 2);
                    const uint4 v0 = xp[0], v1 = xp[1];
                    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) { s0 += A::lo_f32(w[j]); s1 += A::hi_f32(w[j]); }
                    sum = s0 + s1;
                }
#pragma unroll
                for (int d = 1; d < GS / 16; d <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
                if ((lane & (GS / 16 - 1)) == 0 && lane * 16 < kc) Xs[(lane * 16 / GS) * 8 + m] = sum;
            }
        } else {
            // tensor cores: the activations are the A operand (row = m, 8 consecutive k per lane), B is
            // all ones, so every column of C holds the row sums; rows g and g+8 carry two k-chunks
            const uint16_t* xa = (g < M) ? reinterpret_cast<const uint16_t*>(buf + Geo::X_OFF) + g * XS + tig * 8
                                         : reinterpret_cast<const uint16_t*>(buf + Geo::Z_OFF);
            const int xa_step = (g < M) ? 32 : 0;
            const int ngrp = kc / GS;
            for (int grp = 0; grp < ngrp; ++grp) {
                float c[4];
#pragma unroll
                for (int i = 0; i < GS / 32; ++i) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xa + (grp * (GS / 32) + i) * xa_step);
                    const uint32_t af[4] = {v.x, v.y, v.z, v.w};
                    if (i == 0) A::mma0(c, af, A::ONES, A::ONES); else A::mma(c, af, A::ONES, A::ONES);
                }
                if (tig == 0) Xs[grp * 8 + g] = c[0] + c[2];
            }
        }
        __syncwarp();

        // ---- main loop over the stage's 64-code k-blocks ------------------------------------------
        const uint32_t* c_lo = reinterpret_cast<const uint32_t*>(buf) + g * RS;
        const uint16_t* xrow = (g < M) ? reinterpret_cast<const uint16_t*>(buf + Geo::X_OFF) + g * XS + tig * 16
                                       : reinterpret_cast<const uint16_t*>(buf + Geo::Z_OFF);
        const int xstep = (g < M) ? 64 : 0;
        const float2* pt = reinterpret_cast<const float2*>(buf + Geo::SC_OFF) + g * NGP;
        const float* xsum = Xs + 2 * tig;
        gemv_stage_blocks<AT, BITS, GS, MT>(c_lo, RS, xrow, xstep, pt, NGP, xsum, nblk, tig, acc);
        __syncwarp();
        issue_codes(st + nbuf * NW, b);
        issue_x(st + nbuf * NW, b);
        cp_async_commit();     // always one group per iteration so that the group count stays uniform
    }
    cp_async_wait<0>();

    __syncthreads();   // every warp is done with its buffers
    float* red = reinterpret_cast<float*>(smem);   // overlays the (now idle) stage buffers
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[((warp * MT + mt) * 4 + i) * 32 + lane] = acc[mt][i];
    __syncthreads();
    if (warp < 4) {
        const int i = warp;                // warps 0..3 <-> the 4 accumulator slots
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) v += red[((w * MT + mt) * 4 + i) * 32 + lane];
            const int row = mt * 16 + g + ((i & 2) ? 8 : 0), m = 2 * tig + (i & 1);
            if (row < rows_valid && m < M)
                y16[(int64_t)m * ldy + n0 + row] = A::from_f32(v);
        }
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
    const uint32_t* codes_g = a.codes;
    const void* scales_g = a.scales;
    const void* biases_g = a.biases;
    int64_t x_row0 = 0, y_row0 = 0;
    if (a.pair_expert) {
        const int p = blockIdx.y;
        const int e = a.pair_expert[p] - a.expert_base;
        const bool second = blockIdx.z != 0;
        if (e < 0 || e >= a.num_experts) {                            // expert of another rank: zero output
            if (lane == 0)
                for (int m = 0; m < a.M; ++m) st_any(second ? a.y2 : a.y, (int64_t)(p + m) * a.ldy + n, y_dtype, 0.f);
            return;
        }
        if (a.bits_tab && a.bits_tab[e] != BITS) return;
        codes_g = (second ? a.codes_tab2 : a.codes_tab)[e];
        scales_g = (second ? a.scales_tab2 : a.scales_tab)[e];
        biases_g = (second ? a.biases_tab2 : a.biases_tab)[e];
        x_row0 = p / a.x_div;
        y_row0 = p;
    }
    const uint32_t* row = codes_g + n * rowwords;
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
        const float s = ld_any(scales_g, n * a.G + grp, sc_dtype);
        const float bs = ld_any(biases_g, n * a.G + grp, sc_dtype);
        float q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = (float)((uint32_t)(bitsv >> (j * BITS)) & ((1u << BITS) - 1u));
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            if (m < a.M) {
                float qx = 0.f, sx = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float xv = ld_any(a.x, (x_row0 + m) * a.ldx + oct * 8 + j, x_dtype);
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
        if (lane == 0 && m < a.M)
            st_any((a.pair_expert && blockIdx.z != 0) ? a.y2 : a.y, (y_row0 + m) * a.ldy + n, y_dtype, v);
    }
}

int* status_word() {
    static int* cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_timeout_flag) != cudaSuccess) return nullptr;
        cached[dev] = static_cast<int*>(p);
    }
    return cached[dev];
}

static bool force_simple() {
    const char* e = getenv("JANGQ_FORCE_SIMPLE_GEMV");
    return e && e[0] == '1';
}

// JANGQ_GEMV_KERNEL selects the fast-path kernel: unset = per-width default, "tc" = tensor-memory
// kernel wherever the shape fits it, "pint" = persistent integer warp-MMA kernel wherever it fits,
// "one" = item-streaming integer kernel (one activation row) wherever it fits,
// "mma" = the warp-MMA kernel of this file.  The parity tests force every kernel with it.
static int gemv_kernel_choice() {
    const char* e = getenv("JANGQ_GEMV_KERNEL");
    if (!e) return 0;
    if (e[0] == 'm') return 1;
    if (e[0] == 't') return 3;
    if (e[0] == 'p') return 4;      // persistent integer warp-MMA kernel wherever the shape fits it
    if (e[0] == 'o') return 5;      // item-streaming integer kernel (one activation row) wherever the shape fits it
    return 0;
}

template <typename AT, int BITS, int GS, int MT, int NW>
static int launch_mma_cfg(GemvArgs a, GemvBatch bt, int pairs, int nbuf, cudaStream_t st, bool* launched) {
    const unsigned banks = (a.pair_expert && a.codes_tab2) ? 2u : 1u;
    using Geo = GemvGeom<BITS, GS, MT>;
    *launched = false;
    const int sb = Geo::stage_bytes(a.M);
    a.nbuf = nbuf;
    const size_t smem = (size_t)NW * a.nbuf * sb;
    if (smem > 200 * 1024) return JQ_OK;   // does not fit: general kernel
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_mma_kernel<AT, BITS, GS, MT, NW>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    int64_t grid = 0;
    for (int i = 0; i < bt.count; ++i) {
        grid += (bt.N[i] + 16 * MT - 1) / (16 * MT);
        bt.blk_end[i] = (int)grid;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, (unsigned)pairs, banks);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemv_mma_kernel<AT, BITS, GS, MT, NW>, a, bt));
    *launched = true;
    return JQ_OK;
}

// Shape heuristics.  The kernel is latency-bound per warp, so what matters is how many warps
// the grid puts on every SM and how many stages each of them walks in sequence:
//   * 32-row tiles (MT=2) halve the per-weight cost of the activation operand; they pay off for
//     medium grids (4 to 12 sixteen-row tiles per SM);
//   * a small grid (at most ~2 tiles per SM) with long rows splits K over 8 warps instead of 4;
//   * two pipeline stages keep shared memory small (more resident CTAs); a third one only pays when
//     each warp walks many stages in sequence (8 warps, very long rows).
// The thresholds come from a sweep over the decode shapes of the BASELINE configurations.
template <typename AT, int BITS, int GS>
static int launch_mma(const GemvArgs& a, const GemvBatch& bt, int pairs, cudaStream_t st, bool* launched) {
    const int sms = sm_count();
    int64_t tiles16 = 0;
    for (int i = 0; i < bt.count; ++i) tiles16 += (bt.N[i] + 15) / 16;
    tiles16 *= pairs;
    constexpr int KT = GemvGeom<BITS, GS, 1>::KT;
    const int nst = (int)((a.K + KT - 1) / KT);
    const int mt = (tiles16 >= (int64_t)4 * sms && tiles16 < (int64_t)12 * sms) ? 2 : 1;
    int nw = (mt == 1 && tiles16 <= (int64_t)2 * sms && nst >= 16) ? 8 : 4;
    if (mt == 2) nw = 4;
    const int sb = mt == 2 ? GemvGeom<BITS, GS, 2>::stage_bytes(a.M) : GemvGeom<BITS, GS, 1>::stage_bytes(a.M);
    const int nbuf = (nw == 8 && nst >= 20 && nw * 3 * sb <= 200 * 1024) ? 3 : 2;
    if (mt == 2) {
        // 32-row tiles may not fit either (wide codes, several activation rows, long groups): 16-row tiles then
        const int rc = launch_mma_cfg<AT, BITS, GS, 2, 4>(a, bt, pairs, nbuf, st, launched);
        if (rc != JQ_OK || *launched) return rc;
    }
    if (nw == 8) {
        // eight warps' stages may not fit the shared memory (several activation rows, wide codes): four warps then
        const int rc = launch_mma_cfg<AT, BITS, GS, 1, 8>(a, bt, pairs, nbuf, st, launched);
        if (rc != JQ_OK || *launched) return rc;
    }
    return launch_mma_cfg<AT, BITS, GS, 1, 4>(a, bt, pairs, 2, st, launched);
}

static int launch_mma_any(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, int pairs,
                          cudaStream_t st, bool* launched) {
    int rc = JQ_OK;
#define JQ_GEMV_CASE(B, GSZ)                                                                      \
    if (bits == B && gs == GSZ) {                                                                 \
        rc = (act_dtype == JQ_BF16) ? launch_mma<__nv_bfloat16, B, GSZ>(a, bt, pairs, st, launched) \
                                    : launch_mma<__half, B, GSZ>(a, bt, pairs, st, launched);      \
    }
    JQ_GEMV_CASE(2, 64) JQ_GEMV_CASE(3, 64) JQ_GEMV_CASE(4, 64) JQ_GEMV_CASE(6, 64) JQ_GEMV_CASE(8, 64)
    JQ_GEMV_CASE(2, 128) JQ_GEMV_CASE(3, 128) JQ_GEMV_CASE(4, 128) JQ_GEMV_CASE(6, 128) JQ_GEMV_CASE(8, 128)
#undef JQ_GEMV_CASE
    return rc;
}

// One or several matrices that share x: count entries of (codes, scales, biases, y, N, ldy).  Entries
// that qualify for a fast kernel go out as ONE launch; the general kernel takes them one by one.
struct GemvItems {
    int count;
    const uint32_t* codes[GEMV_MAX_FUSE];
    const void* scales[GEMV_MAX_FUSE];
    const void* biases[GEMV_MAX_FUSE];
    void* y[GEMV_MAX_FUSE];
    int64_t N[GEMV_MAX_FUSE], ldy[GEMV_MAX_FUSE];
};

// ns (optional, M == 1): the activation row does not exist yet; it is rms_norm(ns->res + sum of ns->k rows of ns->y)
// and belongs at x (== ns->out).  The one-row kernel forms it inside its launch; for any other kernel the norm
// goes out as its own launch first.
int qgemv_dispatch_items(const void* x, int x_dtype, int64_t M, int64_t ldx, const GemvItems& it, int sidecar_dtype,
                         int64_t K, int bits, int gs, int y_dtype, int flags, cudaStream_t st, const NormSrc* ns = nullptr) {
    JQ_REQUIRE(it.count >= 1 && it.count <= GEMV_MAX_FUSE, JQ_EINVAL, "bad item count %d", it.count);
    JQ_REQUIRE(valid_dtype(x_dtype) && valid_dtype(sidecar_dtype) && valid_dtype(y_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(M >= 0 && M <= JQ_QGEMV_MAX_M, JQ_EINVAL, "qgemv takes 0 <= M <= %d rows, got %lld", JQ_QGEMV_MAX_M,
               (long long)M);
    bool fast = !force_simple() && (gs == 64 || gs == 128) && x_dtype != JQ_F32 && sidecar_dtype == x_dtype &&
                y_dtype == x_dtype && ((K * bits / 8) % 16 == 0) && aligned(x, 16) && (ldx % 8 == 0) &&
                (gs > 0 && (K / gs) % 4 == 0) && bits != 5;
    GemvItems live = {};      // entries with rows to compute
    for (int i = 0; i < it.count; ++i) {
        int rc = check_quant_shape(it.N[i], K, bits, gs);
        if (rc != JQ_OK) return rc;
        if (M == 0 || it.N[i] == 0) continue;
        JQ_REQUIRE(K > 0, JQ_EINVAL, "K must be positive");
        JQ_REQUIRE(x && it.codes[i] && it.scales[i] && it.biases[i] && it.y[i], JQ_EINVAL, "null pointer");
        JQ_REQUIRE(ldx >= K && it.ldy[i] >= it.N[i], JQ_EINVAL, "leading dimension too small");
        JQ_REQUIRE(it.N[i] < (1ll << 31) && K < (1ll << 31), JQ_EUNSUPPORTED, "dimension too large");
        fast = fast && aligned(it.codes[i], 16) && aligned(it.scales[i], 8) && aligned(it.biases[i], 8);
        const int j = live.count++;
        live.codes[j] = it.codes[i]; live.scales[j] = it.scales[i]; live.biases[j] = it.biases[i];
        live.y[j] = it.y[i]; live.N[j] = it.N[i]; live.ldy[j] = it.ldy[i];
    }
    if (live.count == 0) return JQ_OK;
    const int kern = gemv_kernel_choice();
    for (int64_t m0 = 0; m0 < M; m0 += 8) {
        GemvArgs a = {};
        a.x = (const char*)x + m0 * ldx * dtype_size(x_dtype);
        a.K = K; a.ldx = ldx;
        a.M = (int)((M - m0) < 8 ? (M - m0) : 8);
        a.G = (int)(K / gs);
        a.pdl = (flags & JQ_GEMV_STATIC_WEIGHTS) ? 1 : 0;
        a.x_div = 1; a.ksplit = 1;
        GemvBatch bt = {};
        bt.count = live.count;
        for (int i = 0; i < live.count; ++i) {
            bt.codes[i] = live.codes[i]; bt.scales[i] = live.scales[i]; bt.biases[i] = live.biases[i];
            bt.y[i] = (char*)live.y[i] + m0 * live.ldy[i] * dtype_size(y_dtype);
            bt.N[i] = live.N[i]; bt.ldy[i] = live.ldy[i];
        }
        a.codes = bt.codes[0]; a.scales = bt.scales[0]; a.biases = bt.biases[0]; a.y = bt.y[0];
        a.N = bt.N[0]; a.ldy = bt.ldy[0];
        bool launched = false;
        int rc = JQ_OK;
        // Measured choice on B200 (CUDA events, overlapped launches, working set >> L2):
        //   2-, 4- and 8-bit, M <= 2: persistent integer warp-MMA kernel (22016x4096 2-bit: 12.0 us against
        //          16.2 us for the per-tile integer kernel; 14336x4096 4-bit: 10.2 us and 32000x4096 8-bit:
        //          24.1 us against 14.1 us and 31.1 us for the tensor-memory kernel);
        //   4- and 8-bit, M > 2: tensor-memory kernel;
        //   3/6-bit, M > 2 with 2-bit: bf16 warp-MMA kernel.
        const bool narrow = (bits == 2 || bits == 4 || bits == 8) && a.M <= 2;
        //   one activation row, 2-, 4-, 6- and 8-bit: item-streaming integer kernel.  6-bit 32000x4096: 25.5 us
        //          against 38 us for the bf16 warp-MMA kernel; on the other widths it ties with the persistent
        //          kernel (12288x4096 8-bit 11.9 / 11.4 us, 22016x4096 2-bit 11.3 / 11.0 us, 14336x4096 4-bit
        //          9.8 / 10.2 us; the whole config-2 decode stream 1.105 / 1.108 ms)
        if (fast && (kern == 5 || (kern == 0 && a.M == 1))) {
            if (ns) { a.norm_res = ns->res; a.norm_y = ns->y; a.norm_ldy = ns->ldy; a.norm_k = ns->k; a.norm_eps = ns->eps; }
            rc = launch_one_kernel(a, bt, x_dtype, bits, gs, st, &launched);
            if (rc != JQ_OK) return rc;
            a.norm_res = nullptr;
        }
        if (ns && !launched) {
            rc = jq_residual_rmsnorm(ns->res, ns->y, nullptr, ns->k, 1, K, ns->eps, ns->out, x_dtype, (jq_stream_t)st);
            if (rc != JQ_OK) return rc;
        }
        if (fast && !launched && (kern == 4 || (kern == 0 && narrow))) {
            rc = launch_pint_kernel(a, bt, x_dtype, bits, gs, st, &launched);
            if (rc != JQ_OK) return rc;
        }
        if (fast && !launched && (kern == 3 || (kern == 0 && bits != 2))) {
            rc = launch_tc_kernel(a, bt, x_dtype, bits, gs, st, &launched);
            if (rc != JQ_OK) return rc;
        }
        if (fast && !launched) {
            rc = launch_mma_any(a, bt, x_dtype, bits, gs, 1, st, &launched);
            if (rc != JQ_OK) return rc;
        }
        if (!launched) {
            for (int i = 0; i < bt.count; ++i) {
                GemvArgs s1 = a;
                s1.codes = bt.codes[i]; s1.scales = bt.scales[i]; s1.biases = bt.biases[i]; s1.y = bt.y[i];
                s1.N = bt.N[i]; s1.ldy = bt.ldy[i]; s1.nbuf = 0;
                const unsigned grid = (unsigned)((s1.N + 3) / 4);
                JQ_DISPATCH_BITS(bits, B,
                    (qgemv_simple_kernel<B><<<grid, 128, 0, st>>>(s1, x_dtype, sidecar_dtype, y_dtype, gs)))
                rc = check_launch("qgemv (general)");
                if (rc != JQ_OK) return rc;
            }
        }
    }
    return JQ_OK;
}

int qgemv_dispatch(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
                   const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int gs, void* y,
                   int y_dtype, int64_t ldy, int flags, cudaStream_t st) {
    GemvItems it = {};
    it.count = 1;
    it.codes[0] = codes; it.scales[0] = scales; it.biases[0] = biases; it.y[0] = y; it.N[0] = N; it.ldy[0] = ldy;
    return qgemv_dispatch_items(x, x_dtype, M, ldx, it, sidecar_dtype, K, bits, gs, y_dtype, flags, st);
}

// Routed-expert mat-vec for few (token, slot) pairs: y[p] = deq(W[expert[p]]) . x[p / x_div].
int gather_qgemv_dispatch(const void* x, int act_dtype, int64_t ldx, int x_div, const int32_t* pair_expert,
                          int64_t pairs, const uint32_t* const* codes_tab, const void* const* scales_tab,
                          const void* const* biases_tab, const int32_t* bits_tab, int num_experts, int sidecar_dtype,
                          int64_t N, int64_t K, int bits, int gs, void* y, int64_t ldy, cudaStream_t st,
                          const uint32_t* const* codes_tab2 = nullptr, const void* const* scales_tab2 = nullptr,
                          const void* const* biases_tab2 = nullptr, void* y2 = nullptr, int flags = 0,
                          int expert_base = 0) {
    int rc = check_quant_shape(N, K, bits, gs);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(valid_dtype(act_dtype) && valid_dtype(sidecar_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(pairs >= 0 && pairs < 65536, JQ_EINVAL, "gather mat-vec takes fewer than 65536 pairs, got %lld",
               (long long)pairs);
    if (pairs == 0 || N == 0) return JQ_OK;
    JQ_REQUIRE(K > 0 && x_div > 0 && num_experts > 0, JQ_EINVAL, "bad argument");
    JQ_REQUIRE(x && pair_expert && codes_tab && scales_tab && biases_tab && y, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(ldx >= K && ldy >= N, JQ_EINVAL, "leading dimension too small");
    JQ_REQUIRE(N < (1ll << 31) && K < (1ll << 31), JQ_EUNSUPPORTED, "dimension too large");
    GemvArgs a = {};
    a.x = x; a.y = y;
    a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.M = 1; a.G = (int)(K / gs);
    a.pair_expert = pair_expert; a.codes_tab = codes_tab; a.scales_tab = scales_tab; a.biases_tab = biases_tab;
    a.bits_tab = bits_tab; a.x_div = x_div; a.num_experts = num_experts; a.ksplit = 1;
    JQ_REQUIRE((codes_tab2 == nullptr) == (y2 == nullptr) && (codes_tab2 == nullptr || (scales_tab2 && biases_tab2)), JQ_EINVAL,
               "the second bank needs its three tables and its output");
    a.codes_tab2 = codes_tab2; a.scales_tab2 = scales_tab2; a.biases_tab2 = biases_tab2; a.y2 = y2;
    a.pdl = (flags & JQ_GEMV_STATIC_WEIGHTS) ? 1 : 0;
    a.expert_base = expert_base;
    GemvBatch bt = {};        // one entry: row count and output of every pair's matrix
    bt.count = 1; bt.y[0] = y; bt.N[0] = N; bt.ldy[0] = ldy;
    // the per-expert base pointers are not known on the host: the fast path relies on the caller's
    // promise (checked for the row pitch here) that every expert tensor is 16-byte aligned
    const bool fast = !force_simple() && (gs == 64 || gs == 128) && act_dtype != JQ_F32 && sidecar_dtype == act_dtype &&
                      ((K * bits / 8) % 16 == 0) && aligned(x, 16) && (ldx % 8 == 0) && ((K / gs) % 4 == 0) && bits != 5;
    bool launched = false;
    // Up to 16 pairs (one or two tokens of a top-8 model; a row per x_div pairs): the item-streaming integer kernel,
    // all matrices in one launch.  Other cases (more pairs, per-expert widths): the bf16 warp-MMA kernel.
    const bool sparse = (flags & JQ_GATHER_FEW_LOCAL) != 0;
    if (fast && !bits_tab && (pairs <= 16 || sparse) && x_div >= 1 && gemv_kernel_choice() != 1) {
        rc = launch_gather_one(x, nullptr, nullptr, 0.f, ldx, x_div, pair_expert, (int)pairs,
                               codes_tab2 ? 2 : 1, codes_tab, scales_tab, biases_tab, codes_tab2, scales_tab2, biases_tab2,
                               num_experts, expert_base, act_dtype, N, K, bits, gs, y, y2, ldy, a.pdl != 0, st, &launched,
                               sparse);
        if (rc != JQ_OK) return rc;
    }
    if (fast && !launched) {
        rc = launch_mma_any(a, bt, act_dtype, bits, gs, (int)pairs, st, &launched);
        if (rc != JQ_OK) return rc;
    }
    if (!launched) {
        dim3 grid((unsigned)((N + 3) / 4), (unsigned)pairs, codes_tab2 ? 2u : 1u);
        JQ_DISPATCH_BITS(bits, B,
            (qgemv_simple_kernel<B><<<grid, 128, 0, st>>>(a, act_dtype, sidecar_dtype, act_dtype, gs)))
        rc = check_launch("gather qgemv (general)");
        if (rc != JQ_OK) return rc;
    }
    return JQ_OK;
}

// Fused form of several mat-vecs: consecutive entries that share x, K, the bit width and the group size
// become one launch (at most GEMV_MAX_FUSE matrices each).
int qgemv_dispatch_batched(const JqGemvDesc* descs, int count, int64_t M, int act_dtype, int sidecar_dtype, int flags,
                           cudaStream_t st, const NormSrc* ns = nullptr) {
    JQ_REQUIRE(count >= 0 && count <= JQ_QGEMV_MAX_BATCH, JQ_EINVAL, "count must be in [0, %d]", JQ_QGEMV_MAX_BATCH);
    JQ_REQUIRE(count == 0 || descs, JQ_EINVAL, "null descriptor table");
    int i = 0;
    while (i < count) {
        const JqGemvDesc& d0 = descs[i];
        GemvItems it = {};
        int j = i;
        while (j < count && it.count < GEMV_MAX_FUSE) {
            const JqGemvDesc& d = descs[j];
            if (d.x != d0.x || d.ldx != d0.ldx || d.K != d0.K || d.bits != d0.bits || d.group_size != d0.group_size) break;
            const int k = it.count++;
            it.codes[k] = d.codes; it.scales[k] = d.scales; it.biases[k] = d.biases; it.y[k] = d.y;
            it.N[k] = d.N; it.ldy[k] = d.ldy;
            ++j;
        }
        int rc = qgemv_dispatch_items(d0.x, act_dtype, M, d0.ldx, it, sidecar_dtype, d0.K, d0.bits, d0.group_size,
                                      act_dtype, flags, st, i == 0 ? ns : nullptr);
        if (rc != JQ_OK) return rc;
        i = j;
    }
    return JQ_OK;
}

}  // namespace jq

extern "C" {

int jq_gather_qgemv(const void* x, int act_dtype, int64_t ldx, int x_div, const int32_t* pair_expert, int64_t pairs,
                    const uint32_t* const* codes_tab, const void* const* scales_tab, const void* const* biases_tab,
                    const int32_t* bits_tab, int num_experts, int sidecar_dtype, int64_t N, int64_t K, int bits,
                    int group_size, void* y, int64_t ldy, jq_stream_t stream) {
    return jq::gather_qgemv_dispatch(x, act_dtype, ldx, x_div, pair_expert, pairs, codes_tab, scales_tab, biases_tab,
                                     bits_tab, num_experts, sidecar_dtype, N, K, bits, group_size, y, ldy,
                                     (cudaStream_t)stream);
}

int jq_gather_qgemv2(const void* x, int act_dtype, int64_t ldx, int x_div, const int32_t* pair_expert, int64_t pairs,
                     const uint32_t* const* codes_tab, const void* const* scales_tab, const void* const* biases_tab,
                     const uint32_t* const* codes_tab2, const void* const* scales_tab2, const void* const* biases_tab2,
                     const int32_t* bits_tab, int num_experts, int sidecar_dtype, int64_t N, int64_t K, int bits,
                     int group_size, void* y, void* y2, int64_t ldy, int expert_base, int flags, jq_stream_t stream) {
    return jq::gather_qgemv_dispatch(x, act_dtype, ldx, x_div, pair_expert, pairs, codes_tab, scales_tab, biases_tab,
                                     bits_tab, num_experts, sidecar_dtype, N, K, bits, group_size, y, ldy,
                                     (cudaStream_t)stream, codes_tab2, scales_tab2, biases_tab2, y2, flags, expert_base);
}

int jq_gather_qgemv_swiglu(const void* gate, const void* up, int act_dtype, int64_t ld_in, const float* weights,
                           float limit, const int32_t* pair_expert, int64_t pairs, const uint32_t* const* codes_tab,
                           const void* const* scales_tab, const void* const* biases_tab, const int32_t* bits_tab,
                           int num_experts, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y,
                           int64_t ldy, int expert_base, int flags, void* h_scratch, jq_stream_t stream) {
    using namespace jq;
    int rc = check_quant_shape(N, K, bits, group_size);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(act_dtype == JQ_BF16 || act_dtype == JQ_F16, JQ_EINVAL, "16-bit activations only");
    JQ_REQUIRE(pairs >= 0 && pairs < 65536, JQ_EINVAL, "fewer than 65536 pairs");
    if (pairs == 0 || N == 0) return JQ_OK;
    JQ_REQUIRE(gate && up && pair_expert && codes_tab && scales_tab && biases_tab && y, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(ld_in >= K && ldy >= N, JQ_EINVAL, "leading dimension too small");
    cudaStream_t st = (cudaStream_t)stream;
    const bool fast = (group_size == 64 || group_size == 128) && sidecar_dtype == act_dtype && !bits_tab &&
                      aligned(gate, 16) && aligned(up, 16) && (ld_in % 8 == 0) && gemv_kernel_choice() != 1;
    bool launched = false;
    const bool sparse = (flags & JQ_GATHER_FEW_LOCAL) != 0;
    if (fast && (pairs <= 16 || sparse)) {
        rc = launch_gather_one(gate, up, weights, limit, ld_in, 1, pair_expert, (int)pairs, 1, codes_tab, scales_tab,
                               biases_tab, nullptr, nullptr, nullptr, num_experts, expert_base, act_dtype, N, K, bits,
                               group_size, y, nullptr, ldy, (flags & JQ_GEMV_STATIC_WEIGHTS) != 0, st, &launched, sparse);
        if (rc != JQ_OK) return rc;
    }
    if (launched) return JQ_OK;
    JQ_REQUIRE(h_scratch != nullptr, JQ_EWORKSPACE,
               "this shape takes the two-launch path: pass h_scratch, [pairs, K] of the activation type");
    rc = jq_moe_swiglu(gate, up, ld_in, weights, nullptr, nullptr, h_scratch, K, K, pairs, limit, act_dtype, stream);
    if (rc != JQ_OK) return rc;
    return gather_qgemv_dispatch(h_scratch, act_dtype, K, 1, pair_expert, pairs, codes_tab, scales_tab, biases_tab, bits_tab,
                                 num_experts, sidecar_dtype, N, K, bits, group_size, y, ldy, st, nullptr, nullptr, nullptr,
                                 nullptr, flags, expert_base);
}

int jq_qgemv(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
             const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y,
             int y_dtype, int64_t ldy, jq_stream_t stream) {
    return jq::qgemv_dispatch(x, x_dtype, M, ldx, codes, scales, biases, sidecar_dtype, N, K, bits, group_size, y,
                              y_dtype, ldy, 0, (cudaStream_t)stream);
}

int jq_qgemv_ex(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
                const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y,
                int y_dtype, int64_t ldy, int flags, jq_stream_t stream) {
    return jq::qgemv_dispatch(x, x_dtype, M, ldx, codes, scales, biases, sidecar_dtype, N, K, bits, group_size, y,
                              y_dtype, ldy, flags, (cudaStream_t)stream);
}

int jq_qgemv_batched(const JqGemvDesc* descs, int count, int64_t M, int act_dtype, int sidecar_dtype,
                     jq_stream_t stream) {
    return jq::qgemv_dispatch_batched(descs, count, M, act_dtype, sidecar_dtype, 0, (cudaStream_t)stream);
}

int jq_qgemv_batched_ex(const JqGemvDesc* descs, int count, int64_t M, int act_dtype, int sidecar_dtype, int flags,
                        jq_stream_t stream) {
    return jq::qgemv_dispatch_batched(descs, count, M, act_dtype, sidecar_dtype, flags, (cudaStream_t)stream);
}

int jq_qgemv_batched_norm(const void* res, const void* y, int64_t ldy, int k, float eps, void* x_out,
                          const JqGemvDesc* descs, int count, int act_dtype, int sidecar_dtype, int flags,
                          jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(count >= 1 && count <= JQ_QGEMV_MAX_BATCH && descs, JQ_EINVAL, "count must be in [1, %d]", JQ_QGEMV_MAX_BATCH);
    JQ_REQUIRE(act_dtype == JQ_BF16 || act_dtype == JQ_F16, JQ_EINVAL, "16-bit activations only");
    JQ_REQUIRE(res && y && x_out && k >= 1, JQ_EINVAL, "null pointer or k < 1");
    const int64_t K = descs[0].K;
    JQ_REQUIRE(K > 0 && K <= 4096 && K % 8 == 0 && ldy >= K && ldy % 8 == 0, JQ_EUNSUPPORTED,
               "rows of at most 4096 elements, a multiple of 8, ldy %% 8 == 0");
    JQ_REQUIRE(aligned(res, 16) && aligned(y, 16) && aligned(x_out, 16), JQ_EINVAL, "res, y and x_out must be 16-byte aligned");
    for (int i = 0; i < count; ++i)
        JQ_REQUIRE(descs[i].x == x_out && descs[i].K == K, JQ_EINVAL, "every entry reads x_out (desc %d does not)", i);
    JQ_REQUIRE(x_out != res && x_out != y, JQ_EINVAL, "x_out must not overlap res or y (every CTA reads them)");
    // the separate norm launch (other widths) reads contiguous rows; only the fused read takes a leading dimension
    JQ_REQUIRE(k == 1 || ldy == K, JQ_EUNSUPPORTED, "y rows must be contiguous (ldy == K) when k > 1");
    NormSrc ns = {res, y, ldy, k, eps, x_out};
    return qgemv_dispatch_batched(descs, count, 1, act_dtype, sidecar_dtype, flags, (cudaStream_t)stream, &ns);
}

int jq_device_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, jq::g_timeout_flag, sizeof(int)) != cudaSuccess)
        return jq::fail(JQ_ECUDA, "could not read the device status word");
    if (v != 0)
        return jq::fail(JQ_ETIMEOUT, "a bounded device-side wait ran out:%s%s",
                        (v & jq::JQ_STATUS_LOCAL_WAIT) ? " a kernel's own pipeline or grid barrier" : "",
                        (v & jq::JQ_STATUS_PEER_WAIT) ? " a rank of the expert-parallel exchange did not arrive" : "");
    return JQ_OK;
}

int jq_device_status_clear(void) {
    const int v = 0;
    if (cudaMemcpyToSymbol(jq::g_timeout_flag, &v, sizeof(int)) != cudaSuccess)
        return jq::fail(JQ_ECUDA, "could not clear the device status word");
    return JQ_OK;
}

}  // extern "C"
