// K2, integer warp-MMA form: decode-shaped quantized mat-vec  y[M,N] = x[M,K] . deq(W)[N,K]^T, M <= 2,
// with the codes as unsigned bytes in mma.sync.m16n8k32 (u8 x s8 -> s32) and the activations as
// signed 8-bit limbs.
//
// Bound: HBM bandwidth.  Algorithmic bytes per launch =
//     N*K*bits/8 (codes) + N*(K/gs)*2*2 (scales, biases) + M*K*2 + M*N*2.
//
// Arithmetic: the one of the tensor-memory kernel (jq_qgemv_tc.cu).  Per quantization group g and
// activation row m,  x[k] ~ e(g,m) * xi[k]  with a shared power-of-two e and |xi| <= 2^22, and
// xi = l0 + 256*l1 + 65536*l2 in signed digits; the MMA returns the exact integer sums
// D_l = sum_k q[k] * l_l[k], and  acc += e * ( s * (D0 + 256*D1 + 65536*D2) + b * sum_k xi[k] ).
//
// Structure: the one of the warp-MMA kernel of jq_qgemv.cu (one CTA = 16*MT weight rows x all of K,
// NW warps that split K into private cp.async stages of codes + scales/biases), with two changes:
//   * the activations are converted to limbs once per CTA (all warps, after griddepcontrol.wait)
//     into shared memory, together with the per-group (e, sum xi) table; a stage carries weights only;
//   * the inner loop needs no dequantization arithmetic for 8-bit codes and one AND (+ shift) per four
//     codes for 4- and 2-bit codes: bytes go straight into the A fragment.  The 16 codes a lane owns in a
//     64-code block are fed in the order that is cheapest to unpack; the limbs are stored in the same
//     order.  Columns of the MMA: limbs l0,l1,l2 of activation row 0 in columns 0-2, of row 1 in 4-6.
#include <cstdlib>

#include "jq_mma.cuh"
#include "jq_qgemv.cuh"

namespace jq {

namespace imv {

// m16n8k32, A unsigned 8-bit (row-major fragment), B signed 8-bit, s32 accumulate
__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma0(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                      uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// The lane's 16 codes (u[], code j at bit j*BITS) -> 4 registers of 4 bytes.  Byte order:
//   8-bit: natural;  4-bit: per 8 codes the even ones, then the odd ones;  2-bit: code j is byte j>>2 of
//   register j&3.  (The limbs of x use the same order: see prepare_limbs.)
template <int BITS>
__device__ __forceinline__ void to_bytes(const uint32_t (&u)[Unit<BITS>::WORDS], uint32_t (&r)[4]) {
    if constexpr (BITS == 8) {
        r[0] = u[0]; r[1] = u[1]; r[2] = u[2]; r[3] = u[3];
    } else if constexpr (BITS == 4) {
        r[0] = u[0] & 0x0F0F0F0Fu; r[1] = (u[0] >> 4) & 0x0F0F0F0Fu;
        r[2] = u[1] & 0x0F0F0F0Fu; r[3] = (u[1] >> 4) & 0x0F0F0F0Fu;
    } else {
        static_assert(BITS == 2, "widths of this kernel: 2, 4, 8");
        r[0] = u[0] & 0x03030303u; r[1] = (u[0] >> 2) & 0x03030303u;
        r[2] = (u[0] >> 4) & 0x03030303u; r[3] = (u[0] >> 6) & 0x03030303u;
    }
}

template <int BITS, int GS, int MT> struct Geom {
    static constexpr int KT = (BITS <= 4 || GS == 128) ? 512 : 256;   // codes per row and stage
    static constexpr int ROWS = 16 * MT;
    static constexpr int PAD = BITS == 2 ? 4 : BITS == 8 ? 16 : 8;    // conflict-free unit loads
    static constexpr int RS = KT * BITS / 32 + PAD;      // code row stride, words
    static constexpr int NG = KT / GS;                   // groups per stage (4 or 8)
    static constexpr int NQ = NG / 4;                    // 8-byte sidecar quads per row
    static constexpr int NGP = NG + 1;                   // padded sidecar row stride, float2
    static constexpr int SC_OFF = ROWS * RS * 4;         // float2 (s, b) [ROWS][NGP]
    static constexpr int STAGE = SC_OFF + ROWS * NGP * 8;
};

// CTA-wide shared memory before the per-warp stages: [128 zero bytes][tab: G x 2 float2][limbs: 3*M rows]
__host__ __device__ inline int limb_stride(int K) { return K + 64; }     // bytes per limb row
__host__ __device__ inline int head_bytes(int K, int G, int M) {
    return 128 + G * 16 + ((3 * M * limb_stride(K) + 127) / 128) * 128;
}

template <typename AT, int BITS, int GS, int MT, int NW>
__global__ void __launch_bounds__(NW * 32)
qgemv_imma_kernel(const GemvArgs a, const GemvBatch bt) {
    using A = Act<AT>;
    using Geo = Geom<BITS, GS, MT>;
    static_assert(NW == 4 || NW == 8, "4 or 8 warps split K");
    constexpr int ROWS = Geo::ROWS, KT = Geo::KT, RS = Geo::RS, NG = Geo::NG, NQ = Geo::NQ, NGP = Geo::NGP;
    constexpr int BPG = GS / 64;
    constexpr int UW = Unit<BITS>::WORDS;
    constexpr int THREADS = NW * 32;

    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int K = (int)a.K, G = a.G, M = a.M, nbuf = a.nbuf;
    const int nst = (K + KT - 1) / KT;
    const int64_t rowbytes = a.K * BITS / 8;
    const int LS = limb_stride(K);
    uint8_t* zero = smem;
    float2* tab = reinterpret_cast<float2*>(smem + 128);                 // [G][2]
    uint8_t* limbs = smem + 128 + G * 16;                                // [3*M][LS]
    uint8_t* mybuf = smem + head_bytes(K, G, M) + (size_t)warp * nbuf * Geo::STAGE;
    const uint16_t* xs16 = reinterpret_cast<const uint16_t*>(a.x);
    int mi = 0, blk0 = 0;                                                // matrix of a fused launch
    while (mi + 1 < bt.count && (int)blockIdx.x >= bt.blk_end[mi]) { blk0 = bt.blk_end[mi]; ++mi; }
    const int64_t N = bt.N[mi], ldy = bt.ldy[mi];
    const int64_t n0 = (int64_t)((int)blockIdx.x - blk0) * ROWS;
    const int rows_valid = (int)min((int64_t)ROWS, N - n0);
    const uint16_t* sc16 = reinterpret_cast<const uint16_t*>(bt.scales[mi]);
    const uint16_t* bi16 = reinterpret_cast<const uint16_t*>(bt.biases[mi]);
    uint16_t* y16 = reinterpret_cast<uint16_t*>(bt.y[mi]);

    // ---- stage copies (weights only): 16 bytes per lane and instruction ---------------------------------
    const uint8_t* code_base = reinterpret_cast<const uint8_t*>(bt.codes[mi]) + n0 * rowbytes;
    auto issue_codes = [&](int st, int b) {
        if (st < nst) {
            const int k0 = st * KT;
            const int kc = min(KT, K - k0);
            uint8_t* buf = mybuf + (size_t)b * Geo::STAGE;
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
    // scales/biases of a stage: pair index -> (row, quad of 4 groups), one 8-byte load each
    constexpr int SCP = (ROWS * NQ + 31) / 32;
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
                dst[0] = make_float2(A::lo_f32(sv[i].x), A::lo_f32(bv[i].x));
                dst[1] = make_float2(A::hi_f32(sv[i].x), A::hi_f32(bv[i].x));
                dst[2] = make_float2(A::lo_f32(sv[i].y), A::lo_f32(bv[i].y));
                dst[3] = make_float2(A::hi_f32(sv[i].y), A::hi_f32(bv[i].y));
            }
        }
    };

    // Weights first (static by contract): under programmatic dependent launch they stream while the
    // predecessor still runs; the activations are touched only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
    for (int i = 0; i < GEMV_MAX_NBUF; ++i)
        if (i < nbuf) {
            issue_codes(warp + i * NW, i);
            cp_async_commit();
        }
    fetch_sc(warp);
    if (tid < 32) reinterpret_cast<uint32_t*>(zero)[tid] = 0u;
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations -> limbs + per-group (e, sum xi), once per CTA ------------------------------------
    {
        constexpr int LPG = GS / 8;                      // eight activations per lane, LPG lanes per group
        constexpr int PF = 2;
        const int per_row = K / 8;
        const int items = M * per_row;                   // a multiple of 32
        for (int base0 = warp * 32; base0 < items; base0 += THREADS * PF) {
            uint4 rawv[PF];
#pragma unroll
            for (int i = 0; i < PF; ++i) {
                const int it = base0 + i * THREADS + lane;
                if (it < items) {
                    const int m = it / per_row;
                    rawv[i] = *reinterpret_cast<const uint4*>(xs16 + (int64_t)m * a.ldx + (it - m * per_row) * 8);
                }
            }
#pragma unroll
            for (int i = 0; i < PF; ++i) {
                const int it = base0 + i * THREADS + lane;
                if (it >= items) break;                  // warp-uniform: items is a multiple of 32
                const int m = it / per_row;
                const int ko = it - m * per_row;         // octet of the row
                const uint32_t w[4] = {rawv[i].x, rawv[i].y, rawv[i].z, rawv[i].w};
                float v[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) { v[2 * j] = A::lo_f32(w[j]); v[2 * j + 1] = A::hi_f32(w[j]); }
                uint32_t amax = 0u;                      // largest magnitude, as bits (NaN/inf sort highest)
#pragma unroll
                for (int j = 0; j < 8; ++j) amax = max(amax, __float_as_uint(v[j]) & 0x7FFFFFFFu);
#pragma unroll
                for (int d = 1; d < LPG; d <<= 1) amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
                uint32_t eb = amax >> 23;
                const bool finite = eb != 255u;
                eb = max(eb, 21u);
                const float scale = __uint_as_float((275u - eb) << 23);      // 2^(21 - E)
                float e = __uint_as_float((eb - 21u) << 23);                 // 2^(E - 21)
                if (!finite) e = __uint_as_float(0x7FC00000u);               // non-finite input -> NaN output
                int xi[8];
                int sum = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { xi[j] = __float2int_rn(v[j] * scale); sum += xi[j]; }
#pragma unroll
                for (int d = 1; d < LPG; d <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
                const int u = ko >> 1, hf = ko & 1;      // 16-code unit of the row, which half of it
                uint8_t* dst = limbs + (size_t)(3 * m) * LS + u * 16;     // the unit in limb row 0 of this activation row
                store_limbs8<BITS>(dst, dst + LS, dst + 2 * LS, hf, xi);
                if ((ko & (LPG - 1)) == 0) tab[(ko / LPG) * 2 + m] = make_float2(e, (float)sum);
            }
        }
    }
    __syncthreads();

    // column g of the MMA: limb g & 3 of activation row g >> 2 (limb 3 does not exist: zeros)
    const int bm = g >> 2, bl = g & 3;
    const bool bvalid = bl < 3 && bm < M;
    const uint8_t* brow = bvalid ? limbs + (size_t)(3 * bm + bl) * LS + tig * 16 : zero;
    const int bstep = bvalid ? 64 : 0;                   // bytes per 64-code block
    // accumulators: rows g and g+8 of every row tile, activation row tig >> 1 (lanes tig, tig^1 hold the same)
    const int am = tig >> 1;
    float acc[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = 0.f;

    int it = 0;
    for (int st = warp; st < nst; st += NW, ++it) {
        const int b = it % nbuf;
        const int kc = min(KT, K - st * KT);
        const int nblk = kc >> 6;
        uint8_t* buf = mybuf + (size_t)b * Geo::STAGE;
        store_sc(buf);
        if (st + NW < nst) fetch_sc(st + NW);
        if (nbuf == 3) cp_async_wait<2>(); else cp_async_wait<1>();   // this stage's copies have landed
        __syncwarp();

        const uint32_t* c_lo = reinterpret_cast<const uint32_t*>(buf) + g * RS;
        const float2* pt = reinterpret_cast<const float2*>(buf + Geo::SC_OFF) + g * NGP;
        const uint8_t* bp = brow + (size_t)(bvalid ? st * KT : 0);
        const float2* tp = tab + (size_t)(st * NG) * 2 + (am < M ? am : 0);
        int cg[MT][4];
#pragma unroll 2
        for (int blk = 0; blk < nblk; ++blk) {
            const uint4 bq = *reinterpret_cast<const uint4*>(bp);
            bp += bstep;
            const bool first = (blk % BPG) == 0;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t ulo[UW], uhi[UW], rl[4], rh[4];
                load_unit<BITS>(c_lo + mt * 16 * RS, blk, tig, ulo);
                load_unit<BITS>(c_lo + (mt * 16 + 8) * RS, blk, tig, uhi);
                to_bytes<BITS>(ulo, rl);
                to_bytes<BITS>(uhi, rh);
                if (first) imma0(cg[mt], rl[0], rh[0], rl[1], rh[1], bq.x, bq.y);
                else imma(cg[mt], rl[0], rh[0], rl[1], rh[1], bq.x, bq.y);
                imma(cg[mt], rl[2], rh[2], rl[3], rh[3], bq.z, bq.w);
            }
            if (blk % BPG == BPG - 1) {
                const float2 es = *tp;                   // (e, sum xi) of this group and activation row
                tp += 2;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const float2 sb_lo = pt[mt * 16 * NGP], sb_hi = pt[(mt * 16 + 8) * NGP];
                    // even tig: columns (l0, l1); odd tig: (l2, none)
                    float p_lo, p_hi;
                    if ((tig & 1) == 0) {
                        p_lo = (float)(cg[mt][0] + 256 * cg[mt][1]);
                        p_hi = (float)(cg[mt][2] + 256 * cg[mt][3]);
                    } else {
                        p_lo = (float)cg[mt][0] * 65536.f;
                        p_hi = (float)cg[mt][2] * 65536.f;
                    }
                    p_lo += __shfl_xor_sync(0xFFFFFFFFu, p_lo, 1);
                    p_hi += __shfl_xor_sync(0xFFFFFFFFu, p_hi, 1);
                    acc[mt][0] = fmaf(es.x, fmaf(sb_lo.x, p_lo, sb_lo.y * es.y), acc[mt][0]);
                    acc[mt][1] = fmaf(es.x, fmaf(sb_hi.x, p_hi, sb_hi.y * es.y), acc[mt][1]);
                }
                ++pt;
            }
        }
        __syncwarp();
        issue_codes(st + nbuf * NW, b);
        cp_async_commit();     // always one group per iteration so that the group count stays uniform
    }
    cp_async_wait<0>();

    __syncthreads();   // every warp is done with its buffers
    float* red = reinterpret_cast<float*>(smem + head_bytes(K, G, M));   // overlays the (now idle) stage buffers
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 2; ++i) red[((warp * MT + mt) * 2 + i) * 32 + lane] = acc[mt][i];
    __syncthreads();
    if (warp < 2) {
        const int i = warp;                // warps 0, 1 <-> rows g, g+8
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) v += red[((w * MT + mt) * 2 + i) * 32 + lane];
            const int row = mt * 16 + g + 8 * i;
            if ((tig & 1) == 0 && am < M && row < rows_valid) y16[(int64_t)am * ldy + n0 + row] = A::from_f32(v);
        }
    }
}

template <typename AT, int BITS, int GS, int MT, int NW>
static int launch_cfg(GemvArgs a, GemvBatch bt, int nbuf, cudaStream_t st, bool* launched) {
    using Geo = Geom<BITS, GS, MT>;
    *launched = false;
    a.nbuf = nbuf;
    const size_t smem = (size_t)head_bytes((int)a.K, a.G, a.M) + (size_t)NW * nbuf * Geo::STAGE;
    if (smem > 200 * 1024) return JQ_OK;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_imma_kernel<AT, BITS, GS, MT, NW>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    int64_t grid = 0;
    for (int i = 0; i < bt.count; ++i) {
        grid += (bt.N[i] + 16 * MT - 1) / (16 * MT);
        bt.blk_end[i] = (int)grid;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemv_imma_kernel<AT, BITS, GS, MT, NW>, a, bt));
    *launched = true;
    return JQ_OK;
}

static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return (e && e[0] >= '0' && e[0] <= '9') ? atoi(e) : dflt;
}

// The limbs are prepared by every CTA for all of K, so the CTA should own enough rows to amortise
// that: 32 rows (MT=2) unless the grid would leave SMs empty; 8 warps when the rows are long.
template <typename AT, int BITS, int GS>
static int launch_shape(const GemvArgs& a, const GemvBatch& bt, cudaStream_t st, bool* launched) {
    const int sms = sm_count();
    int64_t tiles16 = 0;
    for (int i = 0; i < bt.count; ++i) tiles16 += (bt.N[i] + 15) / 16;
    constexpr int KT = Geom<BITS, GS, 1>::KT;
    const int nst = (int)((a.K + KT - 1) / KT);
    int mt = env_int("JANGQ_IMMA_MT", tiles16 >= (int64_t)2 * sms ? 2 : 1);
    int nw = env_int("JANGQ_IMMA_NW", (nst >= 16 && tiles16 <= (int64_t)4 * sms) ? 8 : 4);
    int nbuf = env_int("JANGQ_IMMA_NBUF", 2);
    if (mt != 2) mt = 1;
    if (nw != 8) nw = 4;
    if (nbuf != 3) nbuf = 2;
    if (mt == 2 && nw == 8) return launch_cfg<AT, BITS, GS, 2, 8>(a, bt, nbuf, st, launched);
    if (mt == 2) return launch_cfg<AT, BITS, GS, 2, 4>(a, bt, nbuf, st, launched);
    if (nw == 8) return launch_cfg<AT, BITS, GS, 1, 8>(a, bt, nbuf, st, launched);
    return launch_cfg<AT, BITS, GS, 1, 4>(a, bt, nbuf, st, launched);
}

}  // namespace imv

// Dense mat-vecs (one launch for all matrices of `bt`) on the integer warp-MMA kernel; *launched stays
// false when the shape does not fit it (widths other than 2/4/8, more than 2 activation rows).
int launch_imma_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                       bool* launched) {
    *launched = false;
    if (!(bits == 2 || bits == 4 || bits == 8) || a.M > 2 || a.K % 64 != 0) return JQ_OK;
    int rc = JQ_OK;
#define JQ_IMMA_CASE(B, GSZ)                                                                         \
    if (bits == B && gs == GSZ) {                                                                    \
        rc = (act_dtype == JQ_BF16) ? imv::launch_shape<__nv_bfloat16, B, GSZ>(a, bt, st, launched)  \
                                    : imv::launch_shape<__half, B, GSZ>(a, bt, st, launched);        \
    }
    JQ_IMMA_CASE(2, 64) JQ_IMMA_CASE(4, 64) JQ_IMMA_CASE(8, 64) JQ_IMMA_CASE(2, 128) JQ_IMMA_CASE(4, 128) JQ_IMMA_CASE(8, 128)
#undef JQ_IMMA_CASE
    return rc;
}

}  // namespace jq
