// K2, persistent integer warp-MMA form: decode-shaped quantized mat-vec  y[M,N] = x[M,K] . deq(W)[N,K]^T
// for 2-, 4- and 8-bit codes, M <= 2.
//
// Bound: HBM bandwidth on paper; in practice the instruction issue rate.  Algorithmic bytes per launch =
//     N*K*bits/8 (codes) + N*(K/gs)*2*2 (scales, biases) + M*K*2 + M*N*2.
// A 64-code block of 16 rows is 256 bytes of 2-bit codes; to stream them at the HBM rate an SM may spend
// about 34 warp instructions on it, so this kernel is written against an instruction budget.
//
// Arithmetic: per quantization group the
// activations are  x[k] ~ e * xi[k]  (e a power of two) with xi in three signed 8-bit limbs, the codes
// are the unsigned operand of mma.sync.m16n8k32 (u8 x s8 -> s32), the limb sums are exact integers and
//     acc += e * s * (D0 + 256 D1 + 65536 D2) + b * sum_k x[k].
// What is new:
//   * no shifts when unpacking: the codes of bit position p inside a byte stay where they are,
//     A = word & (mask << p) = 2^p * q, and the activations that meet them are scaled by 2^-p before they
//     are cut into limbs (exact: a power of two).  A 32-bit word of codes costs one AND per register.
//   * the limb sums of one lane (D0 + 256 D1 in even lanes of a quad, D2 in odd ones) are converted and
//     accumulated separately; the factor 65536 and the cross-lane add happen once per item.
//
// Structure: one persistent CTA per SM with NW warps.  The CTA owns a contiguous run of 16-row tiles,
// prepares the limbs once, and its warps walk the (tile, K-stage) items of that run round-robin:
// consecutive warps stream consecutive K-stages of the same rows.  An item is 16 rows x KT codes (2 KB of
// codes) plus the raw 2-byte scales and biases, copied by cp.async into a private ring of `nbuf` stages
// per warp: no register staging, no CTA barrier.  A warp adds the item's result to its own row sums in
// shared memory; one CTA barrier at the end, then the warps' sums are added and stored.
#include "jq_qgemv.cuh"
#include "jq_stream_dev.cuh"

namespace jq {

namespace pint {

constexpr int MAX_SMEM = 227 * 1024;

using namespace imma_ops;

__device__ __forceinline__ void cp_async_wait_dyn(int pending) {   // pending in 1..3
    if (pending == 1) cp_async_wait<1>();
    else if (pending == 2) cp_async_wait<2>();
    else cp_async_wait<3>();
}

template <int BITS, int GS> struct Geom {
    static constexpr int KT = BITS == 2 ? 512 : 256;      // codes per row and stage: 128 bytes (256 for 8-bit codes)
    static constexpr int NBLK = KT / 64;                  // 64-code blocks per stage
    static constexpr int ROWB = KT * BITS / 8;
    static constexpr int RSB = ROWB + (BITS == 2 ? 16 : BITS == 4 ? 32 : 64);   // padded row stride: conflict-free unit loads
    static constexpr int NG = KT / GS;                    // groups per stage: 8, 4 or 2
    static constexpr int SCB = NG * 2;                    // bytes of scales (or biases) per row and stage
    static constexpr int SC_OFF = 16 * RSB;               // scales [16 rows][NG] (2-byte), then biases [16][NG]
    static constexpr int STAGE = SC_OFF + 2 * 16 * SCB;
};

struct TileInfo {             // one 16-row tile of the CTA's run
    const uint8_t* codes;     // first row of the tile
    const uint16_t* scales;
    const uint16_t* biases;
    uint16_t* y;              // output element of the tile's first row, activation row 0
    int rows_valid, ldy;
    int pad[6];
};
static_assert(sizeof(TileInfo) == 64, "TileInfo is read with 16-byte loads");

// CTA-wide shared memory before the per-warp stages:
//   [64 zero bytes][tiles: TPC TileInfo][tab: G*2 float2][limbs: 3*M rows of K+64 bytes][ysum: NW * M * TPC*16 f32]
__host__ __device__ inline int limb_stride(int K) { return K + 64; }
__host__ __device__ inline int head_bytes(int K, int G, int M, int tpc, int nw) {
    return 64 + tpc * 64 + G * 16 + ((3 * M * limb_stride(K) + 127) / 128) * 128 + nw * M * tpc * 64;
}

template <typename AT, int BITS, int GS, int NW, bool M1>
__global__ void __launch_bounds__(NW * 32, 1)
qgemv_pint_kernel(const GemvArgs a, const GemvBatch bt) {
    using A = Act<AT>;
    using Geo = Geom<BITS, GS>;
    constexpr int KT = Geo::KT, NBLK = Geo::NBLK, ROWB = Geo::ROWB, RSB = Geo::RSB, NG = Geo::NG, SCB = Geo::SCB;
    constexpr int BPG = GS / 64;
    constexpr int UW = Unit<BITS>::WORDS;
    constexpr int THREADS = NW * 32;

    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int K = (int)a.K, G = a.G, M = a.M, TPC = a.ksplit;     // ksplit: 16-row tiles per CTA in this kernel
    const int nbuf = a.nbuf;
    const int nst = (K + KT - 1) / KT;
    const int64_t rowbytes = a.K * BITS / 8;
    const int LS = limb_stride(K);
    uint8_t* zero = smem;
    TileInfo* tiles = reinterpret_cast<TileInfo*>(smem + 64);
    float2* tab = reinterpret_cast<float2*>(smem + 64 + TPC * 64);                 // [G][2] (e, sum x)
    uint8_t* limbs = smem + 64 + TPC * 64 + G * 16;                                 // [3*M][LS]
    float* ysum = reinterpret_cast<float*>(limbs + ((3 * M * LS + 127) / 128) * 128);   // [NW][M][TPC*16]
    uint8_t* mybuf = smem + head_bytes(K, G, M, TPC, NW) + (size_t)warp * nbuf * Geo::STAGE;
    float* myy = ysum + (size_t)warp * M * TPC * 16;
    const uint16_t* xs16 = reinterpret_cast<const uint16_t*>(a.x);

    // tiles of all matrices of the launch are numbered consecutively; blk_end[i] = first tile after matrix i
    const int tile0 = (int)blockIdx.x * TPC;
    const int ntile = min(TPC, bt.blk_end[bt.count - 1] - tile0);
    if (tid < ntile) {
        const int gt = tile0 + tid;
        int mi = 0, first = 0;
        while (mi + 1 < bt.count && gt >= bt.blk_end[mi]) { first = bt.blk_end[mi]; ++mi; }
        const int64_t row0 = (int64_t)(gt - first) * 16;
        TileInfo ti = {};
        ti.codes = reinterpret_cast<const uint8_t*>(bt.codes[mi]) + row0 * rowbytes;
        ti.scales = reinterpret_cast<const uint16_t*>(bt.scales[mi]) + row0 * G;
        ti.biases = reinterpret_cast<const uint16_t*>(bt.biases[mi]) + row0 * G;
        ti.y = reinterpret_cast<uint16_t*>(bt.y[mi]) + row0;
        ti.rows_valid = (int)min((int64_t)16, bt.N[mi] - row0);
        ti.ldy = (int)bt.ldy[mi];
        tiles[tid] = ti;
    }
    if (tid < 16) reinterpret_cast<uint32_t*>(zero)[tid] = 0u;
    for (int i = tid; i < NW * M * TPC * 16; i += THREADS) ysum[i] = 0.f;
    __syncthreads();

    // copies of one item (tile lt, stage st): 16 code rows of 128 bytes + 16 x SCB bytes of scales and of biases
    constexpr int CPR = ROWB / 16, RPI = 32 / CPR;       // 8 (16) lanes per row, 4 (2) rows per instruction
    const int crow = lane / CPR, ccol = lane % CPR;
    const int64_t lane_src = (int64_t)crow * rowbytes + ccol * 16;
    const int lane_dst = crow * RSB + ccol * 16;
    const int srow = lane & 15, sarr = lane >> 4;
    auto issue = [&](int lt, int st, int b) {
        if (lt < ntile) {
            const int rows_valid = tiles[lt].rows_valid;
            const int kc = min(KT, K - st * KT);
            uint8_t* buf = mybuf + (size_t)b * Geo::STAGE;
            const uint8_t* src = tiles[lt].codes + (int64_t)st * ROWB + lane_src;
            uint8_t* dst = buf + lane_dst;
            const bool col_ok = ccol * 128 < kc * BITS;   // a short last stage has fewer 16-byte chunks per row
#pragma unroll
            for (int r = 0; r < 16; r += RPI) {
                if (col_ok && r + crow < rows_valid) cp_async16(dst, src);
                src += (int64_t)RPI * rowbytes;
                dst += RPI * RSB;
            }
            const uint16_t* sp = (sarr ? tiles[lt].biases : tiles[lt].scales) + (int64_t)min(srow, rows_valid - 1) * G + st * NG;
            uint8_t* sd = buf + Geo::SC_OFF + sarr * (16 * SCB) + srow * SCB;
            if constexpr (SCB == 16) {
                cp_async8(sd, sp);
                if (kc > KT / 2) cp_async8(sd + 8, sp + 4);
            } else if constexpr (SCB == 8) {
                cp_async8(sd, sp);
            } else {
                cp_async4(sd, sp);
            }
        }
    };

    // Weights first (static by contract): under programmatic dependent launch they stream while the
    // predecessor still runs; the activations are touched only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int it_lt = 0, it_st = warp;                  // (tile, stage) of the next item to copy
    auto advance = [&](int& lt, int& st) {
        st += NW;
        while (st >= nst) { st -= nst; ++lt; }
    };
    while (it_st >= nst) { it_st -= nst; ++it_lt; }
    int lt = it_lt, st = it_st;                   // (tile, stage) of the next item to compute
    issue(it_lt, it_st, 0);
    cp_async_commit();
    advance(it_lt, it_st);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations -> limbs + per-group (e, sum x), once per CTA --------------------------------------
    // The first load of x is issued here and the rest of the ring is filled while it is in flight.
    constexpr int LPG = GS / 16;                         // sixteen activations per lane, LPG lanes per group
    const int per_row = K / 16;                          // a multiple of LPG
    const int units = M * per_row;
    auto load_x = [&](int it, uint4& r0, uint4& r1) {
        r0 = make_uint4(0u, 0u, 0u, 0u);
        r1 = r0;
        if (it < units) {
            const int m = it / per_row;
            const uint4* p = reinterpret_cast<const uint4*>(xs16 + (int64_t)m * a.ldx + (size_t)(it - m * per_row) * 16);
            r0 = p[0]; r1 = p[1];
        }
    };
    uint4 xr0, xr1;
    if constexpr (M1) {
        // one activation row: 8 activations per thread (one 16-byte load, requested before the ring is filled)
        xr0 = tid < K / 8 ? stream::ld_cg16(xs16 + (size_t)tid * 8) : make_uint4(0u, 0u, 0u, 0u);
        xr1 = xr0;
    } else {
        load_x(warp * 32 + lane, xr0, xr1);
    }
    for (int i = 1; i < nbuf; ++i) {
        issue(it_lt, it_st, i);
        cp_async_commit();
        advance(it_lt, it_st);
    }
    if constexpr (M1) {
        stream::PrepSrc src;
        src.xs = xs16; src.have_pre = true; src.pre = xr0;
        stream::prep_limbs<AT, BITS, GS>(src, K, limbs, tab, LS, 0, tid, THREADS);
    } else {
        for (int base = warp * 32; base < units; base += THREADS) {
            const int it = base + lane;
            const bool live = it < units;
            const int m = live ? it / per_row : 0;
            const int U = it - m * per_row;              // 16-code unit of the row
            const uint4 r0 = xr0, r1 = xr1;
            if (base + THREADS < units) load_x(it + THREADS, xr0, xr1);
            const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float v[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[2 * j] = A::lo_f32(w[j]); v[2 * j + 1] = A::hi_f32(w[j]); }
            uint32_t amax = 0u;                          // largest magnitude, as bits (NaN/inf sort highest)
            float xs = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) { amax = max(amax, __float_as_uint(v[j]) & 0x7FFFFFFFu); xs += v[j]; }
#pragma unroll
            for (int d = 1; d < LPG; d <<= 1) {
                amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
                xs += __shfl_xor_sync(0xFFFFFFFFu, xs, d);
            }
            uint32_t eb = amax >> 23;
            const bool finite = eb != 255u;
            eb = max(eb, 21u);
            const float scale = __uint_as_float((275u - eb) << 23);      // 2^(21 - E): |x| * scale < 2^22
            float e = __uint_as_float((eb - 21u) << 23);                 // 2^(E - 21)
            if (!finite) e = __uint_as_float(0x7FC00000u);               // non-finite input -> NaN output
            uint32_t t[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                // the code that meets element j is scaled by 2^code_shift(j): scale the element down by it
                const float sj = scale * (1.f / (float)(1 << code_shift<BITS>(j)));
                t[j] = ((uint32_t)__float2int_rn(v[j] * sj) + 0x8080u) ^ 0x8080u;   // bytes 0..2: signed limbs
            }
            if (live) {
#pragma unroll
                for (int L = 0; L < 3; ++L) {
                    const uint32_t sel = ((4u + L) << 4) | L;            // byte L of both sources
                    uint32_t wd[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        wd[i] = __byte_perm(__byte_perm(t[elem<BITS>(i, 0)], t[elem<BITS>(i, 1)], sel),
                                            __byte_perm(t[elem<BITS>(i, 2)], t[elem<BITS>(i, 3)], sel), 0x5410);
                    *reinterpret_cast<uint4*>(limbs + (size_t)(3 * m + L) * LS + (size_t)U * 16) =
                        make_uint4(wd[0], wd[1], wd[2], wd[3]);
                }
                if ((U & (LPG - 1)) == 0) {
                    if constexpr (M1) {
                        tab[(U / LPG) * 2] = make_float2(e, 0.f);
                        tab[(U / LPG) * 2 + 1] = make_float2(0.f, xs);
                    } else {
                        tab[(U / LPG) * 2 + m] = make_float2(e, xs);
                    }
                }
            }
        }
    }
    __syncthreads();

    // column g of the MMA: limb g & 3 of activation row g >> 2 (limb 3 does not exist: zeros)
    const int bm = g >> 2, bl = g & 3;
    const bool bvalid = bl < 3 && bm < M;
    const uint8_t* brow = bvalid ? limbs + (size_t)(3 * bm + bl) * LS + tig * 16 : zero + tig * 16;
    // A lane's columns: even tig (l0, l1) -> D0 + 256 D1; odd tig (l2, none) -> D2, weighed 65536 at the end;
    // both belong to activation row tig >> 1.  With one activation row (M1) the lanes tig >= 2 have no
    // columns (their D is 0) and carry the bias term instead: a lane computes  acc += f * (D * el + xl)
    // with (f, el, xl) = (scale, e, 0) for tig < 2 and (bias, 0, sum x) for tig >= 2 -- the same two FMAs.
    const int am = tig >> 1;
    const float wl = M1 ? (tig == 1 ? 65536.f : tig == 3 ? 0.f : 1.f) : ((tig & 1) ? 65536.f : 1.f);
    const float2* tabm = tab + (M1 ? am : (am < M ? am : 0));
    const int sc_mine = Geo::SC_OFF + (M1 ? am * 16 * SCB : 0);       // M1: scales for tig < 2, biases for tig >= 2

    int b = 0;
    while (lt < ntile) {
        const uint8_t* buf = mybuf + (size_t)b * Geo::STAGE;
        cp_async_wait_dyn(nbuf - 1);                     // this item's copies have landed
        __syncwarp();

        const uint32_t* c_lo = reinterpret_cast<const uint32_t*>(buf + g * RSB);
        const uint32_t* c_hi = reinterpret_cast<const uint32_t*>(buf + (g + 8) * RSB);
        uint32_t sc_lo[NG / 2], sc_hi[NG / 2], bi_lo[NG / 2], bi_hi[NG / 2];     // packed 2-byte pairs
        auto load_pairs = [&](const uint8_t* p, uint32_t (&d)[NG / 2]) {
            if constexpr (NG == 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(p);
                d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
            } else if constexpr (NG == 4) {
                const uint2 v = *reinterpret_cast<const uint2*>(p);
                d[0] = v.x; d[1] = v.y;
            } else {
                d[0] = *reinterpret_cast<const uint32_t*>(p);
            }
        };
        load_pairs(buf + sc_mine + g * SCB, sc_lo);
        load_pairs(buf + sc_mine + (g + 8) * SCB, sc_hi);
        if constexpr (!M1) {
            load_pairs(buf + Geo::SC_OFF + 16 * SCB + g * SCB, bi_lo);
            load_pairs(buf + Geo::SC_OFF + 16 * SCB + (g + 8) * SCB, bi_hi);
        }
        const uint8_t* bp = brow + (bvalid ? st * KT : 0);
        const int bstep = bvalid ? 64 : 0;
        const float2* tp = tabm + (size_t)(st * NG) * 2;
        float acc_lo = 0.f, acc_hi = 0.f, accb_lo = 0.f, accb_hi = 0.f;
        int cg[4];
        auto block = [&](const int blk) {
            const uint4 bq = *reinterpret_cast<const uint4*>(bp + blk * bstep);
            uint32_t ulo[UW], uhi[UW], rl[4], rh[4];
            load_unit<BITS>(c_lo, blk, tig, ulo);
            load_unit<BITS>(c_hi, blk, tig, uhi);
            to_bytes<BITS>(ulo, rl);
            to_bytes<BITS>(uhi, rh);
            if (blk % BPG == 0) imma0(cg, rl[0], rh[0], rl[1], rh[1], bq.x, bq.y);
            else imma(cg, rl[0], rh[0], rl[1], rh[1], bq.x, bq.y);
            imma(cg, rl[2], rh[2], rl[3], rh[3], bq.z, bq.w);
            if (blk % BPG == BPG - 1) {
                const int gi = blk / BPG;
                const float2 tx = tp[gi * 2];
                const float s_lo = (gi & 1) ? A::hi_f32(sc_lo[gi >> 1]) : A::lo_f32(sc_lo[gi >> 1]);
                const float s_hi = (gi & 1) ? A::hi_f32(sc_hi[gi >> 1]) : A::lo_f32(sc_hi[gi >> 1]);
                const float d_lo = (float)(cg[0] + 256 * cg[1]);
                const float d_hi = (float)(cg[2] + 256 * cg[3]);
                if constexpr (M1) {                      // tx = (e, 0) or (0, sum x)
                    acc_lo = fmaf(s_lo, fmaf(d_lo, tx.x, tx.y), acc_lo);
                    acc_hi = fmaf(s_hi, fmaf(d_hi, tx.x, tx.y), acc_hi);
                } else {                                 // tx = (e, sum x) of the group and activation row
                    const float b_lo = (gi & 1) ? A::hi_f32(bi_lo[gi >> 1]) : A::lo_f32(bi_lo[gi >> 1]);
                    const float b_hi = (gi & 1) ? A::hi_f32(bi_hi[gi >> 1]) : A::lo_f32(bi_hi[gi >> 1]);
                    acc_lo = fmaf(s_lo * tx.x, d_lo, acc_lo);
                    acc_hi = fmaf(s_hi * tx.x, d_hi, acc_hi);
                    accb_lo = fmaf(b_lo, tx.y, accb_lo);
                    accb_hi = fmaf(b_hi, tx.y, accb_hi);
                }
            }
        };
        // only the last stage of 2-bit rows with 64-code groups can be short, and then it is half a stage
        constexpr bool TAIL = BITS == 2 && GS == 64;
        constexpr int HEAD_BLKS = TAIL ? NBLK / 2 : NBLK;
#pragma unroll
        for (int blk = 0; blk < HEAD_BLKS; ++blk) block(blk);
        if constexpr (TAIL) {
            if (K - st * KT >= KT) {
#pragma unroll
                for (int blk = HEAD_BLKS; blk < NBLK; ++blk) block(blk);
            }
        }
        {   // add the item to this warp's row sums
            float p_lo = wl * acc_lo, p_hi = wl * acc_hi;
            p_lo += __shfl_xor_sync(0xFFFFFFFFu, p_lo, 1);
            p_hi += __shfl_xor_sync(0xFFFFFFFFu, p_hi, 1);
            if constexpr (M1) {
                p_lo += __shfl_xor_sync(0xFFFFFFFFu, p_lo, 2);
                p_hi += __shfl_xor_sync(0xFFFFFFFFu, p_hi, 2);
                if (tig == 0) {
                    float* yp = myy + lt * 16 + g;
                    yp[0] += p_lo;
                    yp[8] += p_hi;
                }
            } else if ((tig & 1) == 0 && am < M) {
                float* yp = myy + (size_t)am * TPC * 16 + lt * 16 + g;
                yp[0] += p_lo + accb_lo;
                yp[8] += p_hi + accb_hi;
            }
        }
        __syncwarp();
        issue(it_lt, it_st, b);
        cp_async_commit();     // always one group per iteration so that the group count stays uniform
        advance(it_lt, it_st);
        advance(lt, st);
        if (++b == nbuf) b = 0;
    }
    cp_async_wait<0>();
    __syncthreads();
    for (int i = tid; i < M * ntile * 16; i += THREADS) {
        const int m = i / (ntile * 16), r = i - m * (ntile * 16);
        float v = 0.f;
#pragma unroll 4
        for (int w = 0; w < NW; ++w) v += ysum[((size_t)w * M + m) * TPC * 16 + r];
        const TileInfo& ti = tiles[r >> 4];
        if ((r & 15) < ti.rows_valid) ti.y[(int64_t)m * ti.ldy + (r & 15)] = A::from_f32(v);
    }
}

template <typename AT, int BITS, int GS, int NW, bool M1>
static int launch_cfg_m(GemvArgs a, GemvBatch bt, int nbuf, int tpc, int grid, cudaStream_t st, bool* launched) {
    using Geo = Geom<BITS, GS>;
    *launched = false;
    a.nbuf = nbuf;
    a.ksplit = tpc;
    const size_t smem = (size_t)head_bytes((int)a.K, a.G, a.M, tpc, NW) + (size_t)NW * nbuf * Geo::STAGE;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_pint_kernel<AT, BITS, GS, NW, M1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        MAX_SMEM));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
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
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemv_pint_kernel<AT, BITS, GS, NW, M1>, a, bt));
    *launched = true;
    return JQ_OK;
}

template <typename AT, int BITS, int GS, int NW>
static int launch_cfg(const GemvArgs& a, const GemvBatch& bt, int nbuf, int tpc, int grid, cudaStream_t st, bool* launched) {
    if (a.M == 1) return launch_cfg_m<AT, BITS, GS, NW, true>(a, bt, nbuf, tpc, grid, st, launched);
    return launch_cfg_m<AT, BITS, GS, NW, false>(a, bt, nbuf, tpc, grid, st, launched);
}

// One CTA per SM; every CTA gets the same number of 16-row tiles (the last one the remainder).  The warp
// count and the ring depth are the largest that fit the shared memory next to the limbs.
template <typename AT, int BITS, int GS>
static int launch_shape(const GemvArgs& a, GemvBatch bt, cudaStream_t st, bool* launched) {
    using Geo = Geom<BITS, GS>;
    const int sms = sm_count();
    int64_t tiles = 0;
    for (int i = 0; i < bt.count; ++i) {
        tiles += (bt.N[i] + 15) / 16;
        bt.blk_end[i] = (int)tiles;
    }
    const int tpc = (int)((tiles + sms - 1) / sms);
    const int grid = (int)((tiles + tpc - 1) / tpc);
    if (tpc > 64) return JQ_OK;
    // 20 warps by default; 24 when that saves a round of items (short runs: the slowest warp sets the time)
    const int64_t items = (int64_t)tpc * ((a.K + Geo::KT - 1) / Geo::KT);
    int nw = (items + 23) / 24 < (items + 19) / 20 ? 24 : 20;
    int nbuf = 3;
    while ((size_t)head_bytes((int)a.K, a.G, a.M, tpc, nw) + (size_t)nw * nbuf * Geo::STAGE > (size_t)MAX_SMEM) {
        if (nbuf > 2) --nbuf;
        else if (nw > 16) nw -= 4;
        else return JQ_OK;                 // does not fit: another kernel
    }
    if (nw == 24) return launch_cfg<AT, BITS, GS, 24>(a, bt, nbuf, tpc, grid, st, launched);
    if (nw == 20) return launch_cfg<AT, BITS, GS, 20>(a, bt, nbuf, tpc, grid, st, launched);
    return launch_cfg<AT, BITS, GS, 16>(a, bt, nbuf, tpc, grid, st, launched);
}

}  // namespace pint

// Dense mat-vecs (one launch for all matrices of `bt`) on the persistent integer warp-MMA kernel;
// *launched stays false when the shape does not fit it (widths other than 2/4/8, more than 2 activation rows).
int launch_pint_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                       bool* launched) {
    *launched = false;
    if (!(bits == 2 || bits == 4 || bits == 8) || a.M > 2 || a.K % (4 * gs) != 0) return JQ_OK;
    int rc = JQ_OK;
#define JQ_PINT_CASE(B, GSZ)                                                                          \
    if (bits == B && gs == GSZ) {                                                                     \
        rc = (act_dtype == JQ_BF16) ? pint::launch_shape<__nv_bfloat16, B, GSZ>(a, bt, st, launched)  \
                                    : pint::launch_shape<__half, B, GSZ>(a, bt, st, launched);        \
    }
    JQ_PINT_CASE(2, 64) JQ_PINT_CASE(4, 64) JQ_PINT_CASE(8, 64) JQ_PINT_CASE(2, 128) JQ_PINT_CASE(4, 128) JQ_PINT_CASE(8, 128)
#undef JQ_PINT_CASE
    return rc;
}

}  // namespace jq
