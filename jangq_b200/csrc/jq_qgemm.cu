// K3: prefill-shaped quantized GEMM  Y[M,N] = X[M,K] . deq(W)[N,K]^T  on the 5th-generation
// tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// Bound: dense bf16/f16 tensor throughput for large M; 2*M*N*K flops per launch.
//
// One CTA computes a 128 (M) x BN (N) tile of Y.  Warp roles:
//   warp 0        TMA producer: one elected lane copies the 128 x 64 activation tile of every
//                 k-block into a 128-byte-swizzled shared-memory stage (cp.async.bulk.tensor);
//   warp 1        allocates BN columns of tensor memory; one elected lane issues the MMAs
//                 (4 x tcgen05.mma M=128, N=BN, K=16 per k-block) and commits their completion to
//                 the mbarriers that free the stages;
//   warps 2..     dequantizers, one weight row per thread: packed codes -> registers -> exact
//                 q (16-bit float) -> fma(q, scale, bias) rounded once to the activation type ->
//                 the K-major, 128-byte-swizzled B tile in shared memory (the layout TMA would
//                 have produced), then fence.proxy.async + mbarrier arrive; afterwards the same
//                 warps run the epilogue: tcgen05.ld the accumulator, convert, store Y.
// Every mbarrier wait is bounded; a wait that runs out sets the library's status word and the
// CTA leaves through the common exit (tensor memory is always released).
//
// Numerics: the B operand is the dequantized weight rounded to the activation type (what
// MLX's qmm feeds its matrix units), products are accumulated in f32.
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "jq_mma.cuh"
#include "jq_tc.cuh"

namespace jq {


constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_SMEM = 227 * 1024;   // dynamic shared memory of one CTA
constexpr int GEMM_SB = 2;     // dequantized-weight stages

struct GemmArgs {
    const uint32_t* codes;
    const void* scales;
    const void* biases;
    void* y;
    int64_t M, N, K, ldy;
    int gs, G;
    int y_vec_ok;    // rows of y are 16-byte aligned
    int* status;     // device status word, set to 1 when a bounded wait ran out
    // grouped mode (routed experts): blockIdx.y indexes a tile list built by jq_moe_sort; rows are the
    // expert-sorted (token, slot) pairs, weights come from per-expert pointer tables
    const int32_t* tile_expert;
    const int32_t* tile_row0;
    const int32_t* num_tiles;
    const int32_t* expert_offsets;
    const uint32_t* const* codes_tab;
    const void* const* scales_tab;
    const void* const* biases_tab;
    const int32_t* bits_tab;       // optional per-expert bit width: tiles of other widths exit
};

template <typename AT> __host__ __device__ constexpr uint32_t umma_fmt();
template <> __host__ __device__ constexpr uint32_t umma_fmt<__nv_bfloat16>() { return 1u; }
template <> __host__ __device__ constexpr uint32_t umma_fmt<__half>() { return 0u; }

template <typename AT, int BN>
__host__ __device__ constexpr uint32_t umma_idesc() {
    return (1u << 4) /* D = f32 */ | (umma_fmt<AT>() << 7) | (umma_fmt<AT>() << 10) | ((uint32_t)(BN >> 3) << 17) |
           ((uint32_t)(GEMM_BM >> 4) << 24);             // A and B both K-major, no negate, dense
}

// ---- packed 16-bit float helpers --------------------------------------------------------------------
template <typename AT> struct P2;
template <> struct P2<__nv_bfloat16> {
    __device__ static __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        uint32_t r;
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
        return r;
    }
};
template <> struct P2<__half> {
    __device__ static __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        uint32_t r;
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
        return r;
    }
};

// 32 bits of a row's code stream starting at bit A (negative A: zero-filled below bit 0)
template <int NWORDS, int A>
__device__ __forceinline__ uint32_t stream_at(const uint32_t (&u)[NWORDS]) {
    if constexpr (A < 0) return u[0] << (-A);
    else if constexpr (A % 32 == 0) return u[A / 32];
    else if constexpr (A / 32 + 1 < NWORDS) return __funnelshift_r(u[A / 32], u[A / 32 + 1], A % 32);
    else return u[A / 32] >> (A % 32);
}

// Weights J and J+1 of a 64-code unit: rn(q*s + bias) in the activation type, packed.
// sp2 = (s', s') with s' = s * 2^-TGT, b2 = (bias, bias); s/bias are the same values in f32.
template <typename AT, int BITS, int J>
__device__ __forceinline__ uint32_t dequant_pair(const uint32_t (&u)[2 * BITS], uint32_t sp2, uint32_t b2, float s,
                                                 float bias) {
    if constexpr (BITS <= Act<AT>::MANT) {
        constexpr int TGT = Act<AT>::MANT - BITS;
        constexpr uint32_t MASK = (((1u << BITS) - 1u) << TGT) * 0x00010001u;
        const uint32_t lo = stream_at<2 * BITS, J * BITS - TGT>(u);
        const uint32_t hi = stream_at<2 * BITS, (J + 1) * BITS - TGT>(u);
        const uint32_t v = and_or(prmt(lo, hi, 0x5410), MASK, Act<AT>::MAGIC);   // 2^MANT + q*2^TGT, twice
        const uint32_t q2 = P2<AT>::sub(v, Act<AT>::MAGIC);                       // q * 2^TGT, exact
        return P2<AT>::fma(q2, sp2, b2);                                          // one rounding
    } else {
        // codes wider than the mantissa (8-bit with bf16): exact q in f32 through the 2^23 trick
        static_assert(BITS == 8, "only 8-bit codes take the f32 route");
        const uint32_t word = u[J / 4];
        const float q0 = __uint_as_float(prmt(word, 0x4B000000u, 0x7540u | (uint32_t)(J % 4))) - 8388608.0f;
        const float q1 = __uint_as_float(prmt(word, 0x4B000000u, 0x7540u | (uint32_t)(J % 4 + 1))) - 8388608.0f;
        return Act<AT>::pack_hi(fmaf(q0, s, bias), fmaf(q1, s, bias));
    }
}

// codes 8C .. 8C+7 -> one 16-byte chunk of the B tile
template <typename AT, int BITS, int C>
__device__ __forceinline__ uint4 dequant_chunk(const uint32_t (&u)[2 * BITS], uint32_t sp2, uint32_t b2, float s,
                                               float bias) {
    return make_uint4(dequant_pair<AT, BITS, 8 * C + 0>(u, sp2, b2, s, bias),
                      dequant_pair<AT, BITS, 8 * C + 2>(u, sp2, b2, s, bias),
                      dequant_pair<AT, BITS, 8 * C + 4>(u, sp2, b2, s, bias),
                      dequant_pair<AT, BITS, 8 * C + 6>(u, sp2, b2, s, bias));
}

// Code staging of one CTA: k-blocks per stage, bytes per row and stage, row pitch.  With two row tiles per CTA
// the activation stages take twice the room, so the code stages shrink: rows of 128 bytes lose their padding
// (their 16-byte chunks are XOR-swizzled by the row instead) and the wide odd widths stage fewer k-blocks.
// Rows of 128 bytes are not padded there: their 16-byte chunks are XOR-swizzled by the row instead, so that the
// eight rows a quarter-warp reads together fall into eight different 16-byte bank groups.
// Measured on 4096x14336x4096 (B200, 4-bit): three activation stages with these code stages run at 961 TFLOP/s;
// halving the code stages to make room for a fourth activation stage runs at 830 -- the pace is set by the
// dequantizer warps and their per-stage synchronisation, not by the depth of the TMA pipeline; two threads per
// weight row (twice the dequantizer warps) run at 840.
template <int BITS, int BN, int MT> struct CodeStage {
    static constexpr int CKB = MT == 1 ? (BITS == 2 ? 8 : (BITS == 8 ? 2 : 4))
                                       : (BITS == 2 ? 8 : (BITS == 3 || BITS == 4) ? 4 : 2);
    static constexpr int RB = CKB * 8 * BITS;
    static constexpr bool SWZ = MT == 2 && RB == 128;
    static constexpr int RBP = SWZ ? RB : RB + 16;
    static constexpr int SA = 3;                                    // activation stages
    static constexpr size_t SMEM = 1024 + 256 + (size_t)SA * MT * GEMM_BM * GEMM_BK * 2 + GEMM_SB * BN * GEMM_BK * 2 +
                                   2 * BN * RBP;
};

__device__ __forceinline__ void gemm_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f32x4(const float* own, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(own)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
constexpr int KS_PITCH = 256 + 4;     // floats per staged accumulator row: 16 bytes of skew keep 16-byte accesses apart

// MT: 128-row tiles of the activations per CTA (1 or 2).  With 2 every dequantized weight tile feeds two
// accumulators (2 x BN columns of tensor memory), which halves the dequantizer work per flop: the kernel is
// bound by the dequantizer warps, not by the tensor pipe, with one.
// KS: CTAs of a cluster (along blockIdx.z) that split K, for grids that would leave most SMs idle: every CTA
// accumulates its share of the k-blocks in its own tensor memory; the others stage their accumulators as float32
// in their (by then idle) shared memory, and CTA 0 of the cluster adds them through distributed shared memory
// in rank order and stores the tile.  Both cluster barriers are reached by every thread on every path.
template <typename AT, int BITS, int BN, int DPR, int MT, int KS = 1>
__global__ void __launch_bounds__(64 + BN * DPR)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const GemmArgs a) {
    using A = Act<AT>;
    using CS = CodeStage<BITS, BN, MT>;
    constexpr int GEMM_SA = CS::SA;
    constexpr int NDW = BN / 32 * DPR;                  // dequantizer warps (DPR threads share a weight row)
    constexpr int NDT = NDW * 32;
    constexpr int A_TILE = GEMM_BM * GEMM_BK * 2;       // 16 KB
    constexpr int A_STAGE = MT * A_TILE;
    constexpr int B_STAGE = BN * GEMM_BK * 2;
    constexpr int UW = 2 * BITS;                        // words of one row's 64 codes
    // packed codes are staged through shared memory, CKB k-blocks at a time, so that the global
    // reads are coalesced 16-byte chunks (8+ lanes per row) instead of one sector per thread
    constexpr int CKB = CS::CKB;
    constexpr int RB = CS::RB;                          // bytes per row and code stage (80..192)
    constexpr int RBP = CS::RBP;                        // padded pitch (or swizzled chunks): conflict-free row reads
    constexpr bool SWZ = CS::SWZ;
    constexpr int CPR = RB / 16;                        // 16-byte chunks per row
    constexpr int C_STAGE = BN * RBP;
    static_assert(MT * BN <= 512, "tensor memory holds 512 columns");
    // swizzle of a staged 128-byte code row (8 chunks): by the row
    auto swz_of = [](int row) { return row & 7; };

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the dynamic shared-memory base is only guaranteed 16-byte aligned: realign to 1024
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + GEMM_SA * A_STAGE;
    uint8_t* sC = sB + GEMM_SB * B_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sC + 2 * C_STAGE);
    uint64_t* xfull = bars;                  // [SA]
    uint64_t* xempty = bars + GEMM_SA;       // [SA]
    uint64_t* bfull = bars + 2 * GEMM_SA;    // [SB]
    uint64_t* bempty = bfull + GEMM_SB;      // [SB]
    uint64_t* accfull = bempty + GEMM_SB;    // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n0 = (int64_t)blockIdx.x * BN;
    int64_t m0 = (int64_t)blockIdx.y * (GEMM_BM * MT), m_end = a.M;
    const uint32_t* codes_g = a.codes;
    const void* scales_g = a.scales;
    const void* biases_g = a.biases;
    if (a.tile_expert) {
        // uniform for the whole CTA, before any barrier or tensor-memory allocation
        if ((int)blockIdx.y >= *a.num_tiles) return;
        const int e = a.tile_expert[blockIdx.y];
        if (a.bits_tab && a.bits_tab[e] != BITS) return;
        m0 = a.tile_row0[blockIdx.y];
        m_end = a.expert_offsets[e + 1];
        codes_g = a.codes_tab[e];
        scales_g = a.scales_tab[e];
        biases_g = a.biases_tab[e];
    }
    // this CTA's k-blocks [kb0, kb1): all of them, or its share (whole code stages) of a split K
    const int nkb_all = (int)(a.K / GEMM_BK);
    int kb0 = 0, kb1 = nkb_all;
    const int ks_rank = KS > 1 ? (int)blockIdx.z : 0;
    if constexpr (KS > 1) {
        kb0 = (ks_rank * nkb_all / KS) / CKB * CKB;
        kb1 = ks_rank == KS - 1 ? nkb_all : ((ks_rank + 1) * nkb_all / KS) / CKB * CKB;
    }
    const int nkb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < GEMM_SA; ++i) { mbar_init(xfull + i, 1); mbar_init(xempty + i, 1); }
        for (int i = 0; i < GEMM_SB; ++i) { mbar_init(bfull + i, NDW); mbar_init(bempty + i, 1); }
        mbar_init(accfull, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, MT * BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (int lk = 0; lk < nkb && ok; ++lk) {
                const int s = lk % GEMM_SA;
                if (lk >= GEMM_SA) ok = mbar_wait(xempty + s, (uint32_t)((lk / GEMM_SA) - 1) & 1u, 1u << 18);
                if (!ok) break;
                mbar_expect_tx(xfull + s, A_STAGE);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)      // rows past M read as zeros
                    tma_load_2d(sA + s * A_STAGE + mt * A_TILE, &xmap, (kb0 + lk) * GEMM_BK, (int)m0 + mt * GEMM_BM,
                                xfull + s);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc<AT, BN>();
            for (int kb = 0; kb < nkb && ok; ++kb) {      // kb: local index
                const int s = kb % GEMM_SA, t = kb % GEMM_SB;
                ok = mbar_wait(xfull + s, (uint32_t)(kb / GEMM_SA) & 1u, 1u << 18) &&
                     mbar_wait(bfull + t, (uint32_t)(kb / GEMM_SB) & 1u, 1u << 18);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(sA + s * A_STAGE), b_addr = smem_u32(sB + t * B_STAGE);
#pragma unroll
                for (int k = 0; k < GEMM_BK / 16; ++k)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        umma_f16(tmem_base + (uint32_t)(mt * BN), umma_desc_sw128(a_addr + mt * A_TILE + k * 32),
                                 umma_desc_sw128(b_addr + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(xempty + s);
                umma_commit(bempty + t);
            }
            if (ok) umma_commit(accfull);
        }
    } else {
        // ---------------- dequantizers: one weight row per thread ----------------
        const int dt = threadIdx.x - 64;                      // 0 .. NDT-1
        const int r = dt % BN;                                // row within the tile
        const int half = dt / BN;                             // DPR = 2: which 32 codes of the k-block (warp-uniform)
        const int64_t n = min(n0 + r, a.N - 1);               // rows past N are computed but never stored
        const int64_t rowbytes = a.K * BITS / 8;
        const uint8_t* cbytes = reinterpret_cast<const uint8_t*>(codes_g);
        const uint16_t* srow = reinterpret_cast<const uint16_t*>(scales_g) + n * a.G;
        const uint16_t* brow = reinterpret_cast<const uint16_t*>(biases_g) + n * a.G;
        const uint32_t row_off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
        const uint32_t sw = (uint32_t)(r & 7);
        const int gs = a.gs;
        const int st0 = kb0 / CKB, nstage = (kb1 + CKB - 1) / CKB;     // code stages [st0, nstage) (absolute)

        // all dequantizer threads copy code stage `st` together: consecutive lanes take consecutive
        // 16-byte chunks of a row; always one commit so that group counting stays uniform
        auto issue_codes = [&](int st, int buf) {
            if (st < nstage) {
                const int64_t off = (int64_t)st * RB;
                const int rem = (int)min((int64_t)RB, rowbytes - off);
                uint8_t* dstb = sC + buf * C_STAGE;
                for (int c = dt; c < BN * CPR; c += NDT) {
                    const int row = c / CPR, col = c - row * CPR;
                    if (col * 16 < rem)
                        cp_async16(dstb + row * RBP + (SWZ ? (col ^ swz_of(row)) : col) * 16,
                                   cbytes + min(n0 + row, a.N - 1) * rowbytes + off + col * 16);
                }
            }
            cp_async_commit();
        };

        // Scales and biases: one vector load per code stage (CKB consecutive groups of this row) when
        // the row is suitably aligned and groups are 64 or 128 wide; otherwise scalar loads per k-block.
        // Either way they are fetched one step ahead of their use.
        constexpr int SCW = CKB / 2;                          // 32-bit words holding CKB 16-bit sidecars
        const int gpk_shift = (gs == 128) ? 1 : 0;            // k-blocks per group: 1 (gs 64) or 2 (gs 128)
        const bool sc_vec = (gs >= 64) && (a.G % (CKB >> gpk_shift) == 0) &&
                            ((reinterpret_cast<uintptr_t>(srow) | reinterpret_cast<uintptr_t>(brow)) % (2 * CKB) == 0) &&
                            ((a.G * 2) % (2 * CKB) == 0);
        uint32_t scw[SCW], bcw[SCW], scn[SCW], bcn[SCW];
#pragma unroll
        for (int i = 0; i < SCW; ++i) scw[i] = bcw[i] = scn[i] = bcn[i] = 0u;
        auto load_sc_stage = [&](int st, uint32_t (&so)[SCW], uint32_t (&bo)[SCW]) {
            // groups of stage st: first = st*CKB >> gpk_shift, count = CKB >> gpk_shift (a multiple of 2 words when vec)
            const int gfirst = (st * CKB) >> gpk_shift;
            const int cnt = CKB >> gpk_shift;
            if (gfirst + cnt <= a.G) {
                const uint32_t* sp = reinterpret_cast<const uint32_t*>(srow + gfirst);
                const uint32_t* bp = reinterpret_cast<const uint32_t*>(brow + gfirst);
                if (cnt == 8) {
                    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sp)), bv = __ldg(reinterpret_cast<const uint4*>(bp));
                    so[0] = sv.x; if (SCW > 1) so[1 % SCW] = sv.y; if (SCW > 2) { so[2 % SCW] = sv.z; so[3 % SCW] = sv.w; }
                    bo[0] = bv.x; if (SCW > 1) bo[1 % SCW] = bv.y; if (SCW > 2) { bo[2 % SCW] = bv.z; bo[3 % SCW] = bv.w; }
                } else if (cnt == 4) {
                    const uint2 sv = __ldg(reinterpret_cast<const uint2*>(sp)), bv = __ldg(reinterpret_cast<const uint2*>(bp));
                    so[0] = sv.x; if (SCW > 1) so[1 % SCW] = sv.y;
                    bo[0] = bv.x; if (SCW > 1) bo[1 % SCW] = bv.y;
                } else if (cnt == 2) {
                    so[0] = __ldg(sp); bo[0] = __ldg(bp);
                } else {                                       // cnt == 1
                    so[0] = __ldg(srow + gfirst); bo[0] = __ldg(brow + gfirst);
                }
            } else {                                           // ragged last stage: element loads
#pragma unroll
                for (int i = 0; i < CKB; ++i) {
                    const int gi = gfirst + i;
                    if (i < cnt && gi < a.G) {
                        const uint32_t sv = __ldg(srow + gi), bv = __ldg(brow + gi);
                        if (i & 1) { so[i / 2] |= sv << 16; bo[i / 2] |= bv << 16; }
                        else { so[i / 2] = sv; bo[i / 2] = bv; }
                    }
                }
            }
        };
        uint16_t s0h = 0, b0h = 0, s1h = 0, b1h = 0, s0n = 0, b0n = 0, s1n = 0, b1n = 0;
        if (sc_vec) {
            load_sc_stage(st0, scw, bcw);
        } else {
            const int g0 = kb0 * GEMM_BK / gs;
            s0h = __ldg(srow + g0); b0h = __ldg(brow + g0);
            s1h = s0h; b1h = b0h;
            if (gs == 32) { s1h = __ldg(srow + g0 + 1); b1h = __ldg(brow + g0 + 1); }
        }
        issue_codes(st0, 0);
        // After a timed-out wait the warp keeps walking the loops (copies and the named barrier
        // only), so that no other dequantizer warp is left waiting at the barrier.
        for (int st = st0; st < nstage; ++st) {
            cp_async_wait<0>();
            asm volatile("bar.sync 1, %0;" ::"n"(NDT) : "memory");  // stage st landed; stage st-1 fully consumed
            issue_codes(st + 1, (st + 1 - st0) & 1);
            if (sc_vec && st + 1 < nstage) load_sc_stage(st + 1, scn, bcn);
            const uint8_t* crow = sC + ((st - st0) & 1) * C_STAGE + r * RBP;
#pragma unroll
            for (int kbi = 0; kbi < CKB; ++kbi) {
                const int kb = st * CKB + kbi;             // absolute k-block; lk: its index in this CTA's share
                if (kb >= kb1) break;
                const int lk = kb - kb0;
                const int t = lk % GEMM_SB;
                uint32_t cur[UW];
                if constexpr (DPR == 1) {
                    if constexpr ((8 * BITS) % 16 == 0) {
                        const uint4* cp = reinterpret_cast<const uint4*>(crow + (SWZ ? 0 : kbi * 8 * BITS));
#pragma unroll
                        for (int i = 0; i < UW / 4; ++i) {
                            const uint4 v = SWZ ? cp[(kbi * (UW / 4) + i) ^ swz_of(r)] : cp[i];
                            cur[4 * i] = v.x; cur[4 * i + 1] = v.y; cur[4 * i + 2] = v.z; cur[4 * i + 3] = v.w;
                        }
                    } else {
                        const uint2* cp = reinterpret_cast<const uint2*>(crow + kbi * 8 * BITS);
#pragma unroll
                        for (int i = 0; i < UW / 2; ++i) {
                            const uint2 v = cp[i];
                            cur[2 * i] = v.x; cur[2 * i + 1] = v.y;
                        }
                    }
                } else {
                    // this thread's 32 codes are BITS whole words; the other half stays zero
                    auto cword = [&](int off) {      // word at byte `off` of the staged row
                        const int phys = SWZ ? ((((off >> 4) ^ swz_of(r)) << 4) | (off & 15)) : off;
                        return *reinterpret_cast<const uint32_t*>(crow + phys);
                    };
                    const int off0 = kbi * 8 * BITS + half * BITS * 4;
#pragma unroll
                    for (int i = 0; i < UW; ++i) cur[i] = 0u;
                    if (half == 0) {
#pragma unroll
                        for (int i = 0; i < BITS; ++i) cur[i] = cword(off0 + 4 * i);
                    } else {
#pragma unroll
                        for (int i = 0; i < BITS; ++i) cur[BITS + i] = cword(off0 + 4 * i);
                    }
                }
                if (sc_vec) {
                    const int gi = kbi >> gpk_shift;                      // group within the stage (static after unrolling)
                    const uint32_t swd = scw[gi / 2], bwd = bcw[gi / 2];
                    s0h = (uint16_t)((gi & 1) ? (swd >> 16) : (swd & 0xFFFFu));
                    b0h = (uint16_t)((gi & 1) ? (bwd >> 16) : (bwd & 0xFFFFu));
                    s1h = s0h; b1h = b0h;
                } else if (kb + 1 < kb1) {        // scalar path: sidecars of the next k-block
                    const int k1 = (kb + 1) * GEMM_BK;
                    const int g0 = k1 / gs;
                    s0n = __ldg(srow + g0); b0n = __ldg(brow + g0);
                    s1n = s0n; b1n = b0n;
                    if (gs == 32) { s1n = __ldg(srow + g0 + 1); b1n = __ldg(brow + g0 + 1); }
                }
                constexpr int TGTC = (BITS <= A::MANT) ? A::MANT - BITS : 0;
                constexpr float POST = 1.0f / (float)(1 << TGTC);
                const float s0 = A::to_f32(s0h), s1 = A::to_f32(s1h), bias0 = A::to_f32(b0h), bias1 = A::to_f32(b1h);
                // s * 2^-TGT is exact (power-of-two scaling) unless it underflows the 16-bit type
                const uint32_t sp0 = A::pack_hi(s0 * POST, s0 * POST), sp1 = A::pack_hi(s1 * POST, s1 * POST);
                const uint32_t bb0 = (uint32_t)b0h * 0x00010001u, bb1 = (uint32_t)b1h * 0x00010001u;
                if (ok && lk >= GEMM_SB)   // warp-uniform outcome
                    ok = __all_sync(0xFFFFFFFFu, mbar_wait(bempty + t, (uint32_t)((lk / GEMM_SB) - 1) & 1u, 1u << 18));
                if (ok) {
                    uint8_t* dst = sB + t * B_STAGE + row_off;
#define JQ_CHUNK(C, SP, BB, S, BI) \
    *reinterpret_cast<uint4*>(dst + (((uint32_t)(C) ^ sw) << 4)) = dequant_chunk<AT, BITS, C>(cur, SP, BB, S, BI);
                    if (DPR == 1 || half == 0) {
                        JQ_CHUNK(0, sp0, bb0, s0, bias0) JQ_CHUNK(1, sp0, bb0, s0, bias0)
                        JQ_CHUNK(2, sp0, bb0, s0, bias0) JQ_CHUNK(3, sp0, bb0, s0, bias0)
                    }
                    if (DPR == 1 || half == 1) {
                        JQ_CHUNK(4, sp1, bb1, s1, bias1) JQ_CHUNK(5, sp1, bb1, s1, bias1)
                        JQ_CHUNK(6, sp1, bb1, s1, bias1) JQ_CHUNK(7, sp1, bb1, s1, bias1)
                    }
#undef JQ_CHUNK
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bfull + t);
                }
                if (!sc_vec) { s0h = s0n; b0h = b0n; s1h = s1n; b1h = b1n; }
            }
            if (sc_vec) {
#pragma unroll
                for (int i = 0; i < SCW; ++i) { scw[i] = scn[i]; bcw[i] = bcn[i]; }
            }
        }
        cp_async_wait<0>();

        // ---------------- epilogue: TMEM -> registers -> Y ----------------
        if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait(accfull, 0, 1u << 18));
        if constexpr (KS > 1) {
            // split K: the accumulator is complete, so nothing reads this CTA's stages any more; the CTAs behind
            // rank 0 leave theirs as float32 rows at the start of their shared memory (rank 0 stores after the
            // cluster barrier below)
            if (ok && ks_rank != 0) {
                tc_fence_after();
                const int q = warp & 3, part = (warp - 2) / 4;
                constexpr int COLS_PER_WARP = BN / (NDW / 4);
                float* srow_f = reinterpret_cast<float*>(smem) + (size_t)(q * 32 + lane) * KS_PITCH;
#pragma unroll 1
                for (int c0 = part * COLS_PER_WARP; c0 < (part + 1) * COLS_PER_WARP; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(srow_f + c0 + 4 * j) =
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                }
            }
        }
        if (KS == 1 && ok) {
            tc_fence_after();
            const int q = warp & 3;                               // TMEM lane quarter this warp may read
            const int part = (warp - 2) / 4;                      // the NDW/4 warps of a quarter split the columns
            constexpr int COLS_PER_WARP = BN / (NDW / 4);
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
            const int64_t m = m0 + mt * GEMM_BM + q * 32 + lane;
            uint16_t* yrow = reinterpret_cast<uint16_t*>(a.y) + m * a.ldy + n0;
#pragma unroll 1
            for (int c0 = part * COLS_PER_WARP; c0 < (part + 1) * COLS_PER_WARP; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * BN + c0), v);
                if (m < m_end) {
                    if (a.y_vec_ok && n0 + c0 + 32 <= a.N) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 o;
                            o.x = A::pack_hi(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
                            o.y = A::pack_hi(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                            o.z = A::pack_hi(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                            o.w = A::pack_hi(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                            *reinterpret_cast<uint4*>(yrow + c0 + 8 * j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c0 + j < a.N) yrow[c0 + j] = A::from_f32(__uint_as_float(v[j]));
                    }
                }
            }
            }
        }
    }
    if constexpr (KS > 1) {
        static_assert(KS == 1 || (MT == 1 && BN == 256), "split K: one 128 x 256 accumulator per CTA");
        gemm_cluster_sync();                               // the staged accumulators are complete
        if (warp >= 2 && ks_rank == 0 && ok) {
            tc_fence_after();
            const int q = warp & 3, part = (warp - 2) / 4;
            constexpr int COLS_PER_WARP = BN / (NDW / 4);
            const float* srow_f = reinterpret_cast<const float*>(smem) + (size_t)(q * 32 + lane) * KS_PITCH;
            const int64_t m = m0 + q * 32 + lane;
            uint16_t* yrow = reinterpret_cast<uint16_t*>(a.y) + m * a.ldy + n0;
#pragma unroll 1
            for (int c0 = part * COLS_PER_WARP; c0 < (part + 1) * COLS_PER_WARP; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                for (int rk = 1; rk < KS; ++rk) {           // rank order: the same sum whatever the timing
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 t = ld_cluster_f32x4(srow_f + c0 + 4 * j, (uint32_t)rk);
                        f[4 * j] += t.x; f[4 * j + 1] += t.y; f[4 * j + 2] += t.z; f[4 * j + 3] += t.w;
                    }
                }
                if (m < m_end) {
                    if (a.y_vec_ok && n0 + c0 + 32 <= a.N) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 o;
                            o.x = A::pack_hi(f[8 * j + 0], f[8 * j + 1]);
                            o.y = A::pack_hi(f[8 * j + 2], f[8 * j + 3]);
                            o.z = A::pack_hi(f[8 * j + 4], f[8 * j + 5]);
                            o.w = A::pack_hi(f[8 * j + 6], f[8 * j + 7]);
                            *reinterpret_cast<uint4*>(yrow + c0 + 8 * j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c0 + j < a.N) yrow[c0 + j] = A::from_f32(f[j]);
                    }
                }
            }
        }
        gemm_cluster_sync();                               // the others keep their shared memory until rank 0 has read it
    }
    if (!ok) atomicOr(a.status, JQ_STATUS_LOCAL_WAIT);
    tc_fence_before();
    const int gave_up = __syncthreads_or(ok ? 0 : 1);
    if (warp == 1) {
        // after a wait that gave up, copies and MMAs of this CTA may still be in flight: give them a millisecond
        // to land before the tensor memory goes back and the CTA's shared memory is reused
        if (gave_up)
            for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        tc_fence_after();
        tmem_dealloc(tmem_base, MT * BN);
    }
}

// ---- host side ------------------------------------------------------------------------------------------
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// m_tiles: 128-row tiles of a dense GEMM (MT of them per CTA), or entries of a grouped GEMM's tile list (one CTA
// each, whatever MT)
template <typename AT, int BITS, int BN, int DPR, int MT = 1, int KS = 1>
static int launch_gemm(const CUtensorMap& xmap, const GemmArgs& a, int64_t m_tiles, cudaStream_t st) {
    constexpr size_t smem = CodeStage<BITS, BN, MT>::SMEM;
    static_assert(smem <= GEMM_SMEM, "shared memory of one CTA");
    static_assert(KS == 1 || 1024 + 128 * KS_PITCH * sizeof(float) <= smem - 512, "staged accumulator fits the stages");
    static bool attr_done[64] = {};
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemm_tc_kernel<AT, BITS, BN, DPR, MT, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    dim3 grid((unsigned)((a.N + BN - 1) / BN), (unsigned)(a.tile_expert ? m_tiles : (m_tiles + MT - 1) / MT), KS);
    if constexpr (KS > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(64 + BN * DPR);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = KS;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemm_tc_kernel<AT, BITS, BN, DPR, MT, KS>, xmap, a));
        return JQ_OK;
    }
    qgemm_tc_kernel<AT, BITS, BN, DPR, MT, KS><<<grid, 64 + BN * DPR, smem, st>>>(xmap, a);
    return check_launch("qgemm");
}

struct GroupedArgs {
    const int32_t *tile_expert, *tile_row0, *num_tiles, *expert_offsets, *bits_tab;
    const uint32_t* const* codes_tab;
    const void* const* scales_tab;
    const void* const* biases_tab;
    int64_t max_tiles;
    int tile_m;       // rows per entry of the tile list: 128, or 256 (two accumulators per CTA)
};

// Dense when grp == nullptr (codes/scales/biases of one matrix); grouped otherwise (x holds the M
// expert-sorted rows, the weight pointers come from the tables).
int qgemm_dispatch(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
                   const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int gs, void* y,
                   int y_dtype, int64_t ldy, const GroupedArgs* grp, cudaStream_t st) {
    int rc = check_quant_shape(N, K, bits, gs);
    if (rc != JQ_OK) return rc;
    JQ_REQUIRE(M >= 0, JQ_EINVAL, "negative M");
    if (M == 0 || N == 0) return JQ_OK;
    JQ_REQUIRE(K > 0, JQ_EINVAL, "K must be positive");
    JQ_REQUIRE(x && y && (grp || (codes && scales && biases)), JQ_EINVAL, "null pointer");
    JQ_REQUIRE(x_dtype == JQ_BF16 || x_dtype == JQ_F16, JQ_EINVAL, "qgemm activations must be bf16 or f16");
    JQ_REQUIRE(sidecar_dtype == x_dtype && y_dtype == x_dtype, JQ_EUNSUPPORTED,
               "qgemm needs scales/biases and the output in the activation dtype");
    JQ_REQUIRE(K % GEMM_BK == 0, JQ_EUNSUPPORTED, "qgemm needs K to be a multiple of 64, got %lld", (long long)K);
    JQ_REQUIRE((K * bits / 8) % 16 == 0, JQ_EUNSUPPORTED,
               "qgemm needs packed rows of a multiple of 16 bytes (K %% 128 == 0 for odd widths), got K=%lld bits=%d",
               (long long)K, bits);
    JQ_REQUIRE(grp || aligned(codes, 16), JQ_EINVAL, "codes must be 16-byte aligned");
    JQ_REQUIRE(aligned(x, 16) && ldx % 8 == 0 && ldx >= K, JQ_EINVAL, "x must be 16-byte aligned with ldx %% 8 == 0");
    JQ_REQUIRE(ldy >= N, JQ_EINVAL, "ldy too small");
    JQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), JQ_EUNSUPPORTED, "dimension too large");
    EncodeTiledFn enc = encode_tiled_fn();
    JQ_REQUIRE(enc != nullptr, JQ_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");

    CUtensorMap xmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {GEMM_BK, GEMM_BM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&xmap, x_dtype == JQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                      const_cast<void*>(x), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    JQ_REQUIRE(cr == CUDA_SUCCESS, JQ_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)cr);

    GemmArgs a;
    a.codes = codes; a.scales = scales; a.biases = biases; a.y = y;
    a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.gs = gs; a.G = (int)(K / gs);
    a.y_vec_ok = (aligned(y, 16) && ldy % 8 == 0) ? 1 : 0;
    a.status = status_word();
    JQ_REQUIRE(a.status != nullptr, JQ_ECUDA, "could not locate the device status word");
    a.tile_expert = grp ? grp->tile_expert : nullptr;
    a.tile_row0 = grp ? grp->tile_row0 : nullptr;
    a.num_tiles = grp ? grp->num_tiles : nullptr;
    a.expert_offsets = grp ? grp->expert_offsets : nullptr;
    a.codes_tab = grp ? grp->codes_tab : nullptr;
    a.scales_tab = grp ? grp->scales_tab : nullptr;
    a.biases_tab = grp ? grp->biases_tab : nullptr;
    a.bits_tab = grp ? grp->bits_tab : nullptr;
    const int64_t m_tiles = grp ? grp->max_tiles : (M + GEMM_BM - 1) / GEMM_BM;
    if (m_tiles == 0) return JQ_OK;
    JQ_REQUIRE(m_tiles < 65536, JQ_EUNSUPPORTED, "too many row tiles for one launch (%lld)", (long long)m_tiles);
    // 256-wide tiles reuse every activation tile twice as often; narrow outputs keep 128.  Two row tiles per CTA
    // (dense only: the grouped tile lists are per 128 rows) when that still leaves a CTA for most SMs.
    const bool wide = N >= 256;
    JQ_REQUIRE(!grp || grp->tile_m == 128 || (grp->tile_m == 256 && wide && x_dtype == JQ_BF16), JQ_EUNSUPPORTED,
               "tile lists of 256 rows need bf16 activations and N >= 256 (128 otherwise)");
    // Dense GEMMs pick the form with the shortest estimated time.  A CTA walks a k-block in about 1.1 us with one
    // accumulator and 1.3 us with two (measured; the dequantizer warps set the pace), whatever the grid, so what
    // counts is the number of waves and the k-blocks per CTA:
    //   one accumulator            waves(tiles)      * nkb * 1.1
    //   two accumulators (MT = 2)  waves(tiles / 2)  * nkb * 1.3     (every weight tile dequantized once for two)
    //   split K over S CTAs        waves(tiles * S)  * (nkb / S * 1.1 + 8)   (8 us: staging and adding the accumulators)
    bool two = grp ? grp->tile_m == 256 : false;
    int ksplit = 1;
    if (!grp && wide && x_dtype == JQ_BF16) {
        const int64_t sms = sm_count(), ncol = (N + 255) / 256, nkb_all = K / GEMM_BK;
        auto waves = [&](int64_t ctas) { return (double)((ctas + sms - 1) / sms); };
        double best = waves(ncol * m_tiles) * nkb_all * 1.1;
        if (m_tiles >= 2) {
            const double t2 = waves(ncol * ((m_tiles + 1) / 2)) * nkb_all * 1.3;
            if (t2 < best) { best = t2; two = true; }
        }
        for (int S : {2, 4}) {      // clusters of 8 such CTAs were measured at half the speed of 4 (72.9 vs 33.9 us)
            if (nkb_all / S < 16) continue;
            const double ts = waves(ncol * m_tiles * S) * ((double)nkb_all / S * 1.1 + 8.0);
            if (ts < best) { best = ts; two = false; ksplit = S; }
        }
    }
#define JQ_GEMM_CASE(B)                                                                                  \
    if (bits == B) {                                                                                     \
        if (x_dtype == JQ_BF16) {                                                                        \
            if (two) return launch_gemm<__nv_bfloat16, B, 256, 1, 2>(xmap, a, m_tiles, st);              \
            if (ksplit == 4) return launch_gemm<__nv_bfloat16, B, 256, 1, 1, 4>(xmap, a, m_tiles, st);  \
            if (ksplit == 2) return launch_gemm<__nv_bfloat16, B, 256, 1, 1, 2>(xmap, a, m_tiles, st);  \
            return wide ? launch_gemm<__nv_bfloat16, B, 256, 1>(xmap, a, m_tiles, st)                    \
                        : launch_gemm<__nv_bfloat16, B, 128, 1>(xmap, a, m_tiles, st);                   \
        }                                                                                                \
        return launch_gemm<__half, B, 128, 1>(xmap, a, m_tiles, st);                                     \
    }
    JQ_GEMM_CASE(2) JQ_GEMM_CASE(3) JQ_GEMM_CASE(4) JQ_GEMM_CASE(5) JQ_GEMM_CASE(6) JQ_GEMM_CASE(8)
#undef JQ_GEMM_CASE
    return fail(JQ_EUNSUPPORTED, "bits=%d", bits);
}

// ---- allocation-free grouped GEMM ------------------------------------------------------------------
// The grouped GEMM walks a tile list (expert id and first row of every 128-row tile, plus their
// count).  jq_moe_gemm gets that list from buffers the caller allocated for jq_moe_sort; the variant
// below rebuilds it from expert_offsets into this fixed array instead, so the call needs no
// workspace at all.  Every device that loads the library holds the array (about 12 KB) until exit.
constexpr int STATIC_MAX_EXPERTS = 1024;
constexpr int64_t STATIC_MAX_ROWS = 65536;
constexpr int STATIC_MAX_TILES = (int)(STATIC_MAX_ROWS / GEMM_BM) + STATIC_MAX_EXPERTS;
constexpr int STATIC_HDR = 64;     // word 0 = number of tiles; the lists start 256 bytes in
static __device__ __align__(256) int32_t g_static_tiles[STATIC_HDR + 2 * STATIC_MAX_TILES];

// One CTA of STATIC_MAX_EXPERTS threads rewrites the whole list on every call, so nothing of an earlier
// call survives into this one: thread e counts the tiles of expert e, a block-wide exclusive scan gives
// the position of its first tile, and it writes its own tiles (experts ascending, rows ascending: the
// order jq_moe_sort emits).  Tiles past STATIC_MAX_TILES are dropped (offsets beyond the stated rows).
__global__ void __launch_bounds__(STATIC_MAX_EXPERTS)
build_tiles_kernel(const int32_t* __restrict__ offsets, int E, int tile_m, int32_t* __restrict__ out) {
    __shared__ int warp_sum[32];
    int32_t* tile_expert = out + STATIC_HDR;
    int32_t* tile_row0 = out + STATIC_HDR + STATIC_MAX_TILES;
    const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
    int lo = 0, hi = 0;
    if (e < E) { lo = offsets[e]; hi = offsets[e + 1]; }
    const int mine = hi > lo ? (hi - lo + tile_m - 1) / tile_m : 0;
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sum[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xFFFFFFFFu, w, d);
            if (lane >= d) w += v;
        }
        warp_sum[lane] = w;            // inclusive sums of the warps
    }
    __syncthreads();
    int pos = incl - mine + (warp > 0 ? warp_sum[warp - 1] : 0);
    for (int r = lo; r < hi && pos < STATIC_MAX_TILES; r += tile_m, ++pos) {
        tile_expert[pos] = e;
        tile_row0[pos] = r;
    }
    if (e == 0) out[0] = min(warp_sum[31], STATIC_MAX_TILES);
}

// Device address of the array on the current device.  In host code the array's name is only a
// host-side handle, never a device address, so it is resolved with cudaGetSymbolAddress once per
// device (with that device current) and the pointer is what the kernels receive.
static int static_tiles_ptr(int32_t** out) {
    static std::atomic<int32_t*> cached[64];      // zero-initialised; host threads may race on the first call
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    JQ_REQUIRE(dev >= 0 && dev < 64, JQ_EUNSUPPORTED, "device ordinal %d out of range", dev);
    int32_t* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        JQ_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_static_tiles));
        JQ_REQUIRE(p != nullptr, JQ_ECUDA, "cudaGetSymbolAddress returned a null address");
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return JQ_OK;
}

}  // namespace jq

extern "C" {

int jq_moe_gemm_static(const void* x_sorted, int act_dtype, int64_t max_rows, int64_t ldx,
                       const int32_t* expert_offsets, int num_experts, const uint32_t* const* codes_tab,
                       const void* const* scales_tab, const void* const* biases_tab, const int32_t* bits_tab,
                       int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y_sorted, int64_t ldy,
                       jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(expert_offsets && codes_tab && scales_tab && biases_tab, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(num_experts > 0 && num_experts <= STATIC_MAX_EXPERTS, JQ_EUNSUPPORTED,
               "jq_moe_gemm_static holds tile lists for at most %d experts, got %d", STATIC_MAX_EXPERTS, num_experts);
    JQ_REQUIRE(max_rows >= 0 && max_rows <= STATIC_MAX_ROWS, JQ_EUNSUPPORTED,
               "jq_moe_gemm_static holds tile lists for at most %lld rows, got %lld", (long long)STATIC_MAX_ROWS,
               (long long)max_rows);
    if (max_rows == 0 || N == 0) return JQ_OK;
    int32_t* tiles = nullptr;
    int rc = static_tiles_ptr(&tiles);
    if (rc != JQ_OK) return rc;
    build_tiles_kernel<<<1, STATIC_MAX_EXPERTS, 0, (cudaStream_t)stream>>>(expert_offsets, num_experts, GEMM_BM, tiles);
    rc = check_launch("build_tiles");
    if (rc != JQ_OK) return rc;
    GroupedArgs g;
    g.tile_expert = tiles + STATIC_HDR;
    g.tile_row0 = tiles + STATIC_HDR + STATIC_MAX_TILES;
    g.num_tiles = tiles;
    g.expert_offsets = expert_offsets;
    g.bits_tab = bits_tab; g.codes_tab = codes_tab; g.scales_tab = scales_tab; g.biases_tab = biases_tab;
    g.max_tiles = max_rows / GEMM_BM + num_experts;
    g.tile_m = 128;
    return qgemm_dispatch(x_sorted, act_dtype, max_rows, ldx, nullptr, nullptr, nullptr, sidecar_dtype, N, K, bits,
                          group_size, y_sorted, act_dtype, ldy, &g, (cudaStream_t)stream);
}

int jq_qgemm(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes, const void* scales,
             const void* biases, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y,
             int y_dtype, int64_t ldy, jq_stream_t stream) {
    return jq::qgemm_dispatch(x, x_dtype, M, ldx, codes, scales, biases, sidecar_dtype, N, K, bits, group_size, y,
                              y_dtype, ldy, nullptr, (cudaStream_t)stream);
}

int jq_moe_gemm(const void* x_sorted, int act_dtype, int64_t max_rows, int64_t ldx, const int32_t* expert_offsets,
                const int32_t* tile_expert, const int32_t* tile_row0, const int32_t* num_tiles, int64_t max_tiles,
                const uint32_t* const* codes_tab, const void* const* scales_tab, const void* const* biases_tab,
                const int32_t* bits_tab, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size,
                void* y_sorted, int64_t ldy, jq_stream_t stream) {
    return jq_moe_gemm_tiled(x_sorted, act_dtype, max_rows, ldx, expert_offsets, tile_expert, tile_row0, num_tiles,
                             max_tiles, 128, codes_tab, scales_tab, biases_tab, bits_tab, sidecar_dtype, N, K, bits,
                             group_size, y_sorted, ldy, stream);
}

int jq_moe_gemm_tiled(const void* x_sorted, int act_dtype, int64_t max_rows, int64_t ldx, const int32_t* expert_offsets,
                      const int32_t* tile_expert, const int32_t* tile_row0, const int32_t* num_tiles, int64_t max_tiles,
                      int tile_m, const uint32_t* const* codes_tab, const void* const* scales_tab,
                      const void* const* biases_tab, const int32_t* bits_tab, int sidecar_dtype, int64_t N, int64_t K,
                      int bits, int group_size, void* y_sorted, int64_t ldy, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(tile_m == 128 || tile_m == 256, JQ_EINVAL, "tile_m must be 128 or 256");
    JQ_REQUIRE(expert_offsets && tile_expert && tile_row0 && num_tiles && codes_tab && scales_tab && biases_tab,
               JQ_EINVAL, "null pointer");
    JQ_REQUIRE(max_tiles >= 0, JQ_EINVAL, "negative max_tiles");
    GroupedArgs g;
    g.tile_expert = tile_expert; g.tile_row0 = tile_row0; g.num_tiles = num_tiles; g.expert_offsets = expert_offsets;
    g.bits_tab = bits_tab; g.codes_tab = codes_tab; g.scales_tab = scales_tab; g.biases_tab = biases_tab;
    g.max_tiles = max_tiles;
    g.tile_m = tile_m;
    return qgemm_dispatch(x_sorted, act_dtype, max_rows, ldx, nullptr, nullptr, nullptr, sidecar_dtype, N, K, bits,
                          group_size, y_sorted, act_dtype, ldy, &g, (cudaStream_t)stream);
}

}  // extern "C"
