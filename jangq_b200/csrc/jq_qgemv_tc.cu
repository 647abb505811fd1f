// K2 on the 5th-generation tensor cores: decode-shaped quantized mat-vec
//     y[M,N] = x[M,K] . deq(W)[N,K]^T,  M <= 8,
// with the packed codes fed to tcgen05.mma as unsigned 8-bit integers and the activations as
// signed 8-bit limbs.
//
// Bound: HBM bandwidth.  Algorithmic bytes per launch =
//     N*K*bits/8 (codes) + N*(K/gs)*2*2 (scales, biases) + M*K*2 + M*N*2.
//
// Arithmetic.  Per quantization group g and activation row m the activations become fixed
// point with a shared power-of-two exponent,  x[k] ~ e(g,m) * xi[k],  |xi| <= 2^22, and xi is
// written as three signed 8-bit limbs  xi = l0 + 256*l1 + 65536*l2.  bf16/f16 values within
// 2^-14 of the group's largest magnitude are represented exactly, smaller ones are rounded
// to e(g,m) (2^-22 of the group maximum): f32-accumulation grade.  The tensor core computes the
// exact integer sums  D_l[row] = sum_k q[row,k] * l_l[k]  (|D| < 2^23, s32 accumulator), and
// per group   acc[row,m] += e * ( s * (D0 + 256*D1 + 65536*D2) + b * sum_k xi[k] ),
// which is  sum_k (s*q + b) * x[k]  up to the rounding of x described above.
//
// Structure.  One CTA owns 128 weight rows (one per lane of tensor memory) and a K slice; a
// cluster of `ksplit` CTAs covers all of K and rank 0 adds the partial sums through
// distributed shared memory.  Warp roles:
//   warp  0     TMA producer: one lane streams 128-row x 128-byte boxes of packed codes
//               (cp.async.bulk.tensor, 128-byte swizzle) into a ring of 16 KB stages; when the
//               whole K slice fits the ring it is in flight before the activations exist;
//   warps 1-2   MMA issuers (even / odd tiles; issuing one tcgen05.mma costs its thread ~50
//               cycles, more than the tensor core needs for it): per 128-k tile four
//               tcgen05.mma.kind::i8 (M=128, N=16 or 32, K=32).  8-bit codes are the A operand as
//               they arrive (the stage is the K-major, swizzled A tile); narrower codes come from
//               tensor memory.  B (the limbs, prepared once per CTA) is 128-byte-swizzled
//               shared memory.  Warp 1 also owns the tensor-memory allocation;
//   warps 3-10  epilogue in two sets that alternate pairs of tiles, one weight row per thread:
//               prefetch the row's scales/biases with cp.async, tcgen05.ld the group sums,
//               scale, accumulate in registers;
//   warps 11-18 (2- and 4-bit) unpackers, one weight row per thread: read the row's packed
//               bytes of a tile from the stage, expand them to one byte per code in registers and
//               tcgen05.st them as the A operand of the tile.
// The order of the 16 codes inside every 16-byte unit of A is whatever is cheapest to unpack;
// the limbs of x are written in the same order.
// Every mbarrier wait is bounded: a wait that runs out sets the library's status word and the
// CTA runs on to the common exit without waiting again.
#include "jq_mma.cuh"
#include "jq_qgemv.cuh"
#include "jq_tc.cuh"

namespace jq {

namespace tcv {

constexpr int ROWS = 128;        // weight rows per CTA
constexpr int TK = 128;          // k per tile = bytes of one A row per tile
constexpr int MAXNS = 12;        // most stages of packed codes
constexpr int BOX_BYTES = ROWS * 128;   // one TMA box: 128 rows x 128 bytes
constexpr int SQ = 4;            // sidecar quads (4 groups) in flight per row and epilogue set
constexpr int W_MMA = 1, W_EPI = 3, W_UNP = 11;
constexpr uint32_t POLLS = 1u << 18;
__host__ __device__ constexpr int threads_for(int bits) { return bits == 8 ? W_UNP * 32 : (W_UNP + 8) * 32; }

__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* own, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(own)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Ring of tiles in tensor memory: tile t uses A slot (narrow codes) and accumulator t % R.
template <int BITS, int GS, int NCOL> struct Ring {
    static constexpr int GPT = TK / GS;                    // groups per tile (2 or 1)
    static constexpr int DW = GPT * NCOL;                  // accumulator columns of one tile
    static constexpr int R = (256 / DW) < 8 ? (256 / DW) : 8;
    static constexpr int RP = R / 2;                       // ... handled in pairs of tiles: ring of RP pairs
    static constexpr int A_COLS = BITS == 8 ? 0 : R * 32;  // 8-bit codes are read from shared memory
    // a stage of packed codes: one box (4 or 2 tiles of narrow codes) or, for 8-bit codes, two boxes = one pair
    static constexpr int STAGE_BYTES = BITS == 8 ? 2 * BOX_BYTES : BOX_BYTES;
    static constexpr int MAX_STAGES = BITS == 8 ? MAXNS / 2 : MAXNS;
    static constexpr int NEED = A_COLS + R * DW;
    static constexpr int TMEM_COLS = NEED <= 128 ? 128 : NEED <= 256 ? 256 : 512;
};

// tensor maps of the matrices of one (possibly fused) launch
struct TcMaps {
    CUtensorMap m[GEMV_MAX_FUSE];
};

// shared-memory map (offsets from a 1024-byte aligned base)
struct Map {
    int tab, red, sc, b, raw, total;
};
__host__ __device__ inline Map make_map(int ncol, int slice_tiles, int slice_groups, int ns, int stage_bytes) {
    Map m;
    // [0, 512): mbarriers and the tensor-memory slot
    m.tab = 512;                                       // float2 (e, sum xi) [slice_groups][8]
    m.red = m.tab + slice_groups * 64;                 // f32 [2][128][8]
    m.sc = m.red + 2 * ROWS * 8 * 4;                   // [2 sets][SQ][128] cells of 16 bytes (scale quad, bias quad)
    m.b = (m.sc + 2 * SQ * ROWS * 16 + 1023) / 1024 * 1024;   // limbs: slice_tiles tiles of ncol rows x 128 bytes
    m.raw = m.b + slice_tiles * ncol * 128;            // ns stages, 1024-byte aligned
    m.total = m.raw + ns * stage_bytes;
    return m;
}

template <typename AT, int BITS, int GS, int NCOL>
__global__ void __launch_bounds__(threads_for(BITS), BITS == 8 ? 2 : 1)
qgemv_tc_kernel(const __grid_constant__ TcMaps maps, const GemvArgs a, const GemvBatch bt) {
    using A = Act<AT>;
    using RG = Ring<BITS, GS, NCOL>;
    constexpr int THREADS = threads_for(BITS);
    constexpr int PREP = W_UNP * 32;           // warps 0..10 prepare the activations
    constexpr int TILE_B = TK * BITS / 8;      // packed bytes of one row and tile (32, 64 or 128)
    constexpr int TPS = BITS == 8 ? 2 : 128 / TILE_B;   // tiles per stage (4, 2 or 2)
    constexpr int STAGE_BYTES = RG::STAGE_BYTES;
    constexpr int GPT = RG::GPT;
    constexpr int KPG = GS / 32;               // MMAs per group (2 or 4)
    constexpr int TPQ = 4 * GS / TK;           // tiles per sidecar quad (2 or 4)
    constexpr int DW = RG::DW, RP = RG::RP;
    constexpr int MMAX = NCOL == 16 ? 5 : 8;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = a.ksplit, NS = a.nbuf;
    const int rbg = blockIdx.x / S;                      // row block of the launch
    const int cr = blockIdx.x - rbg * S;                 // rank in the cluster (cluster shape (S,1,1))
    int mi = 0, blk0 = 0;                                // matrix of a fused launch, its first row block
    while (mi + 1 < bt.count && rbg >= bt.blk_end[mi]) { blk0 = bt.blk_end[mi]; ++mi; }
    const int rb = rbg - blk0;
    const int64_t N = bt.N[mi], ldy = bt.ldy[mi];
    const CUtensorMap* wmap = &maps.m[mi];
    const int M = a.M, G = a.G;
    const int nquads = G / 4;                            // K in units of 4 groups
    const int q_begin = (int)((int64_t)cr * nquads / S), q_end = (int)((int64_t)(cr + 1) * nquads / S);
    const int sq_max = (nquads + S - 1) / S;             // longest slice of the cluster, quads
    const int nq = q_end - q_begin;                      // this CTA's slice
    const int ntiles = nq * TPQ;                         // even
    const int nstages = (ntiles + TPS - 1) / TPS;
    const int t_begin = q_begin * TPQ;                   // first tile of the slice (global tile index)
    const int k_begin = t_begin * TK;
    const int64_t n0 = (int64_t)rb * ROWS;

    const Map mp = make_map(NCOL, sq_max * TPQ, sq_max * 4, NS, STAGE_BYTES);
    uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem);      // [MAXNS]
    uint64_t* raw_empty = raw_full + MAXNS;                      // [MAXNS]
    uint64_t* a_full = raw_empty + MAXNS;                        // [8]
    uint64_t* d_full = a_full + 8;                               // [8]
    uint64_t* d_empty = d_full + 8;                              // [8]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 8);
    float2* tab = reinterpret_cast<float2*>(smem + mp.tab);
    float* red = reinterpret_cast<float*>(smem + mp.red);
    uint8_t* sc_ring = smem + mp.sc;
    uint8_t* sB = smem + mp.b;
    uint8_t* sRaw = smem + mp.raw;

    const uint16_t* xs16 = reinterpret_cast<const uint16_t*>(a.x);
    const uint16_t* sc16 = reinterpret_cast<const uint16_t*>(bt.scales[mi]);
    const uint16_t* bi16 = reinterpret_cast<const uint16_t*>(bt.biases[mi]);
    uint16_t* y16 = reinterpret_cast<uint16_t*>(bt.y[mi]);

    // ---- set-up: barriers, tensor memory, first weight copies (static data) -----------------------------
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    auto produce = [&](int st) {       // one lane: stage st of the slice
        const int s = st % NS;
        mbar_expect_tx(raw_full + s, STAGE_BYTES);
        if constexpr (BITS == 8) {
            tma_load_2d(sRaw + (size_t)s * STAGE_BYTES, wmap, (t_begin + 2 * st) * 128, (int)n0, raw_full + s);
            tma_load_2d(sRaw + (size_t)s * STAGE_BYTES + BOX_BYTES, wmap, (t_begin + 2 * st + 1) * 128, (int)n0, raw_full + s);
        } else {
            tma_load_2d(sRaw + (size_t)s * STAGE_BYTES, wmap, t_begin * TILE_B + st * 128, (int)n0, raw_full + s);
        }
    };
    if (tid == 0) {
        for (int i = 0; i < MAXNS; ++i) { mbar_init(raw_full + i, 1); mbar_init(raw_empty + i, BITS == 8 ? 1 : 8); }
        for (int i = 0; i < 8; ++i) { mbar_init(a_full + i, 8); mbar_init(d_full + i, 1); mbar_init(d_empty + i, 4); }
        mbar_fence_init();
        for (int st = 0; st < NS && st < nstages; ++st) produce(st);
    }
    if (warp == W_MMA) tmem_alloc(tmem_slot, RG::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base, tmem_d = tmem_base + RG::A_COLS;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;   // tensor-memory lane quarter = warp id mod 4
    bool ok = true;

    float acc[MMAX];
#pragma unroll
    for (int m = 0; m < MMAX; ++m) acc[m] = 0.f;
    const int row = (warp & 3) * 32 + lane;              // epilogue and unpacker threads: own weight row
    const int eset = (warp - W_EPI) >> 2;                // epilogue set (0 or 1) of warps 3..10

    if (warp >= W_UNP) {
        if constexpr (BITS != 8) {
            // ---------------- unpackers: packed codes -> one byte per code -> tensor memory ----------------
            // They depend on the weights only, so they start before the activations are ready.
            static_assert(BITS == 2 || BITS == 4 || BITS == 8, "widths of this kernel");
            constexpr int NCH = TILE_B / 16;                          // 16-byte chunks of one row and tile
            const int half = (warp - W_UNP) >> 2;                     // tiles of a stage alternate between two warp sets
            const uint32_t row_off = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
            for (int st = 0; st < nstages && ok; ++st) {
                const int s = st % NS;
                ok = __all_sync(0xFFFFFFFFu, mbar_wait_relaxed(raw_full + s, (uint32_t)(st / NS) & 1u, POLLS));
                if (!ok) break;
                const uint8_t* rowp = sRaw + (size_t)s * STAGE_BYTES + row_off;
#pragma unroll
                for (int t2 = 0; t2 < TPS / 2; ++t2) {
                    const int tt = 2 * t2 + half;
                    const int t = st * TPS + tt;
                    if (t >= ntiles) break;
                    const int pr = t >> 1, pi = pr % RP;                 // pair of tiles and its ring slot
                    uint32_t v[32];
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const uint4 w = *reinterpret_cast<const uint4*>(
                            rowp + (((uint32_t)(tt * NCH + i) ^ (uint32_t)(row & 7)) << 4));
                        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if constexpr (BITS == 4) {
                                v[8 * i + 2 * j] = ws[j] & 0x0F0F0F0Fu;
                                v[8 * i + 2 * j + 1] = (ws[j] >> 4) & 0x0F0F0F0Fu;
                            } else {
                                v[16 * i + 4 * j] = ws[j] & 0x03030303u;
                                v[16 * i + 4 * j + 1] = (ws[j] >> 2) & 0x03030303u;
                                v[16 * i + 4 * j + 2] = (ws[j] >> 4) & 0x03030303u;
                                v[16 * i + 4 * j + 3] = (ws[j] >> 6) & 0x03030303u;
                            }
                        }
                    }
                    if (pr >= RP) {    // the MMAs of pair pr - RP have read this A slot
                        ok = __all_sync(0xFFFFFFFFu, mbar_wait_relaxed(d_full + pi, (uint32_t)((pr / RP) - 1) & 1u, POLLS));
                        if (!ok) break;
                        tc_fence_after();
                    }
                    tmem_st32(tmem_a + lane_base + (uint32_t)((2 * pi + (t & 1)) * 32), v);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(a_full + pi);
                }
                __syncwarp();                                         // every lane has read its row of the stage
                if (lane == 0) mbar_arrive(raw_empty + s);
            }
        }
    } else {
        // ---- warps 0..10: activations of the slice -> limbs (B operand) + per-group (e, sum xi) ---------------
        // epilogue threads: i-th pair of tiles of set `eset` is pair 2i + eset of the slice; its sidecars are
        // quad 2i + eset (groups of 64: one pair per quad) or quad i (groups of 128: two pairs per quad)
        const int npairs = ntiles / 2;
        const int my_pairs = warp >= W_EPI ? (npairs - eset + 1) / 2 : 0;
        const int64_t n_row = min(n0 + row, N - 1);
        uint8_t* my_sc = sc_ring + (size_t)(eset & 1) * SQ * ROWS * 16;
        auto issue_sc = [&](int i) {
            if (i < my_pairs) {
                uint8_t* cell = my_sc + ((size_t)(i % SQ) * ROWS + row) * 16;
                const int quad = GS == 64 ? 2 * i + eset : i;
                const int64_t off = n_row * G + (int64_t)(q_begin + quad) * 4;
                cp_async8(cell, sc16 + off);
                cp_async8(cell + 8, bi16 + off);
            }
            cp_async_commit();
        };
        if (warp >= W_EPI) {
#pragma unroll
            for (int i = 0; i < SQ - 1; ++i) issue_sc(i);
        }
        {   // rows of B that carry no limb are zero (independent of the activations)
            const int zq = (NCOL - 3 * M) * 8;               // 16-byte chunks per tile, fewer than PREP
            if (tid < zq) {
                const int n = 3 * M + (tid >> 3), c = tid & 7;
                uint8_t* p0 = sB + (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4);
                for (int t = 0; t < ntiles; ++t)
                    *reinterpret_cast<uint4*>(p0 + (size_t)t * (NCOL * 128)) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        {
            // eight consecutive activations per lane; GS/8 adjacent lanes form a quantization group.
            // The loads of all PF rounds are issued together, so their latency is paid once.
            constexpr int LPG = GS / 8;
            constexpr int PF = 2;
            const int per_row = ntiles * (TK / 8);
            const int items = M * per_row;                   // a multiple of 32
            for (int base0 = warp * 32; base0 < items; base0 += PREP * PF) {
                uint4 rawv[PF];
#pragma unroll
                for (int i = 0; i < PF; ++i) {
                    const int it = base0 + i * PREP + lane;
                    if (it < items) {
                        const int m = it / per_row;
                        rawv[i] = *reinterpret_cast<const uint4*>(xs16 + (int64_t)m * a.ldx + k_begin + (it - m * per_row) * 8);
                    }
                }
#pragma unroll
                for (int i = 0; i < PF; ++i) {
                    const int it = base0 + i * PREP + lane;
                    if (it >= items) break;                  // warp-uniform: items is a multiple of 32
                    const int m = it / per_row;
                    const int ko = it - m * per_row;         // octet of the slice
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
                    const int u = ko >> 1, hf = ko & 1;      // 16-code unit of the slice, which half of it
                    const int t = u >> 3, c = u & 7;         // tile of the slice, 16-byte chunk of its 128-byte row
                    uint8_t* tile = sB + (size_t)t * (NCOL * 128);
                    // The order of the 16 codes inside a 16-byte unit of A is whatever is cheapest to unpack;
                    // the limbs follow the same order (store_limbs8).
                    auto unit = [&](int n) {
                        return tile + (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4);
                    };
                    store_limbs8<BITS>(unit(3 * m), unit(3 * m + 1), unit(3 * m + 2), hf, xi);
                    if ((ko & (LPG - 1)) == 0) tab[(ko / LPG) * 8 + m] = make_float2(e, (float)sum);
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes of B -> tensor-core reads
        asm volatile("bar.sync 1, %0;" ::"n"(PREP) : "memory");

        if (warp == 0) {
            // ---------------- TMA producer (the first NS stages are already in flight) ----------------
            if (lane == 0) {
                for (int st = NS; st < nstages; ++st) {
                    ok = mbar_wait_relaxed(raw_empty + st % NS, (uint32_t)((st / NS) - 1) & 1u, POLLS);
                    if (!ok) break;
                    produce(st);
                }
            }
        } else if (warp < W_EPI) {
            // ---------------- MMA issuers: warp 1 takes the even pairs of tiles, warp 2 the odd ones ----------------
            if (lane == 0) {
                constexpr uint32_t idesc = umma_idesc_i8(NCOL);
                const uint32_t b_lo0 = umma_desc_sw128_lo(smem_u32(sB)), raw_lo0 = umma_desc_sw128_lo(smem_u32(sRaw));
                const int npairs_ = ntiles / 2;
                for (int pr = warp - W_MMA; pr < npairs_ && ok; pr += 2) {
                    const int pi = pr % RP, s = pr % NS;
                    if constexpr (BITS == 8) ok = mbar_wait(raw_full + s, (uint32_t)(pr / NS) & 1u, POLLS);
                    else ok = mbar_wait(a_full + pi, (uint32_t)(pr / RP) & 1u, POLLS);
                    if (ok && pr >= RP) ok = mbar_wait(d_empty + pi, (uint32_t)((pr / RP) - 1) & 1u, POLLS);
                    if (!ok) break;
                    tc_fence_after();
                    // descriptors: one 32-bit add per operand and MMA (the issuing thread is the scarce resource)
                    const uint32_t d0 = tmem_d + (uint32_t)(2 * pi * DW);
                    const uint32_t b_lo = b_lo0 + (uint32_t)(2 * pr) * (uint32_t)(NCOL * 128 >> 4);
                    const uint32_t a_lo = raw_lo0 + (uint32_t)s * (uint32_t)(STAGE_BYTES >> 4);
                    const uint32_t a_tm = tmem_a + (uint32_t)(2 * pi * 32);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint32_t dcol = d0 + (uint32_t)(j * DW + (kk / KPG) * NCOL);
                            const uint64_t bdesc = umma_desc_join(b_lo + (uint32_t)((j * NCOL * 128 + kk * 32) >> 4));
                            if constexpr (BITS == 8)
                                umma_i8_ss(dcol, umma_desc_join(a_lo + (uint32_t)((j * BOX_BYTES + kk * 32) >> 4)), bdesc, idesc,
                                           (kk % KPG) ? 1u : 0u);
                            else
                                umma_i8_ts(dcol, a_tm + (uint32_t)(j * 32 + kk * 8), bdesc, idesc, (kk % KPG) ? 1u : 0u);
                        }
                    }
                    umma_commit(d_full + pi);      // sums ready; for narrow codes also: the A slots are free again
                    if constexpr (BITS == 8) { if (pr + NS < npairs_) umma_commit(raw_empty + s); }   // the stage is free again
                }
            }
        } else {
            // ---------------- epilogue: one weight row per thread, two tiles per step ----------------
            for (int i = 0; i < my_pairs && ok; ++i) {
                issue_sc(i + SQ - 1);
                cp_async_wait<SQ - 1>();                              // sidecars of this pair have landed
                const uint4 cell = *reinterpret_cast<const uint4*>(my_sc + ((size_t)(i % SQ) * ROWS + row) * 16);
                const uint32_t sw[2] = {cell.x, cell.y}, bw[2] = {cell.z, cell.w};
                const int pair = 2 * i + eset;
                const int t0i = 2 * pair;                             // first tile of the pair
                const int g0 = t0i * GPT;                             // its first group (of the slice)
                const int gq0 = GS == 64 ? 0 : 2 * (pair & 1);        // ... and that group's place in the sidecar quad
                const int pi = pair % RP;
                ok = mbar_wait_warp(d_full + pi, (uint32_t)(pair / RP) & 1u, POLLS, true);   // one lane polls
                if (!ok) break;
                tc_fence_after();
                if (NCOL == 16 && M == 1) {
                    // three columns per group: load every group of the pair, then one wait
                    uint32_t d4[2 * GPT][4];
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int gi = 0; gi < GPT; ++gi)
                            tmem_ld4_nowait(tmem_d + lane_base + (uint32_t)((2 * pi + j) * DW + gi * NCOL), d4[j * GPT + gi]);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(d_empty + pi);
#pragma unroll
                    for (int j = 0; j < 2 * GPT; ++j) {
                        const int gq = gq0 + j;                       // group of the quad
                        const float s = (gq & 1) ? A::hi_f32(sw[gq >> 1]) : A::lo_f32(sw[gq >> 1]);
                        const float bs = (gq & 1) ? A::hi_f32(bw[gq >> 1]) : A::lo_f32(bw[gq >> 1]);
                        const float2 es = tab[(g0 + j) * 8];
                        const float f = fmaf((float)(int)d4[j][2], 65536.f, fmaf((float)(int)d4[j][1], 256.f, (float)(int)d4[j][0]));
                        acc[0] = fmaf(es.x, fmaf(s, f, bs * es.y), acc[0]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
#pragma unroll
                        for (int gi = 0; gi < GPT; ++gi) {
                            uint32_t dv[NCOL];
                            const uint32_t dcol = tmem_d + lane_base + (uint32_t)((2 * pi + j) * DW + gi * NCOL);
                            if constexpr (NCOL == 16) tmem_ld16(dcol, dv); else tmem_ld32(dcol, dv);
                            const int gq = gq0 + j * GPT + gi;
                            const float s = (gq & 1) ? A::hi_f32(sw[gq >> 1]) : A::lo_f32(sw[gq >> 1]);
                            const float bs = (gq & 1) ? A::hi_f32(bw[gq >> 1]) : A::lo_f32(bw[gq >> 1]);
#pragma unroll
                            for (int m = 0; m < MMAX; ++m) {
                                if (m < M) {
                                    const float2 es = tab[(g0 + j * GPT + gi) * 8 + m];
                                    const float f = fmaf((float)(int)dv[3 * m + 2], 65536.f,
                                                         fmaf((float)(int)dv[3 * m + 1], 256.f, (float)(int)dv[3 * m]));
                                    acc[m] = fmaf(es.x, fmaf(s, f, bs * es.y), acc[m]);
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(d_empty + pi);
                }
            }
            cp_async_wait<0>();
            // the two sets add their partial sums: set 1 -> shared memory -> set 0
            if (eset == 1) {
#pragma unroll
                for (int m = 0; m < MMAX; ++m) red[(ROWS + row) * 8 + m] = acc[m];
            }
            asm volatile("bar.sync 2, 256;" ::: "memory");
            if (eset == 0) {
#pragma unroll
                for (int m = 0; m < MMAX; ++m) acc[m] += red[(ROWS + row) * 8 + m];
            }
        }
    }
    if (!ok) atomicOr(a.status, JQ_STATUS_LOCAL_WAIT);

    // ---- results: direct store, or partial sums to rank 0 through distributed shared memory -----------------
    const bool owner = warp >= W_EPI && warp < W_EPI + 4;             // set 0 holds the CTA's sums
    if (S == 1) {
        if (owner && n0 + row < N) {
#pragma unroll
            for (int m = 0; m < MMAX; ++m)
                if (m < M) y16[(int64_t)m * ldy + n0 + row] = A::from_f32(acc[m]);
        }
    } else {
        if (owner) {
#pragma unroll
            for (int m = 0; m < MMAX; ++m) red[row * 8 + m] = acc[m];
        }
        cluster_sync_all();
        if (cr == 0) {
            for (int idx = tid; idx < ROWS * M; idx += THREADS) {
                const int m = idx / ROWS, rr = idx - m * ROWS;
                float v = red[rr * 8 + m];
                for (int s = 1; s < S; ++s) v += ld_cluster_f32(red + rr * 8 + m, (uint32_t)s);
                if (n0 + rr < N) y16[(int64_t)m * ldy + n0 + rr] = A::from_f32(v);
            }
        }
        cluster_sync_all();    // peers keep their shared memory alive until rank 0 has read it
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem_base, RG::TMEM_COLS);
    }
}

template <typename AT, int BITS, int GS, int NCOL>
static int launch_cfg(const TcMaps& maps, GemvArgs a, GemvBatch bt, int S, int ns, cudaStream_t st, bool* launched) {
    constexpr int TPQ = 4 * GS / TK;
    const int nquads = a.G / 4;
    const int sq_max = (nquads + S - 1) / S;
    const Map mp = make_map(NCOL, sq_max * TPQ, sq_max * 4, ns, Ring<BITS, GS, NCOL>::STAGE_BYTES);
    const int smem = mp.total + 1024;
    if (smem > 227 * 1024) return JQ_OK;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_tc_kernel<AT, BITS, GS, NCOL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        227 * 1024));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    a.ksplit = S;
    a.nbuf = ns;
    a.status = status_word();
    JQ_REQUIRE(a.status != nullptr, JQ_ECUDA, "could not locate the device status word");
    int64_t row_blocks = 0;
    for (int i = 0; i < bt.count; ++i) {
        row_blocks += (bt.N[i] + ROWS - 1) / ROWS;
        bt.blk_end[i] = (int)row_blocks;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)row_blocks * (unsigned)S);
    cfg.blockDim = dim3(threads_for(BITS));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (S > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)S;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (a.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemv_tc_kernel<AT, BITS, GS, NCOL>, maps, a, bt));
    *launched = true;
    return JQ_OK;
}

// Cluster size and ring depth.
//   * Few row blocks (at most one CTA per SM): the largest S <= 8 that still gives every SM at most one
//     CTA; the ring then holds the CTA's whole K slice where it fits, so that all of the matrix is in
//     flight before the activations arrive (the launch may overlap its predecessor).
//   * Many row blocks: S grows only until the limbs of a slice fit beside a deep ring; CTAs run in waves.
template <typename AT, int BITS, int GS, int NCOL>
static int launch_shape(const TcMaps& maps, const GemvArgs& a, const GemvBatch& bt, cudaStream_t st, bool* launched) {
    constexpr int TPQ = 4 * GS / TK;
    using RG = Ring<BITS, GS, NCOL>;
    constexpr int TPS = BITS == 8 ? 2 : 8 / BITS;          // tiles per stage
    const int sms = sm_count();
    const int nquads = a.G / 4;
    int64_t row_blocks = 0;
    for (int i = 0; i < bt.count; ++i) row_blocks += (bt.N[i] + ROWS - 1) / ROWS;
    int S = 1;
    if (row_blocks <= sms) {
        while (S < 8 && S < nquads && row_blocks * (S + 1) <= sms) ++S;
    }
    auto fit_ns = [&](int s_) {
        const int sq_max = (nquads + s_ - 1) / s_;
        const int want = (sq_max * TPQ + TPS - 1) / TPS;      // stages of the longest slice
        int ns = want < RG::MAX_STAGES ? want : RG::MAX_STAGES;
        if (BITS == 8 && (ns & 1)) ++ns;                      // see below: even rings only
        if (ns < 2) ns = 2;
        while (ns > 2 && make_map(NCOL, sq_max * TPQ, sq_max * 4, ns, RG::STAGE_BYTES).total + 1024 > 227 * 1024) --ns;
        // 8-bit codes: a stage holds one pair of tiles and the two MMA warps take alternate pairs.  With an
        // even ring every stage barrier is waited on by one warp only, phase after phase; with an odd ring a
        // warp that runs ahead would test a parity two phases away and read a stage that is still in flight.
        if (BITS == 8 && (ns & 1)) --ns;
        return ns;
    };
    // the limbs of a long slice can crowd out the ring: split K further while fewer than 4 stages fit
    while (S < 8 && S < nquads && fit_ns(S) * RG::STAGE_BYTES < 4 * BOX_BYTES &&
           make_map(NCOL, ((nquads + S - 1) / S) * TPQ, 0, 4, BOX_BYTES).total + 1024 > 227 * 1024) ++S;
    if (S < 1 || S > 8 || S > nquads) return JQ_OK;
    const int ns = fit_ns(S);
    if (ns < 2 || ns > RG::MAX_STAGES || (BITS == 8 && (ns & 1))) return JQ_OK;
    return launch_cfg<AT, BITS, GS, NCOL>(maps, a, bt, S, ns, st, launched);
}

}  // namespace tcv


// Dense mat-vecs (one launch for all matrices of `bt`) on the tensor-memory kernel; *launched stays
// false when the shape does not fit it.
int launch_tc_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                     bool* launched) {
    *launched = false;
    const int64_t rowbytes = a.K * bits / 8;
    if (!(bits == 2 || bits == 4 || bits == 8) || a.K % tcv::TK != 0 || a.G % 4 != 0 || a.M > 8 || rowbytes < 128)
        return JQ_OK;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return JQ_OK;
    // the packed codes of every matrix as a [N][rowbytes] byte matrix; a box is 128 rows x 128 bytes,
    // 128-byte swizzled; rows past N and bytes past the row end read as zero
    tcv::TcMaps maps;
    for (int i = 0; i < GEMV_MAX_FUSE; ++i) {
        const int src = i < bt.count ? i : 0;      // unused slots repeat the first map
        const cuuint64_t gdim[2] = {(cuuint64_t)rowbytes, (cuuint64_t)bt.N[src]};
        const cuuint64_t gstride[1] = {(cuuint64_t)rowbytes};
        const cuuint32_t box[2] = {128, (cuuint32_t)tcv::ROWS};
        const cuuint32_t estr[2] = {1, 1};
        if (i >= bt.count) { maps.m[i] = maps.m[0]; continue; }
        CUresult cr = enc(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint32_t*>(bt.codes[src]), gdim,
                          gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        JQ_REQUIRE(cr == CUDA_SUCCESS, JQ_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)cr);
    }
    int rc = JQ_OK;
#define JQ_TC_CASE(B, GSZ)                                                                                    \
    if (bits == B && gs == GSZ) {                                                                             \
        if (act_dtype == JQ_BF16)                                                                             \
            rc = a.M <= 5 ? tcv::launch_shape<__nv_bfloat16, B, GSZ, 16>(maps, a, bt, st, launched)           \
                          : tcv::launch_shape<__nv_bfloat16, B, GSZ, 32>(maps, a, bt, st, launched);          \
        else                                                                                                  \
            rc = a.M <= 5 ? tcv::launch_shape<__half, B, GSZ, 16>(maps, a, bt, st, launched)                  \
                          : tcv::launch_shape<__half, B, GSZ, 32>(maps, a, bt, st, launched);                 \
    }
    JQ_TC_CASE(2, 64) JQ_TC_CASE(4, 64) JQ_TC_CASE(8, 64) JQ_TC_CASE(2, 128) JQ_TC_CASE(4, 128) JQ_TC_CASE(8, 128)
#undef JQ_TC_CASE
    return rc;
}

}  // namespace jq
