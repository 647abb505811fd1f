// Device building blocks of the item-streaming integer mat-vec kernels (jq_qgemv_stream.cu: a whole program
// of dependent ops in one persistent launch; jq_qgemv_one.cu: one op per launch): item geometry, the cp.async
// copies of an item, the activation limbs, the per-item warp-MMA arithmetic and a warp's walk over its items.
//
// An item is 16 weight rows x 256 bytes of packed codes (192 bytes for 6-bit codes) plus the rows' raw
// 2-byte scales and biases of that K range.  Arithmetic: activations as three signed 8-bit limbs under one
// power-of-two exponent per quantization group, codes as the unsigned operand of mma.sync m16n8k32, exact
// integer sums, acc += e*s*(D0 + 256 D1 + 65536 D2) + b*sum(x)  (one activation row).
#pragma once

#include "jq_imma.cuh"

namespace jq {

namespace stream {

using namespace imma_ops;

constexpr int MAX_SMEM = 227 * 1024;
constexpr int MAX_FUSE = 4;          // matrices of one op (they share x, K, the width and the group size)
constexpr int MAXT = 16;             // 16-row tiles one CTA may touch in one op
// bytes of packed codes per row and item: whole 64-code blocks, 256 bytes (192 for 6-bit codes: 4 blocks of 48)
__host__ __device__ constexpr int rowb_of(int bits) { return bits == 6 || bits == 3 ? 192 : 256; }
constexpr int ZERO_BYTES = 1024 + 64;
constexpr int HEAD0 = ZERO_BYTES;      // zeros, then each kernel's own tables
constexpr unsigned long long WAIT_NS = 500ull * 1000 * 1000;

// Shared-memory row stride of an item's code rows: conflict-free unit loads for each width
__host__ __device__ constexpr int rsb_of(int bits) {
    return rowb_of(bits) + (bits == 2 || bits == 6 || bits == 3 ? 16 : bits == 4 ? 32 : 64);
}
// limb bytes of one 64-code block and limb row: one byte per code, except 3-bit (8 codes on 12 byte positions)
__host__ __device__ constexpr int limb_block_bytes(int bits) { return bits == 3 ? 96 : 64; }
// bytes of one item: 16 code rows at the width's stride, then scales [16][NG] and biases [16][NG] (2-byte)
__host__ __device__ constexpr int item_bytes(int bits, int gs) { return 16 * rsb_of(bits) + 2 * 16 * 2 * ((rowb_of(bits) * 8 / bits) / gs); }
constexpr int SLOT = 5376;
static_assert(item_bytes(2, 64) <= SLOT && item_bytes(4, 64) <= SLOT && item_bytes(8, 64) <= SLOT &&
              item_bytes(2, 128) <= SLOT && item_bytes(4, 128) <= SLOT && item_bytes(8, 128) <= SLOT &&
              item_bytes(6, 64) <= SLOT && item_bytes(6, 128) <= SLOT && SLOT % 16 == 0,
              "one slot size for every width");

struct DevOp {                        // one op as the kernel reads it (256 bytes, 16-byte aligned)
    const uint8_t* codes[MAX_FUSE];
    const uint16_t* scales[MAX_FUSE];
    const uint16_t* biases[MAX_FUSE];
    uint16_t* y[MAX_FUSE];
    const uint16_t* x;                // activations (used when x_acc < 0)
    int N[MAX_FUSE];
    int tile_end[MAX_FUSE];           // first tile after matrix i (tiles of all matrices numbered consecutively)
    int K, G, bits, gs;
    int nst, tiles, items, count;     // nst: items per tile (K stages)
    int q, r, mode, S;                // mode 0: CTA c takes q + (c < r) items from c*q + min(c, r);
                                      // mode 1 (fewer tiles than CTAs): CTA c takes part c % S of tile c / S
    int x_acc;                        // >= 0: x is the previous op's accumulator, first row at this index
    int region;                       // accumulator region of this op (op index % 3)
    int pad[8];
};
static_assert(sizeof(DevOp) == 256, "DevOp is copied with 16-byte loads");

struct TileInfo {                     // one tile of the CTA's run (32 bytes)
    const uint8_t* codes;             // first row of the tile
    const uint16_t* scales;
    const uint16_t* biases;
    int rows_valid;
    int xsel;                         // which set of activation limbs the tile multiplies (0 for a dense op)
};

struct OpCtx {                        // this CTA's share of one op, precomputed by the warp that builds the tables
    int start, cnt;                   // run of items
    int tile_first, nlt;              // first tile the run touches, number of tiles it touches
    int stage0;                       // stage of the run's first item inside its first tile
    int pad[3];
};

struct Sync {                         // head of the workspace
    unsigned int barrier;             // arrivals of this launch (monotonic: op j is done at (j + 1) * grid)
    unsigned int done;                // CTAs that left the kernel; the last one resets both counters
    unsigned int abort;               // set when a wait ran out: nobody waits any more
    unsigned int pad[61];
};
static_assert(sizeof(Sync) == 256, "the op table starts 256 bytes in");

__host__ __device__ inline int limb_stride(int K) { return K + 64; }
__host__ __device__ inline int limb_stride_bits(int K, int bits) { return K / 64 * limb_block_bytes(bits) + 64; }
__host__ __device__ inline size_t head_bytes(int kmax, int nw) {
    const size_t limbs = ((size_t)3 * limb_stride(kmax) + 127) / 128 * 128;
    return HEAD0 + 3 * sizeof(DevOp) + 4 * sizeof(OpCtx) + 2 * MAXT * sizeof(TileInfo) + (size_t)(kmax / 64) * 16 + limbs +
           (size_t)nw * MAXT * 16 * sizeof(float);
}

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// The run of items CTA c owns in op o.
__device__ __forceinline__ void cta_range(const DevOp& o, int c, int& start, int& cnt) {
    if (o.mode == 0) {
        start = c * o.q + min(c, o.r);
        cnt = o.q + (c < o.r ? 1 : 0);
    } else if (c < o.tiles * o.S) {
        const int tile = c / o.S, part = c - tile * o.S;
        const int h = (o.nst + o.S - 1) / o.S;
        const int s0 = part * h, s1 = min(o.nst, s0 + h);
        start = tile * o.nst + s0;
        cnt = max(0, s1 - s0);
    } else {
        start = 0;
        cnt = 0;
    }
}

// Per-op constants a warp keeps in registers.
struct OpGeo {
    int rowbytes;      // packed bytes of one weight row
    int G;             // groups per row
    int rowb;          // packed bytes per row of a full item
    int rsb;           // shared-memory stride of an item's code rows
    int ngb;           // bytes of scales (or biases) per row of a full item: 2 * groups per item
    int grpb;          // packed bytes of one quantization group
    int bits, gs;
};
__device__ __forceinline__ OpGeo geo_of(const DevOp& o) {
    OpGeo ge;
    ge.rowbytes = o.K * o.bits / 8;
    ge.G = o.G;
    ge.rowb = rowb_of(o.bits);
    ge.rsb = rsb_of(o.bits);
    ge.grpb = o.bits * o.gs / 8;
    ge.ngb = 2 * (ge.rowb / ge.grpb);
    ge.bits = o.bits;
    ge.gs = o.gs;
    return ge;
}

// cp.async with the destination given as a shared-memory address (no generic-to-shared conversion per copy)
__device__ __forceinline__ void cp16_s(uint32_t saddr, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(src) : "memory");
}
__device__ __forceinline__ void cp8_s(uint32_t saddr, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(saddr), "l"(src) : "memory");
}
__device__ __forceinline__ void cp4_s(uint32_t saddr, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(saddr), "l"(src) : "memory");
}

// cp.async copies of one item (tile ti, K stage st) into slot `buf`: 16 code rows of up to 256 bytes, then
// the rows' scales and biases of the stage.  Rows past the matrix and bytes past the row end are not copied
// (their results are never used).  A whole item (the common case) takes no per-copy predicate.
// Measured and dropped: the 16 code rows as 16 bulk copies of the copy engine (one warp instruction, mbarrier
// completion) instead of eight 16-byte cp.async instructions -- 256-byte bulk requests run at about one per
// 17 cycles and SM, 4.2 TB/s on a 32000x4096 8-bit matrix against 5.4 TB/s with cp.async.
__device__ __forceinline__ void issue_item(uint8_t* buf, const TileInfo& ti, int st, const OpGeo& ge, int lane) {
    const uint32_t sb = smem_u32(buf);
    const int hi = lane >> 4, lo = lane & 15;
    const int rows_valid = ti.rows_valid;
    const int koff = st * ge.rowb;                               // byte offset of the stage inside a row
    const uint8_t* src = ti.codes + (uint32_t)(koff + hi * ge.rowbytes + lo * 16);     // offsets inside a tile fit 32 bits
    const uint32_t dst = sb + hi * ge.rsb + lo * 16;
    const uint32_t gstep = 2u * (uint32_t)ge.rowbytes, sstep = 2u * (uint32_t)ge.rsb;
    const uint16_t* sp = (hi ? ti.biases : ti.scales) + (uint32_t)(min(lo, rows_valid - 1) * ge.G + st * (ge.ngb >> 1));
    const uint32_t sd = sb + 16 * ge.rsb + (hi * 16 + lo) * ge.ngb;
    if (rows_valid == 16 && koff + ge.rowb <= ge.rowbytes) {
        if (lo * 16 < ge.rowb) {
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) cp16_s(dst + rr * sstep, src + rr * gstep);
        }
        if (ge.ngb == 32) {
            cp8_s(sd, sp); cp8_s(sd + 8, sp + 4); cp8_s(sd + 16, sp + 8); cp8_s(sd + 24, sp + 12);
        } else if (ge.ngb == 16) {
            cp8_s(sd, sp); cp8_s(sd + 8, sp + 4);
        } else if (ge.ngb == 8) {
            cp8_s(sd, sp);
        } else {
            cp4_s(sd, sp);
        }
        return;
    }
    // edge item: rows past the matrix are skipped, a row's last stage may be short (whole groups)
    const int kc = min(ge.rowb, ge.rowbytes - koff);
    if (lo * 16 < kc) {
#pragma unroll
        for (int rr = 0; rr < 8; ++rr)
            if (2 * rr + hi < rows_valid) cp16_s(dst + rr * sstep, src + rr * gstep);
    }
    const int ngv_b = (kc / ge.grpb) * 2;                        // bytes of this stage's groups per row
    if (ge.ngb >= 8) {
#pragma unroll
        for (int p = 0; p < 4; ++p)
            if (p * 8 < ngv_b) cp8_s(sd + p * 8, sp + p * 4);
    } else {
        cp4_s(sd, sp);
    }
}

// Where the activations of an op come from.
struct PrepSrc {
    const uint16_t* xs = nullptr;     // rows of the activation type (or the gate products when `up` is set)
    const float* acc = nullptr;       // instead of xs: the previous op's float32 accumulator (one row)
    const uint16_t* up = nullptr;     // SwiGLU source: up products, same layout as xs
    const float* wts = nullptr;       // SwiGLU source: one routing weight per row (nullptr: 1)
    float limit = 0.f;                // SwiGLU clamp (<= 0: none)
    int64_t ldx = 0;                  // elements between rows of xs / up
    int nx = 1;                       // rows (sets of limbs)
    const int* rowmap = nullptr;      // set s reads row rowmap[s] of xs / up / wts (nullptr: row s)
    bool have_pre = false;            // `pre` holds the thread's first 16 bytes of row 0 (requested ahead of time)
    uint4 pre = {0u, 0u, 0u, 0u};
};

// Activations -> limbs + per-group (e, sum x), by the first `nthreads` threads of the CTA (whole warps).
// Set s of the limbs starts at limbs + s * 3 * LS, its table at tab + s * xtab_stride.  Sources: rows of the
// activation type; the previous op's float32 accumulator, rounded to the activation type first (the value
// the output conversion stores); or gate and up products turned into h = silu(g) * u * weight on the fly.
// A thread takes 8 consecutive activations (one 16-byte load), GS / 8 lanes share a quantization group: this
// step sits on the critical path between two dependent mat-vecs, so it is spread over as many threads as K
// allows, and all of a thread's loads go out before its first conversion.
template <typename AT, int BITS, int GS>
__device__ __forceinline__ void prep_limbs(const PrepSrc& src, int K, uint8_t* limbs, float2* tab, int LS,
                                           int xtab_stride, int tid, int nthreads) {
    using A = Act<AT>;
    constexpr int LPG = GS / 8;                          // lanes per group: 8 or 16
    const int lane = tid & 31;
    const int halves = K / 8;                            // per row; a multiple of 32 (K is a multiple of 4 GS)
    const int total = halves * src.nx;
    constexpr int PRE = 4;
    uint4 xq[PRE];
    if (!src.acc) {
#pragma unroll
        for (int i = 0; i < PRE; ++i) {
            const int idx = tid + i * nthreads;
            xq[i] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < total) {
                const int sx = idx / halves, H = idx - sx * halves;
                const int row = src.rowmap ? src.rowmap[sx] : sx;
                xq[i] = (i == 0 && src.have_pre) ? src.pre : ld_cg16(src.xs + row * src.ldx + (size_t)H * 8);
            }
        }
    }
    int round = 0;
    for (int base = (tid >> 5) * 32; base < total; base += nthreads, ++round) {
        const int idx = base + lane;
        const bool live = idx < total;
        const int sx = live ? idx / halves : 0;
        const int H = idx - sx * halves;                 // half-unit of the row: activations [8 H, 8 H + 8)
        const int srow = src.rowmap ? src.rowmap[sx] : sx;
        float v[8];
        if (!live) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        } else if (src.acc) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 r = ld_cg16(src.acc + (size_t)H * 8 + h * 4);
                const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) v[h * 4 + j] = A::to_f32(A::from_f32(__uint_as_float(w[j])));
            }
        } else {
            uint4 r;
            if (round == 0) r = xq[0];
            else if (round == 1) r = xq[1];
            else if (round == 2) r = xq[2];
            else if (round == 3) r = xq[3];
            else r = ld_cg16(src.xs + srow * src.ldx + (size_t)H * 8);
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] = A::lo_f32(w[j]); v[2 * j + 1] = A::hi_f32(w[j]); }
            if (src.up) {
                // xs holds the gate products: h = silu(min(g, limit)) * clip(u, +-limit) * weight, rounded to
                // the activation type (what a separate SwiGLU launch would store)
                const uint4 ru = ld_cg16(src.up + srow * src.ldx + (size_t)H * 8);
                const uint32_t wu[4] = {ru.x, ru.y, ru.z, ru.w};
                const float wt = src.wts ? src.wts[srow] : 1.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float gv = v[j], uv = (j & 1) ? A::hi_f32(wu[j >> 1]) : A::lo_f32(wu[j >> 1]);
                    if (src.limit > 0.f) {
                        gv = fminf(gv, src.limit);
                        uv = fminf(fmaxf(uv, -src.limit), src.limit);
                    }
                    v[j] = A::to_f32(A::from_f32((gv / (1.0f + __expf(-gv))) * uv * wt));
                }
            }
        }
        uint32_t amax = 0u;                              // largest magnitude, as bits (NaN/inf sort highest)
        float xsum = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { amax = max(amax, __float_as_uint(v[j]) & 0x7FFFFFFFu); xsum += v[j]; }
#pragma unroll
        for (int d = 1; d < LPG; d <<= 1) {
            amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
            xsum += __shfl_xor_sync(0xFFFFFFFFu, xsum, d);
        }
        uint32_t eb = amax >> 23;
        const bool finite = eb != 255u;
        eb = max(eb, 21u);
        const float scale = __uint_as_float((275u - eb) << 23);      // 2^(21 - E): |x| * scale < 2^22
        float e = __uint_as_float((eb - 21u) << 23);                 // 2^(E - 21)
        if (!finite) e = __uint_as_float(0x7FC00000u);               // non-finite input -> NaN output
        if (live) {
            // element j meets a code that carries the factor 2^code_shift(j): scale it down by that (the
            // pattern repeats every 4 elements, so both halves of a 16-code unit see the same factors)
            int xi[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                xi[j] = __float2int_rn(v[j] * (scale * (1.f / (float)(1 << code_shift<BITS>(j)))));
            if constexpr (BITS == 3) {
                uint8_t* u0 = limbs + (size_t)sx * 3 * LS + (size_t)H * 12;
                store_limbs3(u0, u0 + LS, u0 + 2 * LS, xi);
            } else {
                uint8_t* u0 = limbs + (size_t)sx * 3 * LS + (size_t)(H >> 1) * 16;
                store_limbs8<BITS == 6 ? 8 : BITS>(u0, u0 + LS, u0 + 2 * LS, H & 1, xi);
            }
            if ((H & (LPG - 1)) == 0) {
                float2* t = tab + (size_t)sx * xtab_stride + (H / LPG) * 2;
                t[0] = make_float2(e, 0.f);                          // lanes that carry scales: D * e
                t[1] = make_float2(0.f, xsum);                       // lanes that carry biases: sum x
            }
        }
    }
}

// One item: 16 rows x nblk 64-code blocks against the limbs.  buf: the item's slot; bp: the lane's limb
// bytes of the stage's first block (MMA column g = limb g for g < 3, zeros otherwise), tp: the lane's
// (e, sum x) entries of the stage's first group.  A lane computes acc += f * (D * el + xl) with
// (f, el, xl) = (scale, e, 0) in the lanes tig < 2 (they hold D0 + 256 D1, resp. D2) and (bias, 0, sum x)
// in the lanes tig >= 2 (their D is 0): the same two FMAs everywhere.  Returns the lane's partial sums of
// rows g and g + 8 (to be weighed by 1 / 65536 / 1 / 0 per tig and added over the quad).
// The blocks are walked in runs of at most 8 (a rolled loop over the runs keeps the loop body within the
// instruction cache; only 2-bit items have two runs).
template <typename AT, int BITS, int GS, bool FULL>
__device__ __forceinline__ void compute_item(const uint8_t* buf, const uint8_t* bp, const float2* tp, int nblk, int g,
                                             int tig, float& acc_lo, float& acc_hi) {
    using A = Act<AT>;
    constexpr int KT = rowb_of(BITS) * 8 / BITS, NBLK = KT / 64, NG = KT / GS, NGB = NG * 2, BPG = GS / 64;
    constexpr int RSB = rsb_of(BITS);
    constexpr int UW = Unit<BITS>::WORDS;
    constexpr int RUN = NBLK < 8 ? NBLK : 8;             // blocks per run
    constexpr int RG = RUN / BPG;                        // groups per run
    constexpr int NR = RG >= 2 ? RG / 2 : 1;             // registers of packed 2-byte pairs per row and run
    const uint32_t* c_lo = reinterpret_cast<const uint32_t*>(buf + g * RSB);
    const uint32_t* c_hi = reinterpret_cast<const uint32_t*>(buf + (g + 8) * RSB);
    const uint8_t* sc = buf + 16 * RSB + (tig >> 1) * (16 * NGB);       // scales for tig < 2, biases for tig >= 2
    const uint8_t* sp_lo = sc + g * NGB;
    const uint8_t* sp_hi = sc + (g + 8) * NGB;
    auto load_pairs = [&](const uint8_t* p, uint32_t (&d)[NR]) {
        if constexpr (NR >= 4) {
#pragma unroll
            for (int i = 0; i < NR / 4; ++i) {
                const uint4 v = *reinterpret_cast<const uint4*>(p + 16 * i);
                d[4 * i] = v.x; d[4 * i + 1] = v.y; d[4 * i + 2] = v.z; d[4 * i + 3] = v.w;
            }
        } else if constexpr (NR == 2) {
            const uint2 v = *reinterpret_cast<const uint2*>(p);
            d[0] = v.x; d[1] = v.y;
        } else {
            d[0] = *reinterpret_cast<const uint32_t*>(p);
        }
    };
#pragma unroll 1
    for (int run = 0; run < NBLK / RUN; ++run) {
        if constexpr (!FULL) {
            if (run * RUN >= nblk) break;
        }
        uint32_t s_lo[NR], s_hi[NR];
        load_pairs(sp_lo, s_lo);
        load_pairs(sp_hi, s_hi);
        int cg[4];
        auto block = [&](const int blk) {
            // only the lanes of the three limb columns load; the other columns are zero without touching memory
            uint32_t ulo[UW], uhi[UW];
            load_unit<BITS>(c_lo, blk, tig, ulo);
            load_unit<BITS>(c_hi, blk, tig, uhi);
            if constexpr (BITS == 3) {
                uint2 b0 = make_uint2(0u, 0u), b1 = b0, b2 = b0;
                if (g < 3) {
                    const uint2* bb = reinterpret_cast<const uint2*>(bp + blk * 96);
                    b0 = bb[0]; b1 = bb[1]; b2 = bb[2];
                }
                uint32_t rl[6], rh[6];
                to_bytes3(ulo, rl);
                to_bytes3(uhi, rh);
                if (blk % BPG == 0) imma0(cg, rl[0], rh[0], rl[1], rh[1], b0.x, b0.y);
                else imma(cg, rl[0], rh[0], rl[1], rh[1], b0.x, b0.y);
                imma(cg, rl[2], rh[2], rl[3], rh[3], b1.x, b1.y);
                imma(cg, rl[4], rh[4], rl[5], rh[5], b2.x, b2.y);
            } else {
                uint4 bq = make_uint4(0u, 0u, 0u, 0u);
                if (g < 3) bq = *reinterpret_cast<const uint4*>(bp + blk * 64);
                uint32_t rl[4], rh[4];
                to_bytes<BITS>(ulo, rl);
                to_bytes<BITS>(uhi, rh);
                if (blk % BPG == 0) imma0(cg, rl[0], rh[0], rl[1], rh[1], bq.x, bq.y);
                else imma(cg, rl[0], rh[0], rl[1], rh[1], bq.x, bq.y);
                imma(cg, rl[2], rh[2], rl[3], rh[3], bq.z, bq.w);
            }
            if (blk % BPG == BPG - 1) {
                const int gi = blk / BPG;
                const float2 tx = tp[gi * 2];
                const float f_lo = (gi & 1) ? A::hi_f32(s_lo[gi >> 1]) : A::lo_f32(s_lo[gi >> 1]);
                const float f_hi = (gi & 1) ? A::hi_f32(s_hi[gi >> 1]) : A::lo_f32(s_hi[gi >> 1]);
                const float d_lo = (float)(cg[0] + 256 * cg[1]);
                const float d_hi = (float)(cg[2] + 256 * cg[3]);
                acc_lo = fmaf(f_lo, fmaf(d_lo, tx.x, tx.y), acc_lo);
                acc_hi = fmaf(f_hi, fmaf(d_hi, tx.x, tx.y), acc_hi);
            }
        };
#pragma unroll
        for (int blk = 0; blk < RUN; ++blk) {
            if constexpr (FULL) {
                block(blk);
            } else {
                if (run * RUN + blk < nblk) block(blk);      // a row's last stage may be short (whole groups)
            }
        }
        c_lo += RUN * 2 * BITS;
        c_hi += RUN * 2 * BITS;
        bp += RUN * limb_block_bytes(BITS);
        tp += RG * 2;
        sp_lo += RG * 2;
        sp_hi += RG * 2;
    }
}

// Everything a warp needs to walk its items of one op.
struct WarpCtx {
    const TileInfo* tl;      // the CTA's tiles of the op
    OpGeo ge;
    int cnt, nst, stage0;    // items of the CTA, stages per tile, stage of the CTA's first item in its first tile
    // the warp's first two items of the next op (if any): tiles, stages, geometry
    const TileInfo* tl1;
    OpGeo ge1;
    int lt1, st1, lt1b, st1b;
    int next_n;              // how many of them exist: 0, 1 or 2
};

// The warp's items of one op.  slot: the slot of the warp's current item; npre: how many of the warp's
// leading items of this op have been requested already (while the previous op was still running): 0..2.
// Every request is one cp.async group, and every loop iteration commits exactly one group (an empty one
// when there is nothing to request), so "all but the newest group" always covers the current item.
// Behind its last item of the op the warp requests its first two items of the next op, so that both of its
// slots are in flight while the CTA sits in the op boundary.
// XSETS: the tiles name their set of activation limbs (TileInfo::xsel; set s starts at limbs + s * 3 * LS and
// tab + s * xtab_stride): the routed-expert gather, where every (token, slot) pair may bring its own row.
template <typename AT, int BITS, int GS, int NW, bool XSETS = false>
__device__ __forceinline__ void run_op(const WarpCtx& w, uint8_t* ring, const uint8_t* limbs, int LS,
                                       const uint8_t* zero, const float2* tab, float* myy, int warp, int lane, int& slot,
                                       int& npre, int xtab_stride = 0) {
    constexpr int RB = rowb_of(BITS), KT = RB * 8 / BITS, NBLK = KT / 64, NG = KT / GS;
    const int g = lane >> 2, tig = lane & 3;
    const bool bvalid = g < 3;
    constexpr int LBB = limb_block_bytes(BITS);              // limb bytes per block: a quarter of them per tig
    const uint8_t* brow = bvalid ? limbs + (size_t)g * LS + tig * (LBB / 4) : zero + tig * 16;
    const float wl = tig == 1 ? 65536.f : tig == 3 ? 0.f : 1.f;
    const float2* tabm = tab + (tig >> 1);
    int il = warp;
    bool have = il < w.cnt;
    if (!have) {
        // no item in this op: request the first items of the next op now (npre is 0 here)
        if (w.next_n >= 1) {
            issue_item(ring + slot * SLOT, w.tl1[w.lt1], w.st1, w.ge1, lane);
            cp_async_commit();
        }
        if (w.next_n >= 2) {
            issue_item(ring + (slot ^ 1) * SLOT, w.tl1[w.lt1b], w.st1b, w.ge1, lane);
            cp_async_commit();
        }
        npre = w.next_n;
        return;
    }
    int pos = w.stage0 + il;
    int lt = pos / w.nst, st = pos - lt * w.nst;
    int ahead = npre;                         // items from the current one on that are requested
    if (ahead == 0) {
        issue_item(ring + slot * SLOT, w.tl[lt], st, w.ge, lane);
        cp_async_commit();
        ahead = 1;
    }
    int pre_next = 0;
    while (have) {
        const int nil = il + NW;
        const bool have_n = nil < w.cnt;
        int nlt = lt, nst_ = st + NW;
        while (nst_ >= w.nst) { nst_ -= w.nst; ++nlt; }
        if (ahead < 2) {
            if (have_n) {
                issue_item(ring + (slot ^ 1) * SLOT, w.tl[nlt], nst_, w.ge, lane);
                ++ahead;
            } else if (w.next_n >= 1) {
                issue_item(ring + (slot ^ 1) * SLOT, w.tl1[w.lt1], w.st1, w.ge1, lane);
                pre_next = 1;
            }
        }
        cp_async_commit();                    // always one group per item so that the count stays uniform
        cp_async_wait<1>();                   // everything but the newest group has landed: the current item
        __syncwarp();
        const uint8_t* buf = ring + slot * SLOT;
        const int kc = min(RB, w.ge.rowbytes - st * RB);
        const int nblk = kc * 8 / (BITS * 64);
        const uint8_t* bp = brow + (bvalid ? st * (KT / 64 * LBB) : 0);
        const float2* tp = tabm + (size_t)(st * NG) * 2;
        if constexpr (XSETS) {
            const int xs_ = w.tl[lt].xsel;
            if (bvalid) bp += (size_t)xs_ * 3 * LS;
            tp += (size_t)xs_ * xtab_stride;
        }
        float a_lo = 0.f, a_hi = 0.f;
        if (nblk == NBLK) compute_item<AT, BITS, GS, true>(buf, bp, tp, nblk, g, tig, a_lo, a_hi);
        else compute_item<AT, BITS, GS, false>(buf, bp, tp, nblk, g, tig, a_lo, a_hi);
        float p_lo = wl * a_lo, p_hi = wl * a_hi;
        p_lo += __shfl_xor_sync(0xFFFFFFFFu, p_lo, 1);
        p_hi += __shfl_xor_sync(0xFFFFFFFFu, p_hi, 1);
        p_lo += __shfl_xor_sync(0xFFFFFFFFu, p_lo, 2);
        p_hi += __shfl_xor_sync(0xFFFFFFFFu, p_hi, 2);
        if (tig == 0) {
            float* yp = myy + lt * 16 + g;
            yp[0] += p_lo;
            yp[8] += p_hi;
        }
        __syncwarp();                         // every lane is done with the slot before it is refilled
        --ahead;
        slot ^= 1;
        il = nil; have = have_n; lt = nlt; st = nst_;
    }
    // the slot just computed is free: the warp's second item of the next op goes there
    if (pre_next == 1 && w.next_n >= 2) {
        issue_item(ring + (slot ^ 1) * SLOT, w.tl1[w.lt1b], w.st1b, w.ge1, lane);
        cp_async_commit();
        pre_next = 2;
    }
    npre = pre_next;
}

}  // namespace stream
}  // namespace jq
