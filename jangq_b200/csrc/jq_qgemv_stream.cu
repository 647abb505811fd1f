// K2, whole-step form: ONE persistent launch walks a program of dependent decode mat-vecs
//     y_j[N_j] = deq(W_j)[N_j, K_j] . x_j[K_j]        (one activation row, 2-, 4- and 8-bit codes)
// e.g. [q,k,v] -> o -> [gate,up] -> down of every layer of a decoder, instead of one launch per op.
//
// Bound: HBM bandwidth.  Algorithmic bytes per op = N*K*bits/8 (codes) + N*(K/gs)*4 (scales, biases) +
// 2*K + 2*N.  With one launch per op, a 17 MB mat-vec (2.7 us of streaming) pays about 3 us of kernel
// boundary, CTA start and limb preparation; here an op boundary is a grid barrier during which the next
// op's weights are already in flight.
//
// Structure: a cooperative launch of one CTA per SM, NW warps each.  An op's work is cut into items of
// 16 weight rows x 256 bytes of packed codes (+ the items' raw 2-byte scales and biases); the items of an
// op are numbered tile-major and CTA c takes a contiguous run of them, warp w every NW-th item of the
// run.  Every warp owns two item slots in shared memory filled by cp.async: while it computes one item the
// next one is in flight, and behind its last item of an op it already requests its first item of the
// next op (weights never depend on earlier ops), so the stream does not stop at an op boundary.
// Arithmetic: the integer warp-MMA form of jq_qgemv_pint.cu (activations as three signed 8-bit limbs under
// one power-of-two exponent per quantization group, codes as the unsigned operand of mma.sync m16n8k32,
// exact integer sums, acc += e*s*(D0 + 256 D1 + 65536 D2) + b*sum(x)).
//
// End of an op, per CTA: the warps' row sums are added in warp order and sent to a float32 accumulator in
// global memory with red.add (a tile's rows come from at most two CTAs, so the sum does not depend on their
// order), then the CTA arrives at a grid barrier (a monotonic counter, release/acquire, bounded wait).
// Behind the barrier every CTA forms the next op's limbs itself -- from the op's activation pointer, or,
// when that pointer is an output of the op just finished, from its float32 accumulator rounded to the
// activation type -- while the accumulator is converted to the output type by whoever's thread index
// matches the row.  Accumulator regions rotate over three ops; the kernel leaves them and its counters at
// zero, so the same prepared program can be launched again and again (also from a CUDA graph).
//
// Every wait is bounded by the global timer; when one runs out the CTA sets the library's status word and an
// abort flag that makes every later wait of the launch return at once.
#include <cstring>
#include <vector>

#include "jq_imma.cuh"

namespace jq {

int* status_word();

namespace stream {

using namespace imma_ops;

constexpr int MAX_SMEM = 227 * 1024;
constexpr int MAX_FUSE = 4;          // matrices of one op (they share x, K, the width and the group size)
constexpr int MAXT = 16;             // 16-row tiles one CTA may touch in one op
constexpr int ROWB = 256;            // bytes of packed codes per row and item
constexpr int ZERO_BYTES = 1024 + 64;
constexpr unsigned long long WAIT_NS = 500ull * 1000 * 1000;

// Shared-memory row stride of an item's code rows: conflict-free unit loads for each width
__host__ __device__ constexpr int rsb_of(int bits) { return ROWB + (bits == 2 ? 16 : bits == 4 ? 32 : 64); }
// bytes of one item: 16 code rows at the width's stride, then scales [16][NG] and biases [16][NG] (2-byte)
__host__ __device__ constexpr int item_bytes(int bits, int gs) { return 16 * rsb_of(bits) + 2 * 16 * 2 * ((ROWB * 8 / bits) / gs); }
constexpr int SLOT = 5376;
static_assert(item_bytes(2, 64) <= SLOT && item_bytes(4, 64) <= SLOT && item_bytes(8, 64) <= SLOT &&
              item_bytes(2, 128) <= SLOT && item_bytes(4, 128) <= SLOT && item_bytes(8, 128) <= SLOT && SLOT % 16 == 0,
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
    int pad;
};

struct Sync {                         // head of the workspace
    unsigned int barrier;             // arrivals of this launch (monotonic: op j is done at (j + 1) * grid)
    unsigned int done;                // CTAs that left the kernel; the last one resets both counters
    unsigned int abort;               // set when a wait ran out: nobody waits any more
    unsigned int pad[61];
};
static_assert(sizeof(Sync) == 256, "the op table starts 256 bytes in");

__host__ __device__ inline int limb_stride(int K) { return K + 64; }
__host__ __device__ inline size_t head_bytes(int kmax, int nw) {
    const size_t limbs = ((size_t)3 * limb_stride(kmax) + 127) / 128 * 128;
    return ZERO_BYTES + 3 * sizeof(DevOp) + 2 * MAXT * sizeof(TileInfo) + (size_t)(kmax / 64) * 16 + limbs +
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
    int rsb;           // shared-memory stride of an item's code rows
    int ngb;           // bytes of scales (or biases) per row of a full item: 2 * groups per item
    int bits, gs;
};
__device__ __forceinline__ OpGeo geo_of(const DevOp& o) {
    OpGeo ge;
    ge.rowbytes = o.K * o.bits / 8;
    ge.G = o.G;
    ge.rsb = rsb_of(o.bits);
    ge.ngb = 2 * (ROWB * 8 / o.bits) / o.gs;
    ge.bits = o.bits;
    ge.gs = o.gs;
    return ge;
}

// cp.async copies of one item (tile ti, K stage st) into slot `buf`: 16 code rows of up to 256 bytes, then
// the rows' scales and biases of the stage.  Rows past the matrix and bytes past the row end are not copied
// (their results are never used).
__device__ __forceinline__ void issue_item(uint8_t* buf, const TileInfo& ti, int st, const OpGeo& ge, int lane) {
    const int kc = min(ROWB, ge.rowbytes - st * ROWB);           // code bytes of this stage
    const int rows_valid = ti.rows_valid;
    {
        const int r2 = lane >> 4, col = lane & 15;
        const uint8_t* src = ti.codes + (int64_t)st * ROWB + (int64_t)r2 * ge.rowbytes + col * 16;
        uint8_t* dst = buf + r2 * ge.rsb + col * 16;
        const bool col_ok = col * 16 < kc;
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            if (col_ok && 2 * rr + r2 < rows_valid) cp_async16(dst, src);
            src += 2 * (int64_t)ge.rowbytes;
            dst += 2 * ge.rsb;
        }
    }
    {
        const int arr = lane >> 4, row = lane & 15;
        const int ngv_b = (kc * 8 / ge.bits / ge.gs) * 2;        // bytes of this stage's groups per row
        const uint16_t* sp = (arr ? ti.biases : ti.scales) + (int64_t)min(row, rows_valid - 1) * ge.G +
                             st * (ge.ngb >> 1);
        uint8_t* sd = buf + 16 * ge.rsb + arr * (16 * ge.ngb) + row * ge.ngb;
        if (ge.ngb >= 8) {
#pragma unroll
            for (int p = 0; p < 4; ++p)
                if (p * 8 < ngv_b) cp_async8(sd + p * 8, sp + p * 4);
        } else {
            cp_async4(sd, sp);
        }
    }
}

// Activations of the next op -> limbs + per-group (e, sum x), by the first `nthreads` threads of the CTA
// (whole warps).  Source: xs (activation type) or, when acc != nullptr, the previous op's float32
// accumulator, rounded to the activation type first (the value the output conversion stores).
template <typename AT, int BITS, int GS>
__device__ __forceinline__ void prep_limbs(const uint16_t* __restrict__ xs, const float* __restrict__ acc, int K,
                                           uint8_t* limbs, float2* tab, int LS, int tid, int nthreads) {
    using A = Act<AT>;
    constexpr int LPG = GS / 16;                         // sixteen activations per lane, LPG lanes per group
    const int lane = tid & 31;
    const int units = K / 16;                            // a multiple of LPG
    for (int base = (tid >> 5) * 32; base < units; base += nthreads) {
        const int U = base + lane;
        const bool live = U < units;
        float v[16];
        if (!live) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
        } else if (acc) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const uint4 r = ld_cg16(acc + (size_t)U * 16 + h * 4);
                const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) v[h * 4 + j] = A::to_f32(A::from_f32(__uint_as_float(w[j])));
            }
        } else {
            const uint4 r0 = ld_cg16(xs + (size_t)U * 16), r1 = ld_cg16(xs + (size_t)U * 16 + 8);
            const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[2 * j] = A::lo_f32(w[j]); v[2 * j + 1] = A::hi_f32(w[j]); }
        }
        uint32_t amax = 0u;                              // largest magnitude, as bits (NaN/inf sort highest)
        float xsum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { amax = max(amax, __float_as_uint(v[j]) & 0x7FFFFFFFu); xsum += v[j]; }
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
            limbs16<BITS>(v, scale, limbs + (size_t)U * 16, limbs + LS + (size_t)U * 16, limbs + 2 * LS + (size_t)U * 16);
            if ((U & (LPG - 1)) == 0) {
                tab[(U / LPG) * 2] = make_float2(e, 0.f);            // lanes that carry scales: D * e
                tab[(U / LPG) * 2 + 1] = make_float2(0.f, xsum);     // lanes that carry biases: sum x
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
template <typename AT, int BITS, int GS, bool FULL>
__device__ __forceinline__ void compute_item(const uint8_t* buf, const uint8_t* bp, const float2* tp, int nblk, int g,
                                             int tig, float& acc_lo, float& acc_hi) {
    using A = Act<AT>;
    constexpr int KT = ROWB * 8 / BITS, NBLK = KT / 64, NG = KT / GS, NGB = NG * 2, BPG = GS / 64;
    constexpr int RSB = rsb_of(BITS);
    constexpr int UW = Unit<BITS>::WORDS;
    constexpr int NR = NG >= 2 ? NG / 2 : 1;             // registers of packed 2-byte pairs per row
    const uint32_t* c_lo = reinterpret_cast<const uint32_t*>(buf + g * RSB);
    const uint32_t* c_hi = reinterpret_cast<const uint32_t*>(buf + (g + 8) * RSB);
    const uint8_t* sc = buf + 16 * RSB + (tig >> 1) * (16 * NGB);       // scales for tig < 2, biases for tig >= 2
    uint32_t s_lo[NR], s_hi[NR];
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
    load_pairs(sc + g * NGB, s_lo);
    load_pairs(sc + (g + 8) * NGB, s_hi);
    int cg[4];
    auto block = [&](const int blk) {
        const uint4 bq = *reinterpret_cast<const uint4*>(bp + blk * 64);
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
            const float f_lo = (gi & 1) ? A::hi_f32(s_lo[gi >> 1]) : A::lo_f32(s_lo[gi >> 1]);
            const float f_hi = (gi & 1) ? A::hi_f32(s_hi[gi >> 1]) : A::lo_f32(s_hi[gi >> 1]);
            const float d_lo = (float)(cg[0] + 256 * cg[1]);
            const float d_hi = (float)(cg[2] + 256 * cg[3]);
            acc_lo = fmaf(f_lo, fmaf(d_lo, tx.x, tx.y), acc_lo);
            acc_hi = fmaf(f_hi, fmaf(d_hi, tx.x, tx.y), acc_hi);
        }
    };
#pragma unroll
    for (int blk = 0; blk < NBLK; ++blk) {
        if constexpr (FULL) {
            block(blk);
        } else {
            if (blk < nblk) block(blk);          // a row's last stage may be short (whole groups)
        }
    }
}

// Everything a warp needs to walk its items of one op.
struct WarpCtx {
    const TileInfo* tl;      // the CTA's tiles of the op
    OpGeo ge;
    int cnt, nst, stage0;    // items of the CTA, stages per tile, stage of the CTA's first item in its first tile
    // the warp's first item of the next op (if any): tile, stage, geometry
    const TileInfo* tl1;
    OpGeo ge1;
    int lt1, st1;
    bool next_has;
};

// The warp's items of one op.  slot / pre: the slot of the warp's current item and whether that item has
// been requested already (while the previous op was still running).
template <typename AT, int BITS, int GS, int NW>
__device__ __forceinline__ void run_op(const WarpCtx& w, uint8_t* ring, const uint8_t* limbs, int LS, const uint8_t* zero,
                                       const float2* tab, float* myy, int warp, int lane, int& slot, bool& pre) {
    constexpr int KT = ROWB * 8 / BITS, NBLK = KT / 64, NG = KT / GS;
    const int g = lane >> 2, tig = lane & 3;
    const bool bvalid = g < 3;
    const uint8_t* brow = bvalid ? limbs + (size_t)g * LS + tig * 16 : zero + tig * 16;
    const float wl = tig == 1 ? 65536.f : tig == 3 ? 0.f : 1.f;
    const float2* tabm = tab + (tig >> 1);
    int il = warp;
    bool have = il < w.cnt;
    bool pre_next = false;
    if (!have) {
        // no item in this op: request the first item of the next op now
        if (w.next_has && !pre) {
            issue_item(ring + slot * SLOT, w.tl1[w.lt1], w.st1, w.ge1, lane);
            cp_async_commit();
            pre_next = true;
        } else {
            pre_next = pre;
        }
        pre = pre_next;
        return;
    }
    int pos = w.stage0 + il;
    int lt = pos / w.nst, st = pos - lt * w.nst;
    if (!pre) {
        issue_item(ring + slot * SLOT, w.tl[lt], st, w.ge, lane);
        cp_async_commit();
    }
    while (have) {
        const int nil = il + NW;
        const bool have_n = nil < w.cnt;
        int nlt = lt, nst_ = st + NW;
        while (nst_ >= w.nst) { nst_ -= w.nst; ++nlt; }
        if (have_n) {
            issue_item(ring + (slot ^ 1) * SLOT, w.tl[nlt], nst_, w.ge, lane);
        } else if (w.next_has) {
            issue_item(ring + (slot ^ 1) * SLOT, w.tl1[w.lt1], w.st1, w.ge1, lane);
            pre_next = true;
        }
        cp_async_commit();                    // always one group per item so that the count stays uniform
        cp_async_wait<1>();                   // the current item's copies have landed
        __syncwarp();
        const uint8_t* buf = ring + slot * SLOT;
        const int kc = min(ROWB, w.ge.rowbytes - st * ROWB);
        const int nblk = kc * 8 / (BITS * 64);
        const uint8_t* bp = brow + (bvalid ? st * KT : 0);
        const float2* tp = tabm + (size_t)(st * NG) * 2;
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
        slot ^= 1;
        il = nil; have = have_n; lt = nlt; st = nst_;
    }
    pre = pre_next;
}

template <typename AT, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
qgemv_stream_kernel(const DevOp* __restrict__ ops, int n_ops, float* __restrict__ yacc, int maxrows, Sync* sync,
                    int* status, int kmax) {
    using A = Act<AT>;
    constexpr int THREADS = NW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, grid = gridDim.x;
    const int LS = limb_stride(kmax);

    uint8_t* zero = smem;
    DevOp* ops_s = reinterpret_cast<DevOp*>(smem + ZERO_BYTES);                       // [3], op j in slot j % 3
    TileInfo* tiles_s = reinterpret_cast<TileInfo*>(ops_s + 3);                        // [2][MAXT], op j in half j & 1
    float2* tab = reinterpret_cast<float2*>(tiles_s + 2 * MAXT);                       // [kmax / 64][2]
    uint8_t* limbs = reinterpret_cast<uint8_t*>(tab) + (size_t)(kmax / 64) * 16;       // [3][LS]
    float* ysum = reinterpret_cast<float*>(limbs + ((size_t)3 * LS + 127) / 128 * 128); // [NW][MAXT * 16]
    uint8_t* ring = smem + head_bytes(kmax, NW) + (size_t)warp * 2 * SLOT;
    float* myy = ysum + (size_t)warp * MAXT * 16;

    // op j's descriptor and this CTA's tiles of it, built by one warp (no CTA barrier needed inside)
    auto build_tables = [&](int j) {
        if (j >= n_ops) return;
        DevOp* od = &ops_s[j % 3];
        if (lane < 16) reinterpret_cast<uint4*>(od)[lane] = ld_cg16(reinterpret_cast<const uint4*>(ops + j) + lane);
        __syncwarp();
        int start, cnt;
        cta_range(*od, c, start, cnt);
        const int tile_first = start / od->nst;
        const int nlt = cnt > 0 ? (start + cnt - 1) / od->nst - tile_first + 1 : 0;
        if (lane < nlt) {
            const int tile = tile_first + lane;
            int mi = 0, first = 0;
            while (mi + 1 < od->count && tile >= od->tile_end[mi]) { first = od->tile_end[mi]; ++mi; }
            const int64_t row0 = (int64_t)(tile - first) * 16;
            TileInfo ti;
            ti.codes = od->codes[mi] + row0 * ((int64_t)od->K * od->bits / 8);
            ti.scales = od->scales[mi] + row0 * od->G;
            ti.biases = od->biases[mi] + row0 * od->G;
            ti.rows_valid = (int)min((int64_t)16, (int64_t)od->N[mi] - row0);
            ti.pad = 0;
            tiles_s[(j & 1) * MAXT + lane] = ti;
        }
        __syncwarp();
    };
    auto prep = [&](const DevOp& o1, const float* acc) {
        if (warp == NW - 1) return;
        const int nth = THREADS - 32;
#define JQ_STREAM_PREP(B, GSZ) \
        if (o1.bits == B && o1.gs == GSZ) prep_limbs<AT, B, GSZ>(o1.x, acc, o1.K, limbs, tab, LS, tid, nth);
        JQ_STREAM_PREP(2, 64) JQ_STREAM_PREP(4, 64) JQ_STREAM_PREP(8, 64)
        JQ_STREAM_PREP(2, 128) JQ_STREAM_PREP(4, 128) JQ_STREAM_PREP(8, 128)
#undef JQ_STREAM_PREP
    };

    for (int i = tid; i < ZERO_BYTES / 4; i += THREADS) reinterpret_cast<uint32_t*>(zero)[i] = 0u;
    for (int i = tid; i < NW * MAXT * 16; i += THREADS) ysum[i] = 0.f;
    if (warp == NW - 1) { build_tables(0); build_tables(1); }
    __syncthreads();

    int slot = 0;
    bool pre = false;
    {   // the warp's first item of op 0, then the limbs of op 0 while it is in flight
        const DevOp& o = ops_s[0];
        int start, cnt;
        cta_range(o, c, start, cnt);
        if (warp < cnt) {
            const int tile_first = start / o.nst;
            const int pos = start - tile_first * o.nst + warp;
            const int lt = pos / o.nst;
            issue_item(ring, tiles_s[lt], pos - lt * o.nst, geo_of(o), lane);
            cp_async_commit();
            pre = true;
        }
        prep(o, nullptr);
    }
    __syncthreads();

    bool aborted = false;
    int prev_rows = 0, prev_region = 0;
    for (int j = 0; j < n_ops; ++j) {
        const DevOp& o = ops_s[j % 3];
        int start, cnt;
        cta_range(o, c, start, cnt);
        const int tile_first = start / o.nst;
        const int nlt = cnt > 0 ? (start + cnt - 1) / o.nst - tile_first + 1 : 0;
        {
            WarpCtx w;
            w.tl = tiles_s + (j & 1) * MAXT;
            w.ge = geo_of(o);
            w.cnt = cnt; w.nst = o.nst; w.stage0 = start - tile_first * o.nst;
            w.next_has = false;
            w.tl1 = w.tl; w.ge1 = w.ge; w.lt1 = 0; w.st1 = 0;
            if (j + 1 < n_ops) {
                const DevOp& o1 = ops_s[(j + 1) % 3];
                int start1, cnt1;
                cta_range(o1, c, start1, cnt1);
                if (warp < cnt1) {
                    const int tf1 = start1 / o1.nst;
                    const int pos1 = start1 - tf1 * o1.nst + warp;
                    w.next_has = true;
                    w.tl1 = tiles_s + ((j + 1) & 1) * MAXT;
                    w.ge1 = geo_of(o1);
                    w.lt1 = pos1 / o1.nst;
                    w.st1 = pos1 - w.lt1 * o1.nst;
                }
            }
#define JQ_STREAM_RUN(B, GSZ) \
            if (o.bits == B && o.gs == GSZ) run_op<AT, B, GSZ, NW>(w, ring, limbs, LS, zero, tab, myy, warp, lane, slot, pre);
            JQ_STREAM_RUN(2, 64) JQ_STREAM_RUN(4, 64) JQ_STREAM_RUN(8, 64)
            JQ_STREAM_RUN(2, 128) JQ_STREAM_RUN(4, 128) JQ_STREAM_RUN(8, 128)
#undef JQ_STREAM_RUN
        }
        __syncthreads();
        // the warps' row sums, added in warp order, go to the op's float32 accumulator
        {
            const TileInfo* tl = tiles_s + (j & 1) * MAXT;
            float* acc = yacc + (size_t)o.region * maxrows + (size_t)tile_first * 16;
            for (int t = tid; t < nlt * 16; t += THREADS) {
                float v = 0.f;
#pragma unroll 4
                for (int ww = 0; ww < NW; ++ww) {
                    v += ysum[(size_t)ww * MAXT * 16 + t];
                    ysum[(size_t)ww * MAXT * 16 + t] = 0.f;
                }
                if ((t & 15) < tl[t >> 4].rows_valid) atomicAdd(acc + t, v);
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            red_release_add(&sync->barrier, 1u);
            const unsigned int target = (unsigned int)(j + 1) * (unsigned int)grid;
            const unsigned long long t0 = now_ns();
            bool ok = !aborted && *reinterpret_cast<volatile unsigned int*>(&sync->abort) == 0u;
            while (ok && ld_acquire(&sync->barrier) < target) {
                __nanosleep(20);
                if (*reinterpret_cast<volatile unsigned int*>(&sync->abort) != 0u) ok = false;
                else if (now_ns() - t0 > WAIT_NS) {
                    ok = false;
                    atomicExch(&sync->abort, 1u);
                    atomicOr(status, JQ_STATUS_LOCAL_WAIT);
                }
            }
            if (!ok) aborted = true;
        }
        __syncthreads();
        // behind the barrier: tables of op j + 2, limbs of op j + 1, output conversion of op j
        const int rows = o.tiles * 16;
        const int gid = c * THREADS + tid;
        float cv = 0.f;
        const float* reg_j = yacc + (size_t)o.region * maxrows;
        if (gid < rows) cv = ld_cg_f32(reg_j + gid);          // requested before the limbs, used after them
        if (warp == NW - 1) build_tables(j + 2);
        if (j + 1 < n_ops) {
            const DevOp& o1 = ops_s[(j + 1) % 3];
            prep(o1, o1.x_acc >= 0 ? reg_j + o1.x_acc : nullptr);
        }
        const bool last = j + 1 == n_ops;
        for (int i = gid; i < rows; i += grid * THREADS) {
            const float v = i == gid ? cv : ld_cg_f32(reg_j + i);
            const int tile = i >> 4;
            int mi = 0, first = 0;
            while (mi + 1 < o.count && tile >= o.tile_end[mi]) { first = o.tile_end[mi]; ++mi; }
            const int row = (tile - first) * 16 + (i & 15);
            if (row < o.N[mi]) o.y[mi][row] = A::from_f32(v);
            if (last) yacc[(size_t)o.region * maxrows + i] = 0.f;
        }
        // the accumulator of op j - 1 is read no more: clear it for op j + 2
        for (int i = gid; i < prev_rows; i += grid * THREADS) yacc[(size_t)prev_region * maxrows + i] = 0.f;
        prev_rows = rows;
        prev_region = o.region;
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(&sync->done, 1u);
        if (old == (unsigned int)grid - 1u) {           // the last CTA to leave re-arms the counters
            sync->barrier = 0u;
            sync->done = 0u;
            __threadfence();
        }
    }
}

static size_t table_bytes(int n_ops) { return ((size_t)n_ops * sizeof(DevOp) + 255) / 256 * 256; }

// Host view of a program: validates the ops and derives what the kernel reads.
struct Plan {
    std::vector<DevOp> dev;
    int kmax = 0, maxrows = 0, nw = 0, grid = 0;
};

static int make_plan(const JqStreamOp* ops, int n_ops, int act_dtype, Plan* out) {
    JQ_REQUIRE(act_dtype == JQ_BF16 || act_dtype == JQ_F16, JQ_EINVAL, "the activation type must be f16 or bf16");
    JQ_REQUIRE(ops && n_ops >= 1 && n_ops <= (1 << 16), JQ_EINVAL, "a program has 1..65536 ops");
    const int grid = sm_count();
    JQ_REQUIRE(grid > 0, JQ_ECUDA, "could not read the number of SMs");
    Plan& p = *out;
    p.grid = grid;
    p.dev.resize(n_ops);
    for (int j = 0; j < n_ops; ++j) {
        const JqStreamOp& s = ops[j];
        DevOp d;
        memset(&d, 0, sizeof(d));
        JQ_REQUIRE(s.count >= 1 && s.count <= MAX_FUSE, JQ_EINVAL, "op %d: 1..%d matrices per op", j, MAX_FUSE);
        JQ_REQUIRE(s.bits == 2 || s.bits == 4 || s.bits == 8, JQ_EUNSUPPORTED, "op %d: the streamed program takes 2-, 4- and 8-bit codes, got %d", j, s.bits);
        JQ_REQUIRE(s.group_size == 64 || s.group_size == 128, JQ_EUNSUPPORTED, "op %d: group size 64 or 128", j);
        JQ_REQUIRE(s.K > 0 && s.K % s.group_size == 0 && s.K < (1 << 24), JQ_EINVAL, "op %d: bad K", j);
        const int G = (int)(s.K / s.group_size);
        JQ_REQUIRE(G % 4 == 0, JQ_EUNSUPPORTED, "op %d: K / group_size must be a multiple of 4", j);
        JQ_REQUIRE(s.x && aligned(s.x, 16), JQ_EINVAL, "op %d: x is null or not 16-byte aligned", j);
        d.x = (const uint16_t*)s.x;
        d.K = (int)s.K; d.G = G; d.bits = s.bits; d.gs = s.group_size; d.count = s.count;
        const int64_t rowbytes = s.K * s.bits / 8;
        d.nst = (int)((rowbytes + ROWB - 1) / ROWB);
        int64_t tiles = 0;
        for (int i = 0; i < s.count; ++i) {
            JQ_REQUIRE(s.N[i] >= 1 && s.N[i] < (1ll << 27), JQ_EINVAL, "op %d: bad row count", j);
            JQ_REQUIRE(s.codes[i] && s.scales[i] && s.biases[i] && s.y[i], JQ_EINVAL, "op %d: null pointer", j);
            JQ_REQUIRE(aligned(s.codes[i], 16) && aligned(s.scales[i], 8) && aligned(s.biases[i], 8) && aligned(s.y[i], 2),
                       JQ_EINVAL, "op %d: codes need 16-byte, scales and biases 8-byte alignment", j);
            d.codes[i] = (const uint8_t*)s.codes[i];
            d.scales[i] = (const uint16_t*)s.scales[i];
            d.biases[i] = (const uint16_t*)s.biases[i];
            d.y[i] = (uint16_t*)s.y[i];
            d.N[i] = (int)s.N[i];
            tiles += (s.N[i] + 15) / 16;
            d.tile_end[i] = (int)tiles;
        }
        JQ_REQUIRE(tiles * d.nst < (1ll << 30), JQ_EUNSUPPORTED, "op %d: too many items", j);
        d.tiles = (int)tiles;
        d.items = (int)(tiles * d.nst);
        if (d.tiles >= grid) {
            d.mode = 0;
            d.q = d.items / grid;
            d.r = d.items % grid;
            d.S = 1;
            const int local = (d.q + 1 + d.nst - 1) / d.nst + 1;       // tiles a run of q + 1 items can touch
            JQ_REQUIRE(local <= MAXT, JQ_EUNSUPPORTED,
                       "op %d: %d rows are too many for one op of a program (a CTA would touch %d row tiles, limit %d): "
                       "split the op by rows", j, d.tiles * 16, local, MAXT);
        } else {
            d.mode = 1;
            d.S = grid / d.tiles >= 2 && d.nst >= 2 ? 2 : 1;           // at most two CTAs per tile: order-free sums
            d.q = d.r = 0;
        }
        d.region = j % 3;
        d.x_acc = -1;
        if (j > 0) {
            // x may be one whole output of the op directly before (read from its accumulator); any other
            // overlap with that op's outputs would be read before it is written
            const DevOp& pv = p.dev[j - 1];
            const char* x0 = (const char*)s.x;
            const char* x1 = x0 + s.K * 2;
            for (int i = 0; i < pv.count; ++i) {
                const char* y0 = (const char*)pv.y[i];
                const char* y1 = y0 + (int64_t)pv.N[i] * 2;
                if (x0 == y0 && pv.N[i] == s.K) {
                    d.x_acc = (i ? pv.tile_end[i - 1] : 0) * 16;
                } else {
                    JQ_REQUIRE(x1 <= y0 || y1 <= x0, JQ_EINVAL,
                               "op %d: x overlaps an output of op %d without being exactly that output", j, j - 1);
                }
            }
        }
        p.kmax = p.kmax > d.K ? p.kmax : d.K;
        p.maxrows = p.maxrows > d.tiles * 16 ? p.maxrows : d.tiles * 16;
        p.dev[j] = d;
    }
    p.nw = 0;
    for (int nw : {16, 12, 8}) {
        if (head_bytes(p.kmax, nw) + (size_t)nw * 2 * SLOT <= (size_t)MAX_SMEM) { p.nw = nw; break; }
    }
    JQ_REQUIRE(p.nw != 0, JQ_EUNSUPPORTED, "K = %d is too long for the streamed program's shared memory", p.kmax);
    return JQ_OK;
}

template <typename AT, int NW>
static int launch(const JqStreamProgram& pg, cudaStream_t st) {
    const size_t smem = head_bytes(pg.kmax, NW) + (size_t)NW * 2 * SLOT;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_stream_kernel<AT, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    int per_sm = 0;
    JQ_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qgemv_stream_kernel<AT, NW>, NW * 32, smem));
    JQ_REQUIRE(per_sm >= 1 && pg.grid <= per_sm * sm_count(), JQ_EUNSUPPORTED,
               "the program's CTAs do not fit the device at once");
    int* status = status_word();
    JQ_REQUIRE(status != nullptr, JQ_ECUDA, "could not locate the device status word");
    char* ws = (char*)pg.workspace;
    Sync* sync = (Sync*)ws;
    const DevOp* ops = (const DevOp*)(ws + sizeof(Sync));
    float* yacc = (float*)(ws + sizeof(Sync) + table_bytes(pg.n_ops));
    int n_ops = pg.n_ops, maxrows = pg.maxrows, kmax = pg.kmax;
    void* args[] = {(void*)&ops, (void*)&n_ops, (void*)&yacc, (void*)&maxrows, (void*)&sync, (void*)&status, (void*)&kmax};
    // the CTAs wait on one another at every op boundary: a cooperative launch guarantees that they are co-resident
    JQ_CUDA_OK(cudaLaunchCooperativeKernel((const void*)qgemv_stream_kernel<AT, NW>, dim3((unsigned)pg.grid), dim3(NW * 32),
                                           args, smem, st));
    return JQ_OK;
}

}  // namespace stream
}  // namespace jq

extern "C" {

size_t jq_qgemv_stream_workspace_bytes(const JqStreamOp* ops, int n_ops) {
    if (!ops || n_ops < 1) return 0;
    int64_t maxrows = 0;
    for (int j = 0; j < n_ops; ++j) {
        int64_t tiles = 0;
        for (int i = 0; i < ops[j].count && i < jq::stream::MAX_FUSE; ++i) tiles += (ops[j].N[i] + 15) / 16;
        maxrows = maxrows > tiles * 16 ? maxrows : tiles * 16;
    }
    return sizeof(jq::stream::Sync) + jq::stream::table_bytes(n_ops) + (size_t)3 * maxrows * sizeof(float);
}

int jq_qgemv_stream_prepare(const JqStreamOp* ops, int n_ops, int act_dtype, void* workspace, size_t workspace_bytes,
                            JqStreamProgram* program, jq_stream_t stream) {
    using namespace jq;
    using namespace jq::stream;
    JQ_REQUIRE(program, JQ_EINVAL, "null program");
    Plan p;
    int rc = make_plan(ops, n_ops, act_dtype, &p);
    if (rc != JQ_OK) return rc;
    const size_t need = sizeof(Sync) + table_bytes(n_ops) + (size_t)3 * p.maxrows * sizeof(float);
    JQ_REQUIRE(workspace && aligned(workspace, 256), JQ_EINVAL, "the workspace must be 256-byte aligned");
    JQ_REQUIRE(workspace_bytes >= need, JQ_EWORKSPACE, "the workspace holds %zu bytes, the program needs %zu",
               workspace_bytes, need);
    cudaStream_t st = (cudaStream_t)stream;
    JQ_CUDA_OK(cudaMemsetAsync(workspace, 0, need, st));
    // pageable source: the call returns once the table has been staged, so `p` may go out of scope
    JQ_CUDA_OK(cudaMemcpyAsync((char*)workspace + sizeof(Sync), p.dev.data(), (size_t)n_ops * sizeof(DevOp),
                               cudaMemcpyHostToDevice, st));
    JQ_CUDA_OK(cudaStreamSynchronize(st));
    program->workspace = workspace;
    program->n_ops = n_ops;
    program->act_dtype = act_dtype;
    program->kmax = p.kmax;
    program->maxrows = p.maxrows;
    program->warps = p.nw;
    program->grid = p.grid;
    return JQ_OK;
}

int jq_qgemv_stream_run(const JqStreamProgram* program, jq_stream_t stream) {
    using namespace jq;
    using namespace jq::stream;
    JQ_REQUIRE(program && program->workspace && program->n_ops >= 1, JQ_EINVAL, "the program was not prepared");
    const JqStreamProgram& pg = *program;
    JQ_REQUIRE(pg.act_dtype == JQ_BF16 || pg.act_dtype == JQ_F16, JQ_EINVAL, "bad activation type");
    cudaStream_t st = (cudaStream_t)stream;
#define JQ_STREAM_LAUNCH(NWV)                                                                              \
    if (pg.warps == NWV)                                                                                   \
        return pg.act_dtype == JQ_BF16 ? launch<__nv_bfloat16, NWV>(pg, st) : launch<__half, NWV>(pg, st);
    JQ_STREAM_LAUNCH(16) JQ_STREAM_LAUNCH(12) JQ_STREAM_LAUNCH(8)
#undef JQ_STREAM_LAUNCH
    return fail(JQ_EINVAL, "the program was not prepared by jq_qgemv_stream_prepare");
}

}  // extern "C"
