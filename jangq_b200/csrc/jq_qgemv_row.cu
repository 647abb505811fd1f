// K2, row-parallel form: decode-shaped quantized mat-vec with the activations shared by the CTA
// and K split over a thread-block cluster.
//
// Bound: HBM bandwidth (same algorithmic bytes as jq_qgemv.cu).
//
// Structure:
//   * a CTA of `nw` warps covers nw*16*MT consecutive weight rows; warp w owns rows
//     [16*MT*w, 16*MT*(w+1)) of it and walks K on its own: private shared-memory stages of
//     16*MT row segments of KT codes plus their scales/biases, all moved by per-lane
//     cp.async (16-byte chunks for codes, 8-byte quads for the sidecars), `nbuf` stages
//     deep, so a warp never waits on another warp inside the K loop and the sidecars are
//     prefetched as far ahead as the codes;
//   * the activations of the CTA's K slice are copied to shared memory once, and the group
//     sums X[group][m] the dequantization offset needs are computed once per CTA, instead
//     of once per warp and stage;
//   * a cluster of `ksplit` CTAs shares a block of rows and splits K into contiguous slices;
//     partial sums meet in the shared memory of cluster rank 0 (distributed shared memory),
//     which writes y.  Short-and-wide matrices fill the machine this way without atomics
//     and without a second pass;
//   * the inner loop (register dequantization into m16n8k16 A operands, activations as the
//     B operand) is gemv_stage_blocks() of jq_qgemv.cuh.
// Weights are prefetched before griddepcontrol.wait, activations after it, so that under
// programmatic dependent launch a mat-vec streams its first stages while its predecessor drains.
#include <cstdlib>

#include "jq_mma.cuh"
#include "jq_qgemv.cuh"

namespace jq {

constexpr int ROW_MAX_NBUF = 4;
constexpr int ROW_SMEM_LIMIT = 200 * 1024;

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

__host__ __device__ constexpr int up128(int v) { return (v + 127) / 128 * 128; }

// Compile-time geometry of a warp's stage and the CTA's shared-memory map.
template <int BITS, int GS, int MT> struct RowGeom {
    static constexpr int KT = (BITS <= 4 || GS == 128) ? 512 : 256;   // codes per row and stage
    static constexpr int ROWS = 16 * MT;                              // rows per warp
    static constexpr int PAD = BITS == 2 ? 4 : BITS == 6 ? 12 : BITS == 8 ? 16 : 8;   // bank-conflict-free units
    static constexpr int RS = KT * BITS / 32 + PAD;      // code row stride, words
    static constexpr int NG = KT / GS;                   // groups per stage (4 or 8)
    static constexpr int NQ = NG / 4;                    // 8-byte sidecar quads per row
    static constexpr int NGP = NG + 1;                   // padded row stride of the f32 table, float2
    static constexpr int RAW_S = ROWS * RS * 4;          // raw scales [ROWS][NG] (16-bit)
    static constexpr int RAW_B = RAW_S + ROWS * NG * 2;  // raw biases [ROWS][NG]
    static constexpr int STAGE = up128(RAW_B + ROWS * NG * 2);
    static constexpr int TABLE = up128(ROWS * NGP * 8);  // float2 (s*POST, b - OFFSET*s), one per warp
    __host__ __device__ static constexpr int warp_bytes(int nbuf) { return TABLE + nbuf * STAGE; }
    // CTA map: [zero chunk 128][red: nw*ROWS*8 f32][Xs: sl*NG*8 f32][x: M rows of sl*KT+8][warp areas]
    __host__ __device__ static constexpr int red_bytes(int nw) { return nw * ROWS * 8 * 4; }
    __host__ __device__ static constexpr int xs_bytes(int sl) { return sl * NG * 8 * 4; }
    __host__ __device__ static constexpr int x_bytes(int sl, int M) { return up128(M * (sl * KT + 8) * 2); }
    __host__ __device__ static constexpr int total(int nw, int sl, int M, int nbuf) {
        return 128 + red_bytes(nw) + xs_bytes(sl) + x_bytes(sl, M) + nw * warp_bytes(nbuf);
    }
};

template <typename AT, int BITS, int GS, int MT>
__global__ void __launch_bounds__(256)
qgemv_row_kernel(const GemvArgs a) {
    using A = Act<AT>;
    using F = Fields<AT, BITS>;
    using Geo = RowGeom<BITS, GS, MT>;
    constexpr int ROWS = Geo::ROWS, KT = Geo::KT, RS = Geo::RS, NG = Geo::NG, NQ = Geo::NQ, NGP = Geo::NGP;

    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x, nthr = blockDim.x, nw = nthr >> 5;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int S = a.ksplit;
    const int rb = blockIdx.x / S;          // block of nw*ROWS rows
    const int cr = blockIdx.x - rb * S;     // rank in the cluster (cluster shape is (S,1,1))
    const int K = (int)a.K, G = a.G, M = a.M, nbuf = a.nbuf;
    const int nst = (K + KT - 1) / KT;
    const int sl = (nst + S - 1) / S;       // longest slice, stages
    const int st_begin = (int)((int64_t)cr * nst / S), st_end = (int)((int64_t)(cr + 1) * nst / S);
    const int k_begin = st_begin * KT, k_end = min(K, st_end * KT);
    const int XSL = sl * KT + 8;            // activation row stride in shared memory, elements
    const int64_t rowbytes = a.K * BITS / 8;

    const uint16_t* xs16 = reinterpret_cast<const uint16_t*>(a.x);
    const uint16_t* sc16 = reinterpret_cast<const uint16_t*>(a.scales);
    const uint16_t* bi16 = reinterpret_cast<const uint16_t*>(a.biases);
    const uint32_t* codes_g = a.codes;
    uint16_t* y16 = reinterpret_cast<uint16_t*>(a.y);
    if (a.pair_expert) {
        const int p = blockIdx.y;           // the same for every CTA of a cluster: they leave together
        const int e = a.pair_expert[p];
        if (e < 0 || e >= a.num_experts) return;                      // expert of another rank
        if (a.bits_tab && a.bits_tab[e] != BITS) return;              // handled by the launch of its own width
        codes_g = a.codes_tab[e];
        sc16 = reinterpret_cast<const uint16_t*>(a.scales_tab[e]);
        bi16 = reinterpret_cast<const uint16_t*>(a.biases_tab[e]);
        xs16 += (int64_t)(p / a.x_div) * a.ldx;
        y16 += (int64_t)p * a.ldy;
    }

    uint8_t* zero = smem;
    float* red = reinterpret_cast<float*>(smem + 128);
    float* Xs = reinterpret_cast<float*>(smem + 128 + Geo::red_bytes(nw));
    uint16_t* xsh = reinterpret_cast<uint16_t*>(smem + 128 + Geo::red_bytes(nw) + Geo::xs_bytes(sl));
    uint8_t* wbase = smem + 128 + Geo::red_bytes(nw) + Geo::xs_bytes(sl) + Geo::x_bytes(sl, M) +
                     (size_t)warp * Geo::warp_bytes(nbuf);
    float2* table = reinterpret_cast<float2*>(wbase);
    uint8_t* stages = wbase + Geo::TABLE;

    const int64_t cta_row0 = (int64_t)rb * nw * ROWS;
    const int64_t n0 = cta_row0 + (int64_t)warp * ROWS;
    const int rows_valid = (int)max((int64_t)0, min((int64_t)ROWS, a.N - n0));

    // ---- one stage of this warp: codes (16 bytes per lane and copy) + sidecar quads (8 bytes) ----------
    const uint8_t* code_base = reinterpret_cast<const uint8_t*>(codes_g) + n0 * rowbytes;
    constexpr int SCP = (ROWS * NQ + 31) / 32;
    auto issue_stage = [&](int st, int slot) {
        if (st < st_end && rows_valid > 0) {
            const int k0 = st * KT;
            const int kc = min(KT, K - k0);
            uint8_t* buf = stages + (size_t)slot * Geo::STAGE;
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
#pragma unroll
            for (int i = 0; i < SCP; ++i) {
                const int pr = lane + 32 * i;
                const int row = pr / NQ, quad = pr % NQ;
                const int grp = st * NG + quad * 4;
                if (pr < ROWS * NQ && grp < G) {
                    const int64_t off = min(n0 + row, a.N - 1) * G + grp;
                    cp_async8(buf + Geo::RAW_S + (row * NG + quad * 4) * 2, sc16 + off);
                    cp_async8(buf + Geo::RAW_B + (row * NG + quad * 4) * 2, bi16 + off);
                }
            }
        }
    };

    // Weights first: they are static by contract, so under programmatic dependent launch they
    // stream while the predecessor still runs; the activations only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
    for (int i = 0; i < ROW_MAX_NBUF; ++i)
        if (i < nbuf) {
            issue_stage(st_begin + i, i);
            cp_async_commit();
        }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const int cpx = (k_end - k_begin) / 8;                         // 16-byte chunks per activation row
        for (int m = 0; m < M; ++m)
            for (int c = tid; c < cpx; c += nthr)
                cp_async16(xsh + (size_t)m * XSL + c * 8, xs16 + (int64_t)m * a.ldx + k_begin + c * 8);
        cp_async_commit();
    }
    if (tid < 8) reinterpret_cast<uint32_t*>(zero)[tid] = 0u;
    cp_async_wait<0>();
    __syncthreads();

    // ---- X[group][m] = sum of the group's activations, once per CTA -------------------------------------
    {
        const int cpm = (k_end - k_begin) / 16;                        // 16-element chunks per row (multiple of 16)
        const int total = M * cpm;
        for (int t0 = 0; t0 < total; t0 += nthr) {
            const int t = t0 + tid;
            const int m = t / cpm, chunk = t - m * cpm;
            float sum = 0.f;
            if (t < total) {
                const uint4* xp = reinterpret_cast<const uint4*>(xsh + (size_t)m * XSL + chunk * 16);
                const uint4 v0 = xp[0], v1 = xp[1];
                const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) { s0 += A::lo_f32(w[j]); s1 += A::hi_f32(w[j]); }
                sum = s0 + s1;
            }
#pragma unroll
            for (int d = 1; d < GS / 16; d <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
            if (t < total && (chunk & (GS / 16 - 1)) == 0) Xs[(chunk * 16 / GS) * 8 + m] = sum;
        }
    }
    __syncthreads();

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

    if (rows_valid > 0) {
        int it = 0;
        for (int st = st_begin; st < st_end; ++st, ++it) {
            const int slot = it % nbuf;
            const int kc = min(KT, K - st * KT);
            uint8_t* buf = stages + (size_t)slot * Geo::STAGE;
            if (nbuf == 2) cp_async_wait<1>(); else if (nbuf == 3) cp_async_wait<2>(); else cp_async_wait<3>();
            __syncwarp();
            // raw 16-bit sidecars -> f32 pairs (s*POST, b - OFFSET*s), each (row, quad) by one lane
#pragma unroll
            for (int i = 0; i < SCP; ++i) {
                const int pr = lane + 32 * i;
                const int row = pr / NQ, quad = pr % NQ;
                if (pr < ROWS * NQ) {
                    const uint2 sv = *reinterpret_cast<const uint2*>(buf + Geo::RAW_S + (row * NG + quad * 4) * 2);
                    const uint2 bv = *reinterpret_cast<const uint2*>(buf + Geo::RAW_B + (row * NG + quad * 4) * 2);
                    float2* dst = table + row * NGP + quad * 4;
                    const float s0 = A::lo_f32(sv.x), s1 = A::hi_f32(sv.x), s2 = A::lo_f32(sv.y), s3 = A::hi_f32(sv.y);
                    dst[0] = make_float2(s0 * F::POST, fmaf(-F::OFFSET, s0, A::lo_f32(bv.x)));
                    dst[1] = make_float2(s1 * F::POST, fmaf(-F::OFFSET, s1, A::hi_f32(bv.x)));
                    dst[2] = make_float2(s2 * F::POST, fmaf(-F::OFFSET, s2, A::lo_f32(bv.y)));
                    dst[3] = make_float2(s3 * F::POST, fmaf(-F::OFFSET, s3, A::hi_f32(bv.y)));
                }
            }
            __syncwarp();
            const uint32_t* c_lo = reinterpret_cast<const uint32_t*>(buf) + g * RS;
            const uint16_t* xrow = (g < M) ? xsh + (size_t)g * XSL + (st - st_begin) * KT + tig * 16
                                           : reinterpret_cast<const uint16_t*>(zero);
            const int xstep = (g < M) ? 64 : 0;
            gemv_stage_blocks<AT, BITS, GS, MT>(c_lo, RS, xrow, xstep, table + g * NGP, NGP,
                                                Xs + (st - st_begin) * NG * 8 + 2 * tig, kc >> 6, tig, acc);
            __syncwarp();
            issue_stage(st + nbuf, slot);
            cp_async_commit();     // one group per iteration keeps the group count uniform
        }
    }
    cp_async_wait<0>();

    if (S == 1) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = mt * 16 + g + ((i & 2) ? 8 : 0), m = 2 * tig + (i & 1);
                if (row < rows_valid && m < M) y16[(int64_t)m * a.ldy + n0 + row] = A::from_f32(acc[mt][i]);
            }
        return;
    }

    // ---- split K: partial sums meet in rank 0's view of every rank's shared memory ---------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = mt * 16 + g + ((i & 2) ? 8 : 0), m = 2 * tig + (i & 1);
            red[(warp * ROWS + row) * 8 + m] = acc[mt][i];
        }
    cluster_sync_all();
    if (cr == 0) {
        const int rows_cta = nw * ROWS;
        for (int idx = tid; idx < rows_cta * M; idx += nthr) {
            const int m = idx / rows_cta, r = idx - m * rows_cta;
            float v = red[r * 8 + m];
            for (int s = 1; s < S; ++s) v += ld_cluster_f32(red + r * 8 + m, (uint32_t)s);
            if (cta_row0 + r < a.N) y16[(int64_t)m * a.ldy + cta_row0 + r] = A::from_f32(v);
        }
    }
    cluster_sync_all();    // peers keep their shared memory alive until rank 0 has read it
}

static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return (e && e[0] >= '0' && e[0] <= '9') ? atoi(e) : dflt;
}

template <typename AT, int BITS, int GS, int MT>
static int launch_row_cfg(GemvArgs a, int pairs, int nw, int S, int nbuf, cudaStream_t st, bool* launched) {
    using Geo = RowGeom<BITS, GS, MT>;
    const int nst = (int)((a.K + Geo::KT - 1) / Geo::KT);
    const int sl = (nst + S - 1) / S;
    const int smem = Geo::total(nw, sl, a.M, nbuf);
    if (smem > ROW_SMEM_LIMIT) return JQ_OK;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_row_kernel<AT, BITS, GS, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ROW_SMEM_LIMIT));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    a.nbuf = nbuf;
    a.ksplit = S;
    const int rows_cta = nw * 16 * MT;
    const unsigned row_blocks = (unsigned)((a.N + rows_cta - 1) / rows_cta);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(row_blocks * (unsigned)S, (unsigned)pairs);
    cfg.blockDim = dim3(nw * 32);
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
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemv_row_kernel<AT, BITS, GS, MT>, a));
    *launched = true;
    return JQ_OK;
}

// Shape heuristics: warps per CTA, rows per warp, cluster size and pipeline depth.
//   * the grid should put at least ~2 CTAs on every SM; when the row blocks alone do not, K is split
//     over a cluster (2, 4 or 8 CTAs) as long as every slice keeps at least two stages;
//   * 32 rows per warp (MT=2) halve the activation-operand work per weight and pay once the
//     16-row tiles alone oversubscribe the machine;
//   * the pipeline is as deep as the slice is long, up to 4 stages, while shared memory allows
//     two CTAs per SM.
template <typename AT, int BITS, int GS>
static int launch_row(const GemvArgs& a, int pairs, cudaStream_t st, bool* launched) {
    const int sms = sm_count();
    constexpr int KT = RowGeom<BITS, GS, 1>::KT;
    const int nst = (int)((a.K + KT - 1) / KT);
    const int64_t tiles16 = (a.N + 15) / 16 * pairs;
    int mt = env_int("JANGQ_ROW_MT", tiles16 >= (int64_t)16 * sms ? 2 : 1);
    int nw = env_int("JANGQ_ROW_NW", 4);
    if (mt != 2) mt = 1;
    if (nw != 8) nw = 4;
    const int64_t row_blocks = ((a.N + nw * 16 * mt - 1) / (nw * 16 * mt)) * pairs;
    int S = 1;
    while (S < 8 && row_blocks * S < (int64_t)2 * sms && nst / (2 * S) >= 2) S *= 2;
    S = env_int("JANGQ_ROW_S", S);
    if (S != 1 && S != 2 && S != 4 && S != 8) S = 1;
    if (S > nst) return JQ_OK;
    int sl = (nst + S - 1) / S;
    int nbuf = sl < 2 ? 2 : sl > ROW_MAX_NBUF ? ROW_MAX_NBUF : sl;
    auto total = [&](int s_, int nb) {
        const int l = (nst + s_ - 1) / s_;
        return mt == 2 ? RowGeom<BITS, GS, 2>::total(nw, l, a.M, nb) : RowGeom<BITS, GS, 1>::total(nw, l, a.M, nb);
    };
    while (nbuf > 2 && total(S, nbuf) > 100 * 1024) --nbuf;            // keep two CTAs per SM
    while (total(S, nbuf) > ROW_SMEM_LIMIT && S < 8 && 2 * S <= nst) S *= 2;   // long rows, many activation rows
    nbuf = env_int("JANGQ_ROW_NBUF", nbuf);
    if (nbuf < 2 || nbuf > ROW_MAX_NBUF) nbuf = 2;
    if (mt == 2) return launch_row_cfg<AT, BITS, GS, 2>(a, pairs, nw, S, nbuf, st, launched);
    return launch_row_cfg<AT, BITS, GS, 1>(a, pairs, nw, S, nbuf, st, launched);
}

int launch_row_kernel(const GemvArgs& a, int act_dtype, int bits, int gs, int pairs, cudaStream_t st, bool* launched) {
    *launched = false;
    int rc = JQ_OK;
#define JQ_ROW_CASE(B, GSZ)                                                                        \
    if (bits == B && gs == GSZ) {                                                                  \
        rc = (act_dtype == JQ_BF16) ? launch_row<__nv_bfloat16, B, GSZ>(a, pairs, st, launched)    \
                                    : launch_row<__half, B, GSZ>(a, pairs, st, launched);          \
    }
    JQ_ROW_CASE(2, 64) JQ_ROW_CASE(3, 64) JQ_ROW_CASE(4, 64) JQ_ROW_CASE(6, 64) JQ_ROW_CASE(8, 64)
    JQ_ROW_CASE(2, 128) JQ_ROW_CASE(3, 128) JQ_ROW_CASE(4, 128) JQ_ROW_CASE(6, 128) JQ_ROW_CASE(8, 128)
#undef JQ_ROW_CASE
    return rc;
}

}  // namespace jq
