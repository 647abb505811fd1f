// K2, item-streaming integer warp-MMA form, one op per launch: decode-shaped quantized mat-vec
//     y[N] = deq(W)[N, K] . x[K]        (one activation row; 2-, 4-, 6- and 8-bit codes)
// for up to four matrices that share x (q/k/v, gate/up) in one launch.
//
// Bound: HBM bandwidth on paper (algorithmic bytes per launch = N*K*bits/8 + N*(K/gs)*4 + 2*K + 2*N); in
// practice the instruction issue rate for narrow codes, so the kernel is written against an instruction
// budget: a warp spends about 27 instructions on a 16-row x 64-code block, about 80 on requesting an item
// and about 80 on the bookkeeping of an item, and an item is 16 rows x 256 bytes of codes (16 blocks of
// 2-bit codes), where the kernel this one replaces for one activation row spent its per-item cost on 8.
//
// Structure: one CTA per SM (NW warps), each CTA owns a contiguous run of 16-row tiles and its warps walk
// the run's (tile, K stage) items round-robin through two private cp.async slots each
// (jq_stream_dev.cuh).  Weights first: under programmatic dependent launch the first two items of every
// warp are requested before griddepcontrol.wait, the activations are read and cut into limbs after it.  The
// warps' row sums meet in shared memory and are stored in the activation type.
#include "jq_qgemv.cuh"
#include "jq_stream_dev.cuh"

namespace jq {

namespace one {

using namespace stream;

__host__ __device__ inline size_t one_head_bytes(int K, int nw, int bits = 8) {
    const size_t limbs = ((size_t)3 * limb_stride_bits(K, bits) + 127) / 128 * 128;
    return HEAD0 + MAXT * sizeof(TileInfo) + 128 + (size_t)(K / 64) * 16 + limbs + (size_t)nw * MAXT * 16 * sizeof(float);
}

template <typename AT, int BITS, int GS, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
qgemv_one_kernel(const GemvArgs a, const GemvBatch bt) {
    using A = Act<AT>;
    constexpr int THREADS = NW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = (int)a.K, G = a.G, TPC = a.ksplit;          // ksplit: 16-row tiles per CTA in this kernel
    const int LS = limb_stride_bits(K, BITS);
    constexpr int RB = rowb_of(BITS);
    const int rowbytes = K * BITS / 8;
    const int nst = (rowbytes + RB - 1) / RB;

    uint8_t* zero = smem;
    TileInfo* tiles = reinterpret_cast<TileInfo*>(smem + HEAD0);                        // [MAXT]
    float* part = reinterpret_cast<float*>(tiles + MAXT);                               // [32] sums of squares per warp
    float2* tab = reinterpret_cast<float2*>(part + 32);                                 // [K / 64][2]
    uint8_t* limbs = reinterpret_cast<uint8_t*>(tab) + (size_t)(K / 64) * 16;           // [3][LS]
    float* ysum = reinterpret_cast<float*>(limbs + ((size_t)3 * LS + 127) / 128 * 128);  // [NW][MAXT * 16]
    uint8_t* ring = smem + one_head_bytes(K, NW, BITS) + (size_t)warp * 2 * SLOT;
    float* myy = ysum + (size_t)warp * MAXT * 16;

    // tiles of all matrices of the launch are numbered consecutively; blk_end[i] = first tile after matrix i
    const int tile0 = (int)blockIdx.x * TPC;
    const int ntile = min(TPC, bt.blk_end[bt.count - 1] - tile0);
    if (tid < ntile) {
        const int gt = tile0 + tid;
        int mi = 0, first = 0;
        while (mi + 1 < bt.count && gt >= bt.blk_end[mi]) { first = bt.blk_end[mi]; ++mi; }
        const int64_t row0 = (int64_t)(gt - first) * 16;
        TileInfo ti;
        ti.codes = reinterpret_cast<const uint8_t*>(bt.codes[mi]) + row0 * rowbytes;
        ti.scales = reinterpret_cast<const uint16_t*>(bt.scales[mi]) + row0 * G;
        ti.biases = reinterpret_cast<const uint16_t*>(bt.biases[mi]) + row0 * G;
        ti.rows_valid = (int)min((int64_t)16, bt.N[mi] - row0);
        ti.xsel = 0;
        tiles[tid] = ti;
    }
    for (int i = tid; i < ZERO_BYTES / 4; i += THREADS) reinterpret_cast<uint32_t*>(zero)[i] = 0u;
    for (int i = lane; i < ntile * 16; i += 32) myy[i] = 0.f;          // each warp clears the row sums it will use
    __syncthreads();

    OpGeo ge;
    ge.rowbytes = rowbytes; ge.G = G; ge.rowb = RB; ge.rsb = rsb_of(BITS);
    ge.grpb = BITS * GS / 8; ge.ngb = 2 * (RB / (BITS * GS / 8)); ge.bits = BITS; ge.gs = GS;
    const int cnt = ntile * nst;

    // Weights first (static by contract): under programmatic dependent launch they stream while the
    // predecessor still runs; the activations are touched only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int slot = 0, npre = 0;
    auto request = [&](int k) {
        const int pos = warp + k * NW;
        if (pos < cnt) {
            const int lt = pos / nst;
            issue_item(ring + k * SLOT, tiles[lt], pos - lt * nst, ge, lane);
            cp_async_commit();
            npre = k + 1;
        }
    };
    // One item per warp goes out before the dependency wait; the activations are requested right behind the
    // wait, ahead of the warp's second item: measured on a chain of launches, an activation load issued
    // behind two items per warp of every SM queues behind about 20 MB of weight traffic, and the limbs are
    // on the critical path of the CTAs that start last.
    request(0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint16_t* xs = reinterpret_cast<const uint16_t*>(a.x);
    PrepSrc src;
    src.xs = xs; src.have_pre = true;
    if (a.norm_res == nullptr) {
        src.pre = tid < K / 8 ? ld_cg16(xs + (size_t)tid * 8) : make_uint4(0u, 0u, 0u, 0u);
        request(1);
    } else {
        // The row is rms_norm(res + sum_j y[j]) (K <= 8 * THREADS: a thread holds its 8 columns in registers
        // from the loads to the limbs).  Every CTA forms the whole row -- (k + 1) * 2 K bytes out of L2 -- which
        // costs less than the launch it replaces; CTA 0 stores the row for whoever needs it next.
        const uint16_t* res = reinterpret_cast<const uint16_t*>(a.norm_res);
        const uint16_t* ys = reinterpret_cast<const uint16_t*>(a.norm_y);
        const bool mine = tid < K / 8;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        if (mine) {
            const uint4 r0 = ld_cg16(res + (size_t)tid * 8);
            const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] = A::lo_f32(w0[j]); v[2 * j + 1] = A::hi_f32(w0[j]); }
            for (int j0 = 0; j0 < a.norm_k; j0 += 4) {           // four rows' loads in flight at a time
                uint4 rr[4];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    rr[q] = j0 + q < a.norm_k ? ld_cg16(ys + (size_t)(j0 + q) * a.norm_ldy + (size_t)tid * 8)
                                              : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int q = 0; q < 4; ++q) {                     // slot order; rows past k add +0
                    const uint32_t wq[4] = {rr[q].x, rr[q].y, rr[q].z, rr[q].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) { v[2 * j] += A::lo_f32(wq[j]); v[2 * j + 1] += A::hi_f32(wq[j]); }
                }
            }
        }
        request(1);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < NW; ++i) tot += part[i];
        const float rn = rsqrtf(tot / (float)K + a.norm_eps);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = (uint32_t)A::from_f32(v[2 * j] * rn) | ((uint32_t)A::from_f32(v[2 * j + 1] * rn) << 16);
        src.pre = make_uint4(o[0], o[1], o[2], o[3]);
        if (blockIdx.x == 0 && mine)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(const_cast<void*>(a.x)) + (size_t)tid * 8) = src.pre;
    }
    prep_limbs<AT, BITS, GS>(src, K, limbs, tab, LS, 0, tid, THREADS);
    __syncthreads();

    WarpCtx w;
    w.tl = tiles; w.ge = ge; w.cnt = cnt; w.nst = nst; w.stage0 = 0;
    w.tl1 = tiles; w.ge1 = ge; w.lt1 = w.st1 = w.lt1b = w.st1b = 0; w.next_n = 0;
    run_op<AT, BITS, GS, NW>(w, ring, limbs, LS, zero, tab, myy, warp, lane, slot, npre);
    cp_async_wait<0>();
    __syncthreads();

    for (int t = tid; t < ntile * 16; t += THREADS) {
        float part[NW];
#pragma unroll
        for (int ww = 0; ww < NW; ++ww) part[ww] = ysum[(size_t)ww * MAXT * 16 + t];
        float v = 0.f;
#pragma unroll
        for (int ww = 0; ww < NW; ++ww) v += part[ww];             // always in warp order
        if ((t & 15) < tiles[t >> 4].rows_valid) {
            const int gt = tile0 + (t >> 4);
            int mi = 0, first = 0;
            while (mi + 1 < bt.count && gt >= bt.blk_end[mi]) { first = bt.blk_end[mi]; ++mi; }
            reinterpret_cast<uint16_t*>(bt.y[mi])[(int64_t)(gt - first) * 16 + (t & 15)] = A::from_f32(v);
        }
    }
}

template <typename AT, int BITS, int GS, int NW>
static int launch_cfg(GemvArgs a, const GemvBatch& bt, int tpc, int grid, cudaStream_t st, bool* launched) {
    const size_t smem = one_head_bytes((int)a.K, NW, BITS) + (size_t)NW * 2 * SLOT;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(qgemv_one_kernel<AT, BITS, GS, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        MAX_SMEM));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    a.ksplit = tpc;
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
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, qgemv_one_kernel<AT, BITS, GS, NW>, a, bt));
    *launched = true;
    return JQ_OK;
}

// One CTA per SM; every CTA gets the same number of 16-row tiles (the last one the remainder).  The warp
// count is the largest whose rings fit the shared memory next to the limbs of a K-long activation row.
template <typename AT, int BITS, int GS>
static int launch_shape(const GemvArgs& a, GemvBatch bt, cudaStream_t st, bool* launched) {
    const int sms = sm_count();
    int64_t tiles = 0;
    for (int i = 0; i < bt.count; ++i) {
        tiles += (bt.N[i] + 15) / 16;
        bt.blk_end[i] = (int)tiles;
    }
    const int tpc = (int)((tiles + sms - 1) / sms);
    const int grid = (int)((tiles + tpc - 1) / tpc);
    if (tpc > MAXT) return JQ_OK;                                 // too many rows for one launch of this kernel
    for (int nw : {16, 12, 8}) {
        if (one_head_bytes((int)a.K, nw, BITS) + (size_t)nw * 2 * SLOT > (size_t)MAX_SMEM) continue;
        if (a.norm_res != nullptr && a.K > 8 * 32 * nw) return JQ_OK;     // the row must fit the CTA's registers
        if (nw == 16) return launch_cfg<AT, BITS, GS, 16>(a, bt, tpc, grid, st, launched);
        if (nw == 12) return launch_cfg<AT, BITS, GS, 12>(a, bt, tpc, grid, st, launched);
        return launch_cfg<AT, BITS, GS, 8>(a, bt, tpc, grid, st, launched);
    }
    return JQ_OK;                                                 // K too long: another kernel
}

// ---- routed-expert gather for one token (decode): every (token, slot) pair multiplies its own expert ---------
// One launch covers `banks` x `pairs` matrices of N x K (gate and up of the k routed experts, or their down
// projections).  Pair p uses expert pair_expert[p] - expert_base of the bank's pointer tables; pairs whose
// expert belongs to another rank get zero rows.  Activations: one shared row (gate/up of one token), one row
// per pair (down), or -- SWIGLU -- one row per pair formed on the fly as silu(g) * u * weight from the gate
// and up products, so that the separate SwiGLU launch between the two gathers disappears.
struct GatherArgs {
    const void* x;                    // activation rows, or the gate products when `up` is set
    const void* up;                   // SwiGLU source: up products [pairs, K]; nullptr otherwise
    const float* wts;                 // SwiGLU source: routing weight per pair (nullptr: 1)
    const int32_t* pair_expert;
    const uint32_t* const* codes_tab[2];
    const void* const* scales_tab[2];
    const void* const* biases_tab[2];
    void* y[2];
    int64_t ldx, ldy;
    float limit;
    int pairs, banks, num_experts, expert_base;
    int N, K, G;
    int x_div;                        // pair p reads activation row p / x_div (pairs: one shared row; 1: a row per pair)
    int tpc;                          // 16-row tiles per CTA
};

// The per-expert pointer tables are static: up to GATHER_TAB_EXPERTS experts' entries are copied into shared memory
// before the dependency wait, which takes one dependent round trip to memory (expert id -> pointer) off the path
// between the routing decision and the first weight bytes.
constexpr int GATHER_TAB_EXPERTS = 128;
constexpr size_t GATHER_TAB_BYTES = (size_t)2 * 3 * GATHER_TAB_EXPERTS * sizeof(void*);

__host__ __device__ inline size_t gather_head_bytes(int K, int nx, int nw, int bits = 8) {
    const size_t limbs = ((size_t)nx * 3 * limb_stride_bits(K, bits) + 127) / 128 * 128;
    return HEAD0 + MAXT * sizeof(TileInfo) + MAXT * sizeof(void*) + 16 + GATHER_TAB_BYTES + (size_t)nx * (K / 64) * 16 +
           limbs + (size_t)nw * MAXT * 16 * sizeof(float);
}

template <typename AT, int BITS, int GS, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
gather_one_kernel(const GatherArgs a) {
    using A = Act<AT>;
    constexpr int THREADS = NW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = a.K, G = a.G, N = a.N;
    const int LS = limb_stride_bits(K, BITS);
    constexpr int RB = rowb_of(BITS);
    const int rowbytes = K * BITS / 8;
    const int nst = (rowbytes + RB - 1) / RB;
    const int nx = (a.pairs + a.x_div - 1) / a.x_div;
    const int tpm = (N + 15) / 16;                                   // tiles per matrix
    const int total = a.banks * a.pairs * tpm;

    uint8_t* zero = smem;
    TileInfo* tiles = reinterpret_cast<TileInfo*>(smem + HEAD0);                          // [MAXT], live tiles only
    uint16_t** ytile = reinterpret_cast<uint16_t**>(tiles + MAXT);                        // [MAXT] first output of the tile
    int* nlive_s = reinterpret_cast<int*>(ytile + MAXT);
    const void** ptab = reinterpret_cast<const void**>(reinterpret_cast<uint8_t*>(ytile + MAXT) + 16);   // [2][3][128]
    float2* tab = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(ptab) + GATHER_TAB_BYTES);       // [nx][K / 64][2]
    uint8_t* limbs = reinterpret_cast<uint8_t*>(tab) + (size_t)nx * (K / 64) * 16;         // [nx][3][LS]
    float* ysum = reinterpret_cast<float*>(limbs + ((size_t)nx * 3 * LS + 127) / 128 * 128);
    uint8_t* ring = smem + gather_head_bytes(K, nx, NW, BITS) + (size_t)warp * 2 * SLOT;
    float* myy = ysum + (size_t)warp * MAXT * 16;

    for (int i = tid; i < ZERO_BYTES / 4; i += THREADS) reinterpret_cast<uint32_t*>(zero)[i] = 0u;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // the routing decision comes from the launch before: no weights can be requested ahead of it, but the pointer
    // tables can be read
    const bool tab_cached = a.num_experts <= GATHER_TAB_EXPERTS;
    if (tab_cached) {
        for (int i = tid; i < a.banks * 3 * a.num_experts; i += THREADS) {
            const int b = i / (3 * a.num_experts), r = i - b * 3 * a.num_experts;
            const int which = r / a.num_experts, e = r - which * a.num_experts;
            const void* v = which == 0 ? (const void*)a.codes_tab[b][e] : which == 1 ? a.scales_tab[b][e] : a.biases_tab[b][e];
            ptab[(b * 3 + which) * GATHER_TAB_EXPERTS + e] = v;
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();

    const int tile0 = (int)blockIdx.x * a.tpc;
    const int ntile = min(a.tpc, total - tile0);
    if (warp == 0) {
        bool live = false;
        TileInfo ti = {};
        uint16_t* yp = nullptr;
        if (lane < ntile) {
            const int gt = tile0 + lane;
            const int j = gt / tpm, tm = gt - j * tpm;               // matrix (bank-major), tile inside it
            const int b = j / a.pairs, p = j - b * a.pairs;
            const int e = a.pair_expert[p] - a.expert_base;
            const int row0 = tm * 16;
            const int rows_valid = min(16, N - row0);
            yp = reinterpret_cast<uint16_t*>(a.y[b]) + (int64_t)p * a.ldy + row0;
            if (e >= 0 && e < a.num_experts) {
                live = true;
                const void* pc = tab_cached ? ptab[(b * 3 + 0) * GATHER_TAB_EXPERTS + e] : (const void*)a.codes_tab[b][e];
                const void* ps = tab_cached ? ptab[(b * 3 + 1) * GATHER_TAB_EXPERTS + e] : a.scales_tab[b][e];
                const void* pb = tab_cached ? ptab[(b * 3 + 2) * GATHER_TAB_EXPERTS + e] : a.biases_tab[b][e];
                ti.codes = reinterpret_cast<const uint8_t*>(pc) + (int64_t)row0 * rowbytes;
                ti.scales = reinterpret_cast<const uint16_t*>(ps) + (int64_t)row0 * G;
                ti.biases = reinterpret_cast<const uint16_t*>(pb) + (int64_t)row0 * G;
                ti.rows_valid = rows_valid;
                ti.xsel = p / a.x_div;
            } else {
                for (int r = 0; r < rows_valid; ++r) yp[r] = 0;     // an expert of another rank: zero rows
            }
        }
        const unsigned mask = __ballot_sync(0xFFFFFFFFu, live);
        if (live) {
            const int pos = __popc(mask & ((1u << lane) - 1u));
            tiles[pos] = ti;
            ytile[pos] = yp;
        }
        if (lane == 0) *nlive_s = __popc(mask);
    }
    __syncthreads();
    const int nlive = *nlive_s;
    for (int i = lane; i < nlive * 16; i += 32) myy[i] = 0.f;

    OpGeo ge;
    ge.rowbytes = rowbytes; ge.G = G; ge.rowb = RB; ge.rsb = rsb_of(BITS);
    ge.grpb = BITS * GS / 8; ge.ngb = 2 * (RB / (BITS * GS / 8)); ge.bits = BITS; ge.gs = GS;
    const int cnt = nlive * nst;
    int slot = 0, npre = 0;
    for (int k = 0; k < 2; ++k) {
        const int pos = warp + k * NW;
        if (pos < cnt) {
            const int lt = pos / nst;
            issue_item(ring + k * SLOT, tiles[lt], pos - lt * nst, ge, lane);
            cp_async_commit();
            npre = k + 1;
        }
    }
    const int xtab_stride = (K / 64) * 2;                               // float2 entries of one activation set
    {
        PrepSrc src;
        src.xs = reinterpret_cast<const uint16_t*>(a.x);
        src.up = reinterpret_cast<const uint16_t*>(a.up);
        src.wts = a.up ? a.wts : nullptr;
        src.limit = a.limit; src.ldx = a.ldx; src.nx = nx;
        prep_limbs<AT, BITS, GS>(src, K, limbs, tab, LS, xtab_stride, tid, THREADS);
    }
    __syncthreads();

    WarpCtx w;
    w.tl = tiles; w.ge = ge; w.cnt = cnt; w.nst = nst; w.stage0 = 0;
    w.tl1 = tiles; w.ge1 = ge; w.lt1 = w.st1 = w.lt1b = w.st1b = 0; w.next_n = 0;
    run_op<AT, BITS, GS, NW, true>(w, ring, limbs, LS, zero, tab, myy, warp, lane, slot, npre, xtab_stride);
    cp_async_wait<0>();
    __syncthreads();

    for (int t = tid; t < nlive * 16; t += THREADS) {
        float part[NW];
#pragma unroll
        for (int ww = 0; ww < NW; ++ww) part[ww] = ysum[(size_t)ww * MAXT * 16 + t];
        float v = 0.f;
#pragma unroll
        for (int ww = 0; ww < NW; ++ww) v += part[ww];             // always in warp order
        if ((t & 15) < tiles[t >> 4].rows_valid) ytile[t >> 4][t & 15] = A::from_f32(v);
    }
}

template <typename AT, int BITS, int GS, int NW>
static int launch_gather_cfg(const GatherArgs& a, int nx, int grid, bool pdl, cudaStream_t st, bool* launched) {
    const size_t smem = gather_head_bytes(a.K, nx, NW, BITS) + (size_t)NW * 2 * SLOT;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(gather_one_kernel<AT, BITS, GS, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    cfg.numAttrs = pdl ? 1 : 0;
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, gather_one_kernel<AT, BITS, GS, NW>, a));
    *launched = true;
    return JQ_OK;
}

template <typename AT, int BITS, int GS>
static int launch_gather_shape(GatherArgs a, bool pdl, cudaStream_t st, bool* launched) {
    const int sms = sm_count();
    const int nx = (a.pairs + a.x_div - 1) / a.x_div;
    const int64_t tiles = (int64_t)a.banks * a.pairs * ((a.N + 15) / 16);
    const int tpc = (int)((tiles + sms - 1) / sms);
    if (tpc > MAXT) return JQ_OK;
    a.tpc = tpc;
    const int grid = (int)((tiles + tpc - 1) / tpc);
    for (int nw : {16, 12, 8}) {
        if (gather_head_bytes(a.K, nx, nw, BITS) + (size_t)nw * 2 * SLOT > (size_t)MAX_SMEM) continue;
        if (nw == 16) return launch_gather_cfg<AT, BITS, GS, 16>(a, nx, grid, pdl, st, launched);
        if (nw == 12) return launch_gather_cfg<AT, BITS, GS, 12>(a, nx, grid, pdl, st, launched);
        return launch_gather_cfg<AT, BITS, GS, 8>(a, nx, grid, pdl, st, launched);
    }
    return JQ_OK;
}

// ---- the same for more pairs of which few are local (expert-parallel decode) -------------------------------------
// With the experts sharded over the ranks every rank sees the pairs of all tokens of the step (up to 128) but owns
// the experts of only about pairs / world of them.  Every CTA first compacts the local pairs (ballots over the
// pair list), then the launch walks them in rounds of up to 16: a round is the one-token gather above over the
// round's pairs -- tile list, requests, limbs, items, row sums.  Rows of the other pairs are written as zeros, pair p
// by CTA p mod grid.  Limbs: one set per activation row when pairs share rows (gate/up: prepared once), else one set
// per pair that this CTA's tiles of the round touch (down: a CTA's tiles lie in one or two pairs).
constexpr int SPARSE_MAX_PAIRS = 128;

__host__ __device__ inline size_t sparse_head_bytes(int K, int nsets, int nw, int bits) {
    const size_t limbs = ((size_t)nsets * 3 * limb_stride_bits(K, bits) + 127) / 128 * 128;
    return HEAD0 + MAXT * sizeof(TileInfo) + MAXT * sizeof(void*) + 64 + SPARSE_MAX_PAIRS * 4 + SPARSE_MAX_PAIRS + MAXT * 4 +
           (size_t)nsets * (K / 64) * 16 + limbs + (size_t)nw * MAXT * 16 * sizeof(float);
}

template <typename AT, int BITS, int GS, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
gather_sparse_kernel(const GatherArgs a, const int nsets) {
    using A = Act<AT>;
    constexpr int THREADS = NW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = a.K, G = a.G, N = a.N;
    const int LS = limb_stride_bits(K, BITS);
    constexpr int RB = rowb_of(BITS);
    const int rowbytes = K * BITS / 8;
    const int nst = (rowbytes + RB - 1) / RB;
    const int tpm = (N + 15) / 16;
    const bool per_pair = a.x_div == 1;                               // a row (and a set of limbs) per pair
    const int nrows = (a.pairs + a.x_div - 1) / a.x_div;

    uint8_t* zero = smem;
    TileInfo* tiles = reinterpret_cast<TileInfo*>(smem + HEAD0);                          // [MAXT]
    uint16_t** ytile = reinterpret_cast<uint16_t**>(tiles + MAXT);                        // [MAXT]
    int* misc = reinterpret_cast<int*>(ytile + MAXT);                                     // [16]: 0 = local pairs, 1 = sets
    int* lp = misc + 16;                                                                  // [128] local pairs, ascending
    uint8_t* lflag = reinterpret_cast<uint8_t*>(lp + SPARSE_MAX_PAIRS);                   // [128] pair is local
    int* rowmap = reinterpret_cast<int*>(lflag + SPARSE_MAX_PAIRS);                       // [MAXT] set -> pair
    float2* tab = reinterpret_cast<float2*>(rowmap + MAXT);                               // [nsets][K / 64][2]
    uint8_t* limbs = reinterpret_cast<uint8_t*>(tab) + (size_t)nsets * (K / 64) * 16;     // [nsets][3][LS]
    float* ysum = reinterpret_cast<float*>(limbs + ((size_t)nsets * 3 * LS + 127) / 128 * 128);
    uint8_t* ring = smem + sparse_head_bytes(K, nsets, NW, BITS) + (size_t)warp * 2 * SLOT;
    float* myy = ysum + (size_t)warp * MAXT * 16;

    for (int i = tid; i < ZERO_BYTES / 4; i += THREADS) reinterpret_cast<uint32_t*>(zero)[i] = 0u;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        int nl = 0;
        for (int p0 = 0; p0 < a.pairs; p0 += 32) {
            const int p = p0 + lane;
            bool live = false;
            if (p < a.pairs) {
                const int e = a.pair_expert[p] - a.expert_base;
                live = e >= 0 && e < a.num_experts;
                lflag[p] = live ? 1 : 0;
            }
            const unsigned mask = __ballot_sync(0xFFFFFFFFu, live);
            if (live) lp[nl + __popc(mask & ((1u << lane) - 1u))] = p;
            nl += __popc(mask);
        }
        if (lane == 0) misc[0] = nl;
    }
    __syncthreads();
    const int nl = misc[0];
    // zero rows of the pairs whose expert lives on another rank
    for (int p = (int)blockIdx.x; p < a.pairs; p += (int)gridDim.x) {
        if (lflag[p]) continue;
        for (int b = 0; b < a.banks; ++b) {
            uint16_t* yr = reinterpret_cast<uint16_t*>(a.y[b]) + (int64_t)p * a.ldy;
            for (int c = tid; c < N; c += THREADS) yr[c] = 0;
        }
    }
    OpGeo ge;
    ge.rowbytes = rowbytes; ge.G = G; ge.rowb = RB; ge.rsb = rsb_of(BITS);
    ge.grpb = BITS * GS / 8; ge.ngb = 2 * (RB / (BITS * GS / 8)); ge.bits = BITS; ge.gs = GS;
    const int xtab_stride = (K / 64) * 2;
    PrepSrc src;
    src.xs = reinterpret_cast<const uint16_t*>(a.x);
    src.up = reinterpret_cast<const uint16_t*>(a.up);
    src.wts = a.up ? a.wts : nullptr;
    src.limit = a.limit; src.ldx = a.ldx;
    if (!per_pair && nl > 0) {                                        // shared rows: all sets once
        src.nx = nrows;
        prep_limbs<AT, BITS, GS>(src, K, limbs, tab, LS, xtab_stride, tid, THREADS);
    }
    for (int q0 = 0; q0 < nl; q0 += 16) {
        const int nq = min(16, nl - q0);
        const int tiles_r = a.banks * nq * tpm;
        const int tpc = (tiles_r + (int)gridDim.x - 1) / (int)gridDim.x;      // <= MAXT (checked by the host)
        const int tile0 = (int)blockIdx.x * tpc;
        const int ntile = max(0, min(tpc, tiles_r - tile0));
        if (warp == 0) {
            int qi = -1;
            if (lane < ntile) {
                const int gt = tile0 + lane;
                const int j = gt / tpm, tm = gt - j * tpm;
                const int b = j / nq;
                qi = j - b * nq;
                const int p = lp[q0 + qi];
                const int e = a.pair_expert[p] - a.expert_base;
                const int row0 = tm * 16;
                TileInfo ti;
                ti.codes = reinterpret_cast<const uint8_t*>(a.codes_tab[b][e]) + (int64_t)row0 * rowbytes;
                ti.scales = reinterpret_cast<const uint16_t*>(a.scales_tab[b][e]) + (int64_t)row0 * G;
                ti.biases = reinterpret_cast<const uint16_t*>(a.biases_tab[b][e]) + (int64_t)row0 * G;
                ti.rows_valid = min(16, N - row0);
                ti.xsel = p / a.x_div;
                tiles[lane] = ti;
                ytile[lane] = reinterpret_cast<uint16_t*>(a.y[b]) + (int64_t)p * a.ldy + row0;
            }
            if (per_pair) {
                // sets of this CTA and round: the distinct pairs of its tiles, numbered by first appearance
                const unsigned peers = __match_any_sync(0xFFFFFFFFu, qi);
                const bool leader = qi >= 0 && (peers & ((1u << lane) - 1u)) == 0;
                const unsigned leaders = __ballot_sync(0xFFFFFFFFu, leader);
                const int first = __ffs(peers) - 1;
                const int set = __popc(leaders & ((1u << first) - 1u));
                if (qi >= 0) tiles[lane].xsel = set;
                if (leader) rowmap[set] = lp[q0 + qi];
                if (lane == 0) misc[1] = __popc(leaders);
            }
        }
        __syncthreads();
        for (int i = lane; i < ntile * 16; i += 32) myy[i] = 0.f;
        const int cnt = ntile * nst;
        int slot = 0, npre = 0;
        for (int k = 0; k < 2; ++k) {
            const int pos = warp + k * NW;
            if (pos < cnt) {
                const int lt = pos / nst;
                issue_item(ring + k * SLOT, tiles[lt], pos - lt * nst, ge, lane);
                cp_async_commit();
                npre = k + 1;
            }
        }
        if (per_pair && ntile > 0) {
            src.nx = misc[1];
            src.rowmap = rowmap;
            prep_limbs<AT, BITS, GS>(src, K, limbs, tab, LS, xtab_stride, tid, THREADS);
        }
        __syncthreads();
        WarpCtx w;
        w.tl = tiles; w.ge = ge; w.cnt = cnt; w.nst = nst; w.stage0 = 0;
        w.tl1 = tiles; w.ge1 = ge; w.lt1 = w.st1 = w.lt1b = w.st1b = 0; w.next_n = 0;
        run_op<AT, BITS, GS, NW, true>(w, ring, limbs, LS, zero, tab, myy, warp, lane, slot, npre, xtab_stride);
        cp_async_wait<0>();
        __syncthreads();
        for (int t = tid; t < ntile * 16; t += THREADS) {
            float v = 0.f;
#pragma unroll
            for (int ww = 0; ww < NW; ++ww) v += ysum[(size_t)ww * MAXT * 16 + t];      // always in warp order
            if ((t & 15) < tiles[t >> 4].rows_valid) ytile[t >> 4][t & 15] = A::from_f32(v);
        }
        __syncthreads();                                                // the lists are rebuilt by the next round
    }
}

template <typename AT, int BITS, int GS, int NW>
static int launch_sparse_cfg(const GatherArgs& a, int nsets, int grid, bool pdl, cudaStream_t st, bool* launched) {
    const size_t smem = sparse_head_bytes(a.K, nsets, NW, BITS) + (size_t)NW * 2 * SLOT;
    static bool attr_done[64] = {};        // per device; benign race: the attribute call is idempotent
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(gather_sparse_kernel<AT, BITS, GS, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    cfg.numAttrs = pdl ? 1 : 0;
    JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, gather_sparse_kernel<AT, BITS, GS, NW>, a, nsets));
    *launched = true;
    return JQ_OK;
}

template <typename AT, int BITS, int GS>
static int launch_sparse_shape(GatherArgs a, bool pdl, cudaStream_t st, bool* launched) {
    const int grid = sm_count();
    const int tpm = (a.N + 15) / 16;
    const int64_t round_tiles = (int64_t)a.banks * 16 * tpm;                       // a full round of 16 pairs
    const int tpc = (int)((round_tiles + grid - 1) / grid);
    if (tpc > MAXT) return JQ_OK;
    // limb sets: the activation rows (shared rows), or the pairs one CTA's tiles of a round can lie in
    const int nsets = a.x_div == 1 ? std::min(16, (tpc + tpm - 1) / tpm + 1) : (a.pairs + a.x_div - 1) / a.x_div;
    if (nsets > 16) return JQ_OK;
    for (int nw : {16, 12, 8}) {
        if (sparse_head_bytes(a.K, nsets, nw, BITS) + (size_t)nw * 2 * SLOT > (size_t)MAX_SMEM) continue;
        if (nw == 16) return launch_sparse_cfg<AT, BITS, GS, 16>(a, nsets, grid, pdl, st, launched);
        if (nw == 12) return launch_sparse_cfg<AT, BITS, GS, 12>(a, nsets, grid, pdl, st, launched);
        return launch_sparse_cfg<AT, BITS, GS, 8>(a, nsets, grid, pdl, st, launched);
    }
    return JQ_OK;
}

}  // namespace one

// Dense mat-vecs with one activation row (one launch for all matrices of `bt`) on the item-streaming integer
// kernel; *launched stays false when the shape does not fit it (other widths, more rows, K / gs not a
// multiple of 4, more than 16 row tiles per SM).
int launch_one_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                      bool* launched) {
    *launched = false;
    if (!(bits == 2 || bits == 3 || bits == 4 || bits == 6 || bits == 8) || a.M != 1 || a.K % (4 * gs) != 0 ||
        a.K >= (1 << 24))
        return JQ_OK;
    int rc = JQ_OK;
#define JQ_ONE_CASE(B, GSZ)                                                                          \
    if (bits == B && gs == GSZ) {                                                                    \
        rc = (act_dtype == JQ_BF16) ? one::launch_shape<__nv_bfloat16, B, GSZ>(a, bt, st, launched)  \
                                    : one::launch_shape<__half, B, GSZ>(a, bt, st, launched);        \
    }
    JQ_ONE_CASE(2, 64) JQ_ONE_CASE(3, 64) JQ_ONE_CASE(4, 64) JQ_ONE_CASE(6, 64) JQ_ONE_CASE(8, 64)
    JQ_ONE_CASE(2, 128) JQ_ONE_CASE(3, 128) JQ_ONE_CASE(4, 128) JQ_ONE_CASE(6, 128) JQ_ONE_CASE(8, 128)
#undef JQ_ONE_CASE
    return rc;
}

}  // namespace jq

namespace jq {

// Routed-expert gather for one token on the item-streaming integer kernel (see GatherArgs); *launched stays false
// when the shape does not fit (more than 16 pairs, other widths, K / gs not a multiple of 4, too many tiles).
int launch_gather_one(const void* x, const void* up, const float* wts, float limit, int64_t ldx, int x_div,
                      const int32_t* pair_expert, int pairs, int banks, const uint32_t* const* codes_tab,
                      const void* const* scales_tab, const void* const* biases_tab, const uint32_t* const* codes_tab2,
                      const void* const* scales_tab2, const void* const* biases_tab2, int num_experts, int expert_base,
                      int act_dtype, int64_t N, int64_t K, int bits, int gs, void* y, void* y2, int64_t ldy, bool pdl,
                      cudaStream_t st, bool* launched, bool sparse) {
    *launched = false;
    if (!(bits == 2 || bits == 3 || bits == 4 || bits == 6 || bits == 8) || !(gs == 64 || gs == 128) || K % (4 * gs) != 0 ||
        pairs < 1 || x_div < 1 || N < 1 || N >= (1 << 24) || K >= (1 << 22))
        return JQ_OK;
    // more than 16 pairs: only when the caller says that few of them are local, and whole rows per x_div pairs
    if (pairs > 16 && (!sparse || pairs > one::SPARSE_MAX_PAIRS || pairs % x_div != 0)) return JQ_OK;
    one::GatherArgs a = {};
    a.x = x; a.up = up; a.wts = wts; a.limit = limit; a.ldx = ldx; a.x_div = x_div;
    a.pair_expert = pair_expert; a.pairs = pairs; a.banks = banks;
    a.codes_tab[0] = codes_tab; a.scales_tab[0] = scales_tab; a.biases_tab[0] = biases_tab;
    a.codes_tab[1] = codes_tab2; a.scales_tab[1] = scales_tab2; a.biases_tab[1] = biases_tab2;
    a.y[0] = y; a.y[1] = y2; a.ldy = ldy;
    a.num_experts = num_experts; a.expert_base = expert_base;
    a.N = (int)N; a.K = (int)K; a.G = (int)(K / gs);
    int rc = JQ_OK;
#define JQ_GATHER_CASE(B, GSZ)                                                                               \
    if (bits == B && gs == GSZ) {                                                                            \
        if (pairs > 16)                                                                                      \
            rc = (act_dtype == JQ_BF16) ? one::launch_sparse_shape<__nv_bfloat16, B, GSZ>(a, pdl, st, launched)  \
                                        : one::launch_sparse_shape<__half, B, GSZ>(a, pdl, st, launched);    \
        else                                                                                                 \
            rc = (act_dtype == JQ_BF16) ? one::launch_gather_shape<__nv_bfloat16, B, GSZ>(a, pdl, st, launched)  \
                                        : one::launch_gather_shape<__half, B, GSZ>(a, pdl, st, launched);    \
    }
    JQ_GATHER_CASE(2, 64) JQ_GATHER_CASE(3, 64) JQ_GATHER_CASE(4, 64) JQ_GATHER_CASE(6, 64) JQ_GATHER_CASE(8, 64)
    JQ_GATHER_CASE(2, 128) JQ_GATHER_CASE(3, 128) JQ_GATHER_CASE(4, 128) JQ_GATHER_CASE(6, 128) JQ_GATHER_CASE(8, 128)
#undef JQ_GATHER_CASE
    return rc;
}

}  // namespace jq
