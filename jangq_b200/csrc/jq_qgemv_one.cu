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

__host__ __device__ inline size_t one_head_bytes(int K, int nw) {
    const size_t limbs = ((size_t)3 * limb_stride(K) + 127) / 128 * 128;
    return HEAD0 + MAXT * sizeof(TileInfo) + (size_t)(K / 64) * 16 + limbs + (size_t)nw * MAXT * 16 * sizeof(float);
}

template <typename AT, int BITS, int GS, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
qgemv_one_kernel(const GemvArgs a, const GemvBatch bt) {
    using A = Act<AT>;
    constexpr int THREADS = NW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = (int)a.K, G = a.G, TPC = a.ksplit;          // ksplit: 16-row tiles per CTA in this kernel
    const int LS = limb_stride(K);
    constexpr int RB = rowb_of(BITS);
    const int rowbytes = K * BITS / 8;
    const int nst = (rowbytes + RB - 1) / RB;

    uint8_t* zero = smem;
    TileInfo* tiles = reinterpret_cast<TileInfo*>(smem + HEAD0);                        // [MAXT]
    float2* tab = reinterpret_cast<float2*>(tiles + MAXT);                              // [K / 64][2]
    uint8_t* limbs = reinterpret_cast<uint8_t*>(tab) + (size_t)(K / 64) * 16;           // [3][LS]
    float* ysum = reinterpret_cast<float*>(limbs + ((size_t)3 * LS + 127) / 128 * 128);  // [NW][MAXT * 16]
    uint8_t* ring = smem + one_head_bytes(K, NW) + (size_t)warp * 2 * SLOT;
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
        ti.pad = 0;
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
    const uint4 xpre = tid < K / 8 ? ld_cg16(xs + (size_t)tid * 8) : make_uint4(0u, 0u, 0u, 0u);
    request(1);
    prep_limbs<AT, BITS, GS>(xs, nullptr, K, limbs, tab, LS, tid, THREADS, true, xpre);
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
    const size_t smem = one_head_bytes((int)a.K, NW) + (size_t)NW * 2 * SLOT;
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
        if (one_head_bytes((int)a.K, nw) + (size_t)nw * 2 * SLOT > (size_t)MAX_SMEM) continue;
        if (nw == 16) return launch_cfg<AT, BITS, GS, 16>(a, bt, tpc, grid, st, launched);
        if (nw == 12) return launch_cfg<AT, BITS, GS, 12>(a, bt, tpc, grid, st, launched);
        return launch_cfg<AT, BITS, GS, 8>(a, bt, tpc, grid, st, launched);
    }
    return JQ_OK;                                                 // K too long: another kernel
}

}  // namespace one

// Dense mat-vecs with one activation row (one launch for all matrices of `bt`) on the item-streaming integer
// kernel; *launched stays false when the shape does not fit it (other widths, more rows, K / gs not a
// multiple of 4, more than 16 row tiles per SM).
int launch_one_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                      bool* launched) {
    *launched = false;
    if (!(bits == 2 || bits == 4 || bits == 6 || bits == 8) || a.M != 1 || a.K % (4 * gs) != 0 || a.K >= (1 << 24)) return JQ_OK;
    int rc = JQ_OK;
#define JQ_ONE_CASE(B, GSZ)                                                                          \
    if (bits == B && gs == GSZ) {                                                                    \
        rc = (act_dtype == JQ_BF16) ? one::launch_shape<__nv_bfloat16, B, GSZ>(a, bt, st, launched)  \
                                    : one::launch_shape<__half, B, GSZ>(a, bt, st, launched);        \
    }
    JQ_ONE_CASE(2, 64) JQ_ONE_CASE(4, 64) JQ_ONE_CASE(6, 64) JQ_ONE_CASE(8, 64)
    JQ_ONE_CASE(2, 128) JQ_ONE_CASE(4, 128) JQ_ONE_CASE(6, 128) JQ_ONE_CASE(8, 128)
#undef JQ_ONE_CASE
    return rc;
}

}  // namespace jq
