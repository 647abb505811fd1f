// K2, whole-step form: ONE persistent launch walks a program of dependent decode mat-vecs
//     y_j[N_j] = deq(W_j)[N_j, K_j] . x_j[K_j]        (one activation row, 2-, 4-, 6- and 8-bit codes)
// e.g. [q,k,v] -> o -> [gate,up] -> down of every layer of a decoder, instead of one launch per op.
//
// Bound: HBM bandwidth.  Algorithmic bytes per op = N*K*bits/8 (codes) + N*(K/gs)*4 (scales, biases) +
// 2*K + 2*N.  With one launch per op, a 17 MB mat-vec (2.7 us of streaming) pays about 3 us of kernel
// boundary, CTA start and limb preparation; here an op boundary is a grid barrier during which the next
// op's weights are already in flight.
//
// Structure: a cooperative launch of one CTA per SM, NW warps each.  An op's work is cut into items of
// 16 weight rows x 256 bytes of packed codes (192 bytes for 6-bit codes; + the items' raw 2-byte scales and biases); the items of an
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

#include "jq_stream_dev.cuh"

namespace jq {

int* status_word();

namespace stream {

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
    DevOp* ops_s = reinterpret_cast<DevOp*>(smem + HEAD0);                            // [3], op j in slot j % 3
    OpCtx* ctx_s = reinterpret_cast<OpCtx*>(ops_s + 3);                                // [4], op j in slot j & 3
    TileInfo* tiles_s = reinterpret_cast<TileInfo*>(ctx_s + 4);                        // [2][MAXT], op j in half j & 1
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
        if (lane == 0) {
            OpCtx cx;
            cx.start = start; cx.cnt = cnt; cx.tile_first = tile_first; cx.nlt = nlt;
            cx.stage0 = start - tile_first * od->nst;
            cx.pad[0] = cx.pad[1] = cx.pad[2] = 0;
            ctx_s[j & 3] = cx;
        }
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
            ti.xsel = 0;
            tiles_s[(j & 1) * MAXT + lane] = ti;
        }
        __syncwarp();
    };
    auto prep = [&](const DevOp& o1, const float* acc) {
        const int nth = THREADS;
        PrepSrc src;
        src.xs = o1.x; src.acc = acc;
#define JQ_STREAM_PREP(B, GSZ) \
        if (o1.bits == B && o1.gs == GSZ) prep_limbs<AT, B, GSZ>(src, o1.K, limbs, tab, LS, 0, tid, nth);
        JQ_STREAM_PREP(2, 64) JQ_STREAM_PREP(4, 64) JQ_STREAM_PREP(6, 64) JQ_STREAM_PREP(8, 64)
        JQ_STREAM_PREP(2, 128) JQ_STREAM_PREP(4, 128) JQ_STREAM_PREP(6, 128) JQ_STREAM_PREP(8, 128)
#undef JQ_STREAM_PREP
    };

    for (int i = tid; i < ZERO_BYTES / 4; i += THREADS) reinterpret_cast<uint32_t*>(zero)[i] = 0u;
    for (int i = tid; i < NW * MAXT * 16; i += THREADS) ysum[i] = 0.f;
    if (warp == NW - 1) { build_tables(0); build_tables(1); }
    __syncthreads();

    int slot = 0, npre = 0;
    {   // the warp's first two items of op 0, then the limbs of op 0 while they are in flight
        const DevOp& o = ops_s[0];
        const OpCtx cx = ctx_s[0];
        for (int k = 0; k < 2; ++k) {
            if (warp + k * NW < cx.cnt) {
                const int pos = cx.stage0 + warp + k * NW;
                const int lt = pos / o.nst;
                issue_item(ring + k * SLOT, tiles_s[lt], pos - lt * o.nst, geo_of(o), lane);
                cp_async_commit();
                npre = k + 1;
            }
        }
        prep(o, nullptr);
    }
    __syncthreads();

    bool aborted = false;
    int prev_rows = 0, prev_region = 0;
    for (int j = 0; j < n_ops; ++j) {
        const DevOp& o = ops_s[j % 3];
        const OpCtx cx = ctx_s[j & 3];
        const int tile_first = cx.tile_first, nlt = cx.nlt;
        {
            WarpCtx w;
            w.tl = tiles_s + (j & 1) * MAXT;
            w.ge = geo_of(o);
            w.cnt = cx.cnt; w.nst = o.nst; w.stage0 = cx.stage0;
            w.next_n = 0;
            w.tl1 = w.tl; w.ge1 = w.ge; w.lt1 = w.st1 = w.lt1b = w.st1b = 0;
            if (j + 1 < n_ops) {
                const DevOp& o1 = ops_s[(j + 1) % 3];
                const OpCtx cx1 = ctx_s[(j + 1) & 3];
                if (warp < cx1.cnt) {
                    const int pos1 = cx1.stage0 + warp;
                    w.next_n = warp + NW < cx1.cnt ? 2 : 1;
                    w.tl1 = tiles_s + ((j + 1) & 1) * MAXT;
                    w.ge1 = geo_of(o1);
                    w.lt1 = pos1 / o1.nst;
                    w.st1 = pos1 - w.lt1 * o1.nst;
                    w.lt1b = (pos1 + NW) / o1.nst;
                    w.st1b = pos1 + NW - w.lt1b * o1.nst;
                }
            }
#define JQ_STREAM_RUN(B, GSZ) \
            if (o.bits == B && o.gs == GSZ) run_op<AT, B, GSZ, NW>(w, ring, limbs, LS, zero, tab, myy, warp, lane, slot, npre);
            JQ_STREAM_RUN(2, 64) JQ_STREAM_RUN(4, 64) JQ_STREAM_RUN(6, 64) JQ_STREAM_RUN(8, 64)
            JQ_STREAM_RUN(2, 128) JQ_STREAM_RUN(4, 128) JQ_STREAM_RUN(6, 128) JQ_STREAM_RUN(8, 128)
#undef JQ_STREAM_RUN
        }
        __syncthreads();
        // the warps' row sums, added in warp order, go to the op's float32 accumulator
        {
            const TileInfo* tl = tiles_s + (j & 1) * MAXT;
            float* acc = yacc + (size_t)o.region * maxrows + (size_t)tile_first * 16;
            for (int t = tid; t < nlt * 16; t += THREADS) {
                float part[NW];
#pragma unroll
                for (int ww = 0; ww < NW; ++ww) {             // independent loads, then the sum in warp order
                    part[ww] = ysum[(size_t)ww * MAXT * 16 + t];
                    ysum[(size_t)ww * MAXT * 16 + t] = 0.f;
                }
                float v = 0.f;
#pragma unroll
                for (int ww = 0; ww < NW; ++ww) v += part[ww];
                if ((t & 15) < tl[t >> 4].rows_valid) atomicAdd(acc + t, v);
            }
        }
        __syncthreads();
        // thread 0 publishes the CTA's sums (the release is cumulative over what the barrier above ordered
        // before it) and waits for the other CTAs; meanwhile the last warp builds the tables of op j + 2
        if (warp == NW - 1) build_tables(j + 2);
        if (tid == 0) {
            red_release_add(&sync->barrier, 1u);
            const unsigned int target = (unsigned int)(j + 1) * (unsigned int)grid;
            const unsigned long long t0 = now_ns();
            bool ok = !aborted;
            unsigned int polls = 0;
            while (ok && ld_acquire(&sync->barrier) < target) {
                if ((++polls & 63u) != 0u) continue;          // the abort flag and the clock: every 64th poll
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
        // behind the barrier: limbs of op j + 1, output conversion of op j
        const int rows = o.tiles * 16;
        const int gid = c * THREADS + tid;
        float cv = 0.f;
        const float* reg_j = yacc + (size_t)o.region * maxrows;
        if (gid < rows) cv = ld_cg_f32(reg_j + gid);          // requested before the limbs, used after them
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
        JQ_REQUIRE(s.bits == 2 || s.bits == 4 || s.bits == 6 || s.bits == 8, JQ_EUNSUPPORTED,
                   "op %d: the streamed program takes 2-, 4-, 6- and 8-bit codes, got %d", j, s.bits);
        JQ_REQUIRE(s.group_size == 64 || s.group_size == 128, JQ_EUNSUPPORTED, "op %d: group size 64 or 128", j);
        JQ_REQUIRE(s.K > 0 && s.K % s.group_size == 0 && s.K < (1 << 24), JQ_EINVAL, "op %d: bad K", j);
        const int G = (int)(s.K / s.group_size);
        JQ_REQUIRE(G % 4 == 0, JQ_EUNSUPPORTED, "op %d: K / group_size must be a multiple of 4", j);
        JQ_REQUIRE(s.x && aligned(s.x, 16), JQ_EINVAL, "op %d: x is null or not 16-byte aligned", j);
        d.x = (const uint16_t*)s.x;
        d.K = (int)s.K; d.G = G; d.bits = s.bits; d.gs = s.group_size; d.count = s.count;
        const int64_t rowbytes = s.K * s.bits / 8;
        d.nst = (int)((rowbytes + rowb_of(s.bits) - 1) / rowb_of(s.bits));
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
