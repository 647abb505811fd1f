// Argument blocks and inner loop shared by the mat-vec kernels (jq_qgemv.cu, jq_qgemv_tc.cu).
#pragma once

#include "jq_mma.cuh"

namespace jq {

struct GemvArgs {
    const void* x;
    const uint32_t* codes;
    const void* scales;
    const void* biases;
    void* y;
    int64_t N, K, ldx, ldy;
    int M, G, nbuf;
    int pdl;      // launched with programmatic stream serialization (weights are static)
    // gather mode (routed experts, decode): blockIdx.y = (token, slot) pair p, expert e = pair_expert[p];
    // weights come from per-expert pointer tables, x row = p / x_div, y row = p, M = 1
    const int32_t* pair_expert;
    const uint32_t* const* codes_tab;
    const void* const* scales_tab;
    const void* const* biases_tab;
    const int32_t* bits_tab;      // optional: experts whose width differs from the launch's are skipped
    int x_div, num_experts;
    int expert_base;              // pair_expert holds global ids; this bank owns [expert_base, expert_base + num_experts)
    // optional second bank (gridDim.z == 2, blockIdx.z == 1): same shapes, own tables and output y2
    const uint32_t* const* codes_tab2;
    const void* const* scales_tab2;
    const void* const* biases_tab2;
    void* y2;
    int ksplit;   // tensor-memory kernel: CTAs of a cluster that split K; one-row kernel: row tiles per CTA
    // one-row kernel, optional: the activation row is formed in the launch as rms_norm(norm_res + sum of the
    // norm_k rows of norm_y) (no weight, f32, rounded to the activation type) and CTA 0 writes it to x
    const void* norm_res;
    const void* norm_y;
    int64_t norm_ldy;
    int norm_k;
    float norm_eps;
    int* status;  // device status word, set to 1 when a bounded wait ran out (tensor-memory kernel)
};

// Matrices of one fused launch: they share the activations (x, ldx), K, the bit width and the group
// size, and differ in weights, output and row count (q/k/v or gate/up of one decoder layer).  The grid
// is the concatenation of their row blocks; blk_end[i] is the first block after matrix i.
constexpr int GEMV_MAX_FUSE = 4;
struct GemvBatch {
    const uint32_t* codes[GEMV_MAX_FUSE];
    const void* scales[GEMV_MAX_FUSE];
    const void* biases[GEMV_MAX_FUSE];
    void* y[GEMV_MAX_FUSE];
    int64_t N[GEMV_MAX_FUSE], ldy[GEMV_MAX_FUSE];
    int blk_end[GEMV_MAX_FUSE];
    int count;
};

// One pipeline stage of one warp: nblk k-blocks of 64 codes for 16*MT weight rows.
//   codes : this lane's first row (row g of the tile) in the staged codes, row stride RS words
//   xrow  : this lane's 16 activations of the first block (row m = g, offset 16*tig), advancing
//           by xstep elements per block (0 for lanes whose m >= M: they read a zero chunk)
//   pt    : (s*POST, b - OFFSET*s) pairs of row g, one per group, row stride NGP
//   xsum  : group sums X[group][8] starting at this lane's column pair (2*tig)
// Per group:  acc += (s*POST) * C + (b - OFFSET*s) * X  with C from the MMAs.
template <typename AT, int BITS, int GS, int MT>
__device__ __forceinline__ void gemv_stage_blocks(const uint32_t* __restrict__ codes, int RS,
                                                  const uint16_t* __restrict__ xrow, int xstep,
                                                  const float2* __restrict__ pt, int NGP,
                                                  const float* __restrict__ xsum, int nblk, int tig,
                                                  float (&acc)[MT][4]) {
    using A = Act<AT>;
    using F = Fields<AT, BITS>;
    constexpr int BPG = GS / 64;
    constexpr int UW = Unit<BITS>::WORDS;
    float cg[MT][F::PASSES][4];
#pragma unroll 2
    for (int blk = 0; blk < nblk; ++blk) {
        uint32_t xr[8];
        {
            const uint4* xp = reinterpret_cast<const uint4*>(xrow);
            const uint4 v0 = xp[0], v1 = xp[1];
            xr[0] = v0.x; xr[1] = v0.y; xr[2] = v0.z; xr[3] = v0.w;
            xr[4] = v1.x; xr[5] = v1.y; xr[6] = v1.z; xr[7] = v1.w;
            xrow += xstep;
        }
        const bool first = (blk % BPG) == 0;
        uint32_t bb[4][2];
        bb[0][0] = make_b<BITS, 0, 0>(xr); bb[0][1] = make_b<BITS, 0, 1>(xr);
        bb[1][0] = make_b<BITS, 1, 0>(xr); bb[1][1] = make_b<BITS, 1, 1>(xr);
        bb[2][0] = make_b<BITS, 2, 0>(xr); bb[2][1] = make_b<BITS, 2, 1>(xr);
        bb[3][0] = make_b<BITS, 3, 0>(xr); bb[3][1] = make_b<BITS, 3, 1>(xr);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            uint32_t ulo[UW], uhi[UW];
            load_unit<BITS>(codes + mt * 16 * RS, blk, tig, ulo);
            load_unit<BITS>(codes + (mt * 16 + 8) * RS, blk, tig, uhi);
#define JQ_STEP(T)                                                                                   \
    {                                                                                                \
        {                                                                                            \
            const uint32_t af[4] = {make_a<AT, BITS, T, 0, 0>(ulo), make_a<AT, BITS, T, 0, 0>(uhi),  \
                                    make_a<AT, BITS, T, 1, 0>(ulo), make_a<AT, BITS, T, 1, 0>(uhi)}; \
            if (T == 0 && first) A::mma0(cg[mt][0], af, bb[T][0], bb[T][1]);                         \
            else A::mma(cg[mt][0], af, bb[T][0], bb[T][1]);                                          \
        }                                                                                            \
        if constexpr (F::PASSES == 2) {                                                              \
            const uint32_t af[4] = {make_a<AT, BITS, T, 0, 1>(ulo), make_a<AT, BITS, T, 0, 1>(uhi),  \
                                    make_a<AT, BITS, T, 1, 1>(ulo), make_a<AT, BITS, T, 1, 1>(uhi)}; \
            if (T == 0 && first) A::mma0(cg[mt][F::PASSES - 1], af, bb[T][0], bb[T][1]);             \
            else A::mma(cg[mt][F::PASSES - 1], af, bb[T][0], bb[T][1]);                              \
        }                                                                                            \
    }
            JQ_STEP(0) JQ_STEP(1) JQ_STEP(2) JQ_STEP(3)
#undef JQ_STEP
        }
        if (blk % BPG == BPG - 1) {
            const float2 xv = *reinterpret_cast<const float2*>(xsum);
            xsum += 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float2 pt_lo = pt[mt * 16 * NGP], pt_hi = pt[(mt * 16 + 8) * NGP];
                float c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    c[i] = cg[mt][0][i];
                    if constexpr (F::PASSES == 2) c[i] = fmaf(16.f, cg[mt][F::PASSES - 1][i], c[i]);
                }
                acc[mt][0] = fmaf(pt_lo.x, c[0], fmaf(pt_lo.y, xv.x, acc[mt][0]));
                acc[mt][1] = fmaf(pt_lo.x, c[1], fmaf(pt_lo.y, xv.y, acc[mt][1]));
                acc[mt][2] = fmaf(pt_hi.x, c[2], fmaf(pt_hi.y, xv.x, acc[mt][2]));
                acc[mt][3] = fmaf(pt_hi.x, c[3], fmaf(pt_hi.y, xv.y, acc[mt][3]));
            }
            ++pt;
        }
    }
}

constexpr int GEMV_MAX_NBUF = 3;   // deepest per-warp stage pipeline of the warp-MMA kernels

// item-streaming integer warp-MMA kernel (jq_qgemv_one.cu), dense mat-vecs of 2-, 4-, 6- and 8-bit codes with one
// activation row; same convention
int launch_one_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                      bool* launched);
// Where the one activation row of a launch comes from when it is formed inside the launch (GemvArgs::norm_*).
struct NormSrc {
    const void* res;
    const void* y;
    int64_t ldy;
    int k;
    float eps;
    void* out;
};

// routed-expert gather for one token on the item-streaming integer kernel (jq_qgemv_one.cu): `banks` x `pairs`
// matrices in one launch, optionally with the activations formed as silu(gate) * up * weight on the fly
int launch_gather_one(const void* x, const void* up, const float* wts, float limit, int64_t ldx, int x_div,
                      const int32_t* pair_expert, int pairs, int banks, const uint32_t* const* codes_tab,
                      const void* const* scales_tab, const void* const* biases_tab, const uint32_t* const* codes_tab2,
                      const void* const* scales_tab2, const void* const* biases_tab2, int num_experts, int expert_base,
                      int act_dtype, int64_t N, int64_t K, int bits, int gs, void* y, void* y2, int64_t ldy, bool pdl,
                      cudaStream_t st, bool* launched, bool sparse = false);

// persistent integer warp-MMA kernel (jq_qgemv_pint.cu), dense mat-vecs of 2- and 4-bit codes with at most 2
// activation rows; same convention
int launch_pint_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                       bool* launched);

// tensor-memory kernel (jq_qgemv_tc.cu), dense mat-vecs only; *launched stays false when the shape does
// not fit it and the caller should use the warp-MMA kernel instead
int launch_tc_kernel(const GemvArgs& a, const GemvBatch& bt, int act_dtype, int bits, int gs, cudaStream_t st,
                     bool* launched);

}  // namespace jq
