// Randomized Hadamard rotation of rows, y = H * diag(signs) * x per power-of-two block of the row
// (jang_tools/turboquant/rotation.py:86-113).  Bundles converted with the rotation store W rotated along
// K (jang_tools/convert.py:1496-1512) and every such linear layer rotates its input the same way at inference
// (jang_tools/loader.py:1763-1767), so this sits directly in front of the quantized mat-vec.
//
// One CTA per row; the row lives in shared memory as float32.  A row of length K is cut into its binary
// digits' blocks, largest first (11008 = 8192 + 2048 + 512 + 256); each block gets the butterflies
// (a, b) -> (a + b, a - b) for h = 1, 2, 4, ... with one barrier per stage, then * float32(1/sqrt(block)).
// The float32 operations and their order are the reference's, so the result does not depend on the launch.
// Bound: HBM for large row counts (read + write one row each); a single decode row is latency-bound
// (log2(K) barriers).
#include "jq_common.cuh"

namespace jq {

template <typename X, typename O>
__global__ void __launch_bounds__(512)
hadamard_kernel(const X* __restrict__ x, int64_t ldx, const float* __restrict__ signs, int K, O* __restrict__ out,
                int64_t ldo) {
    extern __shared__ float row[];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const X* xr = x + (int64_t)blockIdx.x * ldx;
    for (int i = threadIdx.x; i < K; i += blockDim.x) row[i] = __fmul_rn(Elt<X>::to_f32(xr[i]), signs[i]);
    __syncthreads();
    int off = 0, rem = K;
    while (rem > 0) {
        const int d = 1 << (31 - __clz(rem));            // largest power of two <= rem
        float* s = row + off;
        for (int h = 1; h < d; h <<= 1) {
            for (int i = threadIdx.x; i < d / 2; i += blockDim.x) {
                const int lo = (i / h) * 2 * h + (i % h);
                const float a = s[lo], b = s[lo + h];
                s[lo] = __fadd_rn(a, b);
                s[lo + h] = __fsub_rn(a, b);
            }
            __syncthreads();
        }
        const float norm = (float)(1.0 / sqrt((double)d));
        for (int i = threadIdx.x; i < d; i += blockDim.x) s[i] = __fmul_rn(s[i], norm);
        off += d;
        rem -= d;
    }
    __syncthreads();
    O* orow = out + (int64_t)blockIdx.x * ldo;
    for (int i = threadIdx.x; i < K; i += blockDim.x) orow[i] = Elt<O>::from_f32(row[i]);
}

}  // namespace jq

extern "C" {

int jq_hadamard_rotate(const void* x, int x_dtype, int64_t ldx, int64_t rows, int64_t K, const float* signs,
                       void* out, int out_dtype, int64_t ldo, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(valid_dtype(x_dtype) && valid_dtype(out_dtype), JQ_EINVAL, "bad dtype");
    JQ_REQUIRE(rows >= 0 && K >= 0 && K <= 49152, JQ_EINVAL, "rows must be >= 0 and 0 <= K <= 49152");
    if (rows == 0 || K == 0) return JQ_OK;
    JQ_REQUIRE(x && signs && out, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(ldx >= K && ldo >= K, JQ_EINVAL, "leading dimension too small");
    JQ_REQUIRE(rows < (1ll << 31), JQ_EUNSUPPORTED, "too many rows for one launch");
    const size_t smem = (size_t)K * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
    JQ_DISPATCH_DTYPE(x_dtype, X,
        JQ_DISPATCH_DTYPE(out_dtype, O, {
            if (smem > 48 * 1024)
                JQ_CUDA_OK(cudaFuncSetAttribute(hadamard_kernel<X, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            hadamard_kernel<X, O><<<(unsigned)rows, 512, smem, st>>>((const X*)x, ldx, signs, (int)K, (O*)out, ldo);
        }))
    return check_launch("hadamard_rotate");
}

}  // extern "C"
