/*
 * jangq_b200 — C ABI of the B200 (sm_100a) implementation of JANG's affine
 * mixed-bit quantized-inference path.
 *
 * The reference (jjang-ai/jangq) has no FFI of its own: its operator boundary
 * is the MLX Python op signature plus the tensor layout contract
 * (FORMAT.md:57-91, docs/adoption/PORTING.md:62-116).  Each entry point below
 * names the reference call it stands in for.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer valid on the device of `stream`;
 *   - every call only enqueues work on `stream` (a cudaStream_t passed as
 *     void*; NULL = the legacy default stream) and returns without syncing;
 *   - the caller owns every buffer, including workspaces; nothing here
 *     allocates device memory;
 *   - return value: JQ_OK or a JQ_E* status; jq_last_error() gives the detail
 *     for the calling thread;
 *   - tensor layout: codes uint32 [rows, K*bits/32] row-major, LSB-first
 *     bitstream per row; scales/biases [rows, K/group_size];
 *     dequant = code*scale + bias; bits in {2,3,4,5,6,8}; group_size in
 *     {32,64,128}; K % group_size == 0; K*bits % 32 == 0.
 */
#ifndef JANGQ_B200_H
#define JANGQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JQ_OK            0
#define JQ_EINVAL        1   /* bad shape, alignment, dtype or null pointer   */
#define JQ_EUNSUPPORTED  2   /* bits / group_size / size outside the kernels  */
#define JQ_EWORKSPACE    3   /* caller workspace too small                    */
#define JQ_ECUDA         4   /* a CUDA runtime call failed (see last error)   */
#define JQ_ETIMEOUT      5   /* a bounded device-side wait ran out            */

#define JQ_F32   0
#define JQ_F16   1
#define JQ_BF16  2

/* jq_quantize / jq_quantize_rtn flags */
#define JQ_QUANT_F16_TINY_GUARD  1  /* numpy-mirror floor on |scale| for f16 sidecars
                                       (jang_tools/affine.py:46-51); MLX itself has none */
#define JQ_QUANT_IEEE_DIV        4  /* per-weight IEEE division behind a guarded reciprocal instead of the
                                       reciprocal-and-residual form (same codes; for cross-checking) */
/* jq_quantize_mse flags */
#define JQ_QUANT_MSE_EXHAUSTIVE  2  /* evaluate every clip ratio in float64, no float32 screen */

typedef void* jq_stream_t;

int         jq_version(void);
const char* jq_status_string(int status);
const char* jq_last_error(void);

/* K1. Affine group quantizer: stands in for mx.quantize(w, group_size, bits)
 * (jang_tools/convert.py:602-645,1533-1554) and its numpy mirror
 * quantize_native_affine_numpy (jang_tools/affine.py:193-276).
 * w [rows,K] of w_dtype; codes are bit-exact with the reference for the same
 * source dtype; scales/biases are written in sidecar_dtype. */
int jq_quantize(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int group_size,
                int sidecar_dtype, int flags, uint32_t* codes, void* scales, void* biases,
                jq_stream_t stream);

/* K1b. Zero-point round-to-nearest quantizer, the converter's fallback when MLX
 * is missing: quantize_tensor(method="rtn") (jang_tools/quantize.py:211-289,
 * caller convert.py:1564-1592).  Sidecars are float16 as in the reference. */
int jq_quantize_rtn(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int group_size,
                    int sidecar_dtype, int flags, uint32_t* codes, void* scales, void* biases,
                    jq_stream_t stream);

/* K1c. The same zero-point quantizer with the clip-ratio search that is
 * quantize_tensor's default, method="mse" (jang_tools/quantize.py:153-191): 20
 * ratios in [0.7, 1.0] per block, least mean squared error wins; 2-4 bits, wider
 * codes take the K1b arithmetic as in the reference (:153).  Bit-exact with the
 * reference under NumPy >= 2, where the search runs in float64.  A float32 pass
 * first discards the ratios that provably cannot win; JQ_QUANT_MSE_EXHAUSTIVE
 * evaluates all 20 in float64 instead (same result, for cross-checking). */
int jq_quantize_mse(const void* w, int w_dtype, int64_t rows, int64_t K, int bits, int group_size,
                    int sidecar_dtype, int flags, uint32_t* codes, void* scales, void* biases,
                    jq_stream_t stream);

/* Dequantizer: mx.dequantize / dequantize_affine_numpy (jang_tools/affine.py:445-463,
 * loader.py:469).  out [rows,K] of out_dtype; float32 output is bit-exact with the
 * reference (product and sum rounded separately). */
int jq_dequantize(const uint32_t* codes, const void* scales, const void* biases, int sidecar_dtype,
                  int64_t rows, int64_t K, int bits, int group_size, void* out, int out_dtype,
                  jq_stream_t stream);

/* K2. Decode-shaped quantized mat-vec: mx.quantized_matmul(x, W, scales, biases,
 * transpose=True, group_size, bits) for few activation rows
 * (jang_tools/jangrt/linear.py:41-45, dots3/ops.py:44-52; qmv arithmetic
 * dsv41/metal_decode.py:201-234).  y[M,N] = x[M,K] . deq(W)[N,K]^T, f32 accumulate.
 * M <= JQ_QGEMV_MAX_M; x and y are row-major with leading dimensions ldx / ldy
 * (elements).  x_dtype/y_dtype: JQ_BF16 or JQ_F16 (same type for both). */
#define JQ_QGEMV_MAX_M 16
int jq_qgemv(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes,
             const void* scales, const void* biases, int sidecar_dtype, int64_t N, int64_t K,
             int bits, int group_size, void* y, int y_dtype, int64_t ldy, jq_stream_t stream);

/* Same as jq_qgemv with launch flags.
 * JQ_GEMV_STATIC_WEIGHTS: the caller guarantees that codes/scales/biases are not written
 * by earlier work on `stream`.  The kernel is then launched with programmatic stream
 * serialization: it may start, and prefetch its weights, while the previous kernel on
 * the stream is still running, and reads x / writes y only after that kernel has
 * completed.  This is what hides launch latency between the many small mat-vecs of a
 * decode step (the reference measured its decode as dispatch-bound,
 * jang_tools/dsv41/DECODE_DSPARK_METHODS.md:90-93). */
#define JQ_GEMV_STATIC_WEIGHTS 1
/* For the gather mat-vecs (jq_gather_qgemv2, jq_gather_qgemv_swiglu): most pairs name experts outside this bank
 * (expert-parallel decode: about pairs / world are local).  Up to 128 pairs then run on the integer gather, which
 * compacts the local pairs and walks them 16 at a time; without the flag more than 16 pairs take the bf16 warp-MMA
 * gather, which is faster when most pairs are local. */
#define JQ_GATHER_FEW_LOCAL 2
int jq_qgemv_ex(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes,
                const void* scales, const void* biases, int sidecar_dtype, int64_t N, int64_t K,
                int bits, int group_size, void* y, int y_dtype, int64_t ldy, int flags,
                jq_stream_t stream);

/* One launch over several independent matrices (for example q/k/v, or gate/up,
 * of one decoder layer, each with its own bit width): the same arithmetic as
 * jq_qgemv per entry.  `descs` is a HOST array, copied into the launch. */
typedef struct JqGemvDesc {
    const void*     x;       /* [M, K] activations, leading dimension ldx        */
    const uint32_t* codes;   /* [N, K*bits/32]                                   */
    const void*     scales;  /* [N, K/group_size]                                */
    const void*     biases;
    void*           y;       /* [M, N], leading dimension ldy                    */
    int64_t         N, K, ldx, ldy;
    int32_t         bits, group_size;
} JqGemvDesc;
#define JQ_QGEMV_MAX_BATCH 8
int jq_qgemv_batched(const JqGemvDesc* descs, int count, int64_t M, int act_dtype,
                     int sidecar_dtype, jq_stream_t stream);
/* The same with the flags of jq_qgemv_ex.  Consecutive entries that share x, ldx, K, bits and
 * group_size (at most 4 at a time) go out as one launch whose grid is the concatenation of
 * their row blocks; other entries are launched one after the other. */
int jq_qgemv_batched_ex(const JqGemvDesc* descs, int count, int64_t M, int act_dtype,
                        int sidecar_dtype, int flags, jq_stream_t stream);

/* jq_qgemv_batched_ex for one activation row that does not exist yet: the row is
 *     x_out = rms_norm(res + sum_{j<k} y[j, :])      (jq_residual_rmsnorm's arithmetic for T = 1, up to the order
 *                                                     in which the squares are added),
 * formed inside the mat-vec launch: every CTA builds the row in registers on its way to the integer limbs, and
 * one CTA stores it at x_out for the residual path.  With k > 1 this is also the unweighted combine of the routed
 * experts' slot rows, so a decode layer's "combine + residual + norm" launch disappears into the next layer's
 * q/k/v launch.  res [K], y [k, ldy], x_out [K] of the activation type; every descs[i].x must be x_out and every
 * descs[i].K the same K <= 4096.  Widths and shapes the one-row kernel does not take run jq_residual_rmsnorm as a
 * launch of its own first (y rows contiguous then).  x_out must not alias res or y. */
int jq_qgemv_batched_norm(const void* res, const void* y, int64_t ldy, int k, float eps, void* x_out,
                          const JqGemvDesc* descs, int count, int act_dtype, int sidecar_dtype, int flags,
                          jq_stream_t stream);

/* A whole decode step's dependent mat-vecs in ONE persistent launch.  The reference measured its decode
 * as dispatch-bound and fused its dispatches by hand (jang_tools/dsv41/DECODE_DSPARK_METHODS.md:90-128, driver
 * dsv41/metal_decode.py:464-497); on CUDA the same effect needs the boundary between two dependent mat-vecs
 * to be cheaper than a kernel boundary.  A program is an ordered list of ops; op j computes, for each of its
 * 1..4 matrices (they share x, K, the bit width and the group size -- q/k/v, or gate/up),
 *     y_i[N_i] = deq(W_i)[N_i, K] . x[K]            (jq_qgemv's arithmetic, one activation row),
 * and op j + 1 starts only after every output of op j is complete: a grid barrier inside the kernel,
 * across which the next op's weights are already streaming.  x of an op may be any buffer written before
 * the launch or by an op at least two places earlier, or exactly one whole output y_i of the op directly
 * before it (with K == N_i); any other overlap with the previous op's outputs is refused (JQ_EINVAL).
 * Limits: bits 2, 4, 6 or 8; group_size 64 or 128 with K / group_size a multiple of 4; activations, scales,
 * biases and outputs all of act_dtype (f16 or bf16); codes 16-byte, scales/biases 8-byte, x 16-byte
 * aligned; an op whose rows would make one CTA touch more than 16 row tiles (about 35 000 rows at K = 4096)
 * is refused with JQ_EUNSUPPORTED: split it by rows.  Weights must not be written while a program that names
 * them runs.
 *
 * jq_qgemv_stream_workspace_bytes: device bytes a program needs (op table, float32 accumulators, counters).
 * jq_qgemv_stream_prepare: validates the ops (a HOST array), writes the op table into the 256-byte aligned
 *   device workspace and zeroes its counters; synchronises `stream`; call it once, outside stream capture,
 *   and again after jq_device_status() has reported a timeout.  Fills *program (host memory, caller-owned).
 * jq_qgemv_stream_run: one cooperative launch (one CTA per SM) on `stream`; may be captured in a CUDA graph
 *   and replayed.  Two runs of the same program must not overlap (they share the workspace).  Every wait
 *   inside is bounded (0.5 s); if one runs out, jq_device_status() returns JQ_ETIMEOUT and the outputs of that
 *   run are undefined. */
typedef struct JqStreamOp {
    const void*     x;            /* [K] activations of the op                     */
    const uint32_t* codes[4];     /* [N_i, K*bits/32]                              */
    const void*     scales[4];    /* [N_i, K/group_size]                           */
    const void*     biases[4];
    void*           y[4];         /* [N_i]                                         */
    int64_t         N[4];
    int64_t         K;
    int32_t         count;        /* matrices of the op: 1..4                      */
    int32_t         bits, group_size;
} JqStreamOp;
typedef struct JqStreamProgram {  /* filled by jq_qgemv_stream_prepare, read by jq_qgemv_stream_run */
    void*   workspace;
    int32_t n_ops, act_dtype, kmax, maxrows, warps, grid;
} JqStreamProgram;
size_t jq_qgemv_stream_workspace_bytes(const JqStreamOp* ops, int n_ops);
int jq_qgemv_stream_prepare(const JqStreamOp* ops, int n_ops, int act_dtype, void* workspace,
                            size_t workspace_bytes, JqStreamProgram* program, jq_stream_t stream);
int jq_qgemv_stream_run(const JqStreamProgram* program, jq_stream_t stream);

/* K3. Prefill-shaped quantized GEMM: the same mx.quantized_matmul call with many
 * activation rows (MLX switches from qmv to its tiled qmm there; the reference's only
 * statement of that kernel is the tile shape at jang_tools/jangh/kernels.py:34,273-277).
 * Y[M,N] = X[M,K] . deq(W)[N,K]^T on tcgen05 tensor cores: the weights are dequantized to
 * the activation type (one rounding) tile by tile in shared memory, f32 accumulation in
 * tensor memory.  Needs K % 64 == 0 and x/scales/biases/y of the same 16-bit type. */
int jq_qgemm(const void* x, int x_dtype, int64_t M, int64_t ldx, const uint32_t* codes,
             const void* scales, const void* biases, int sidecar_dtype, int64_t N, int64_t K,
             int bits, int group_size, void* y, int y_dtype, int64_t ldy, jq_stream_t stream);

/* ---- K4: routed-MoE gather_qmm --------------------------------------------------------
 * Stands in for mx.gather_qmm(x, W[E,out,packed], scales, biases, rhs_indices, ...) and the
 * sort-by-expert layer logic around it (jang_tools/dots3/ops.py:168-223,
 * dsv41/model.py:847-857,1206-1245; fused decode dsv41/metal_decode.py:334-497).
 * Expert weights are addressed through DEVICE arrays of per-expert device pointers
 * (codes_tab/scales_tab/biases_tab, num_experts entries) so that every expert may have its
 * own bit width: bits_tab (device int32[num_experts], or NULL when all experts share `bits`)
 * makes a launch skip the experts whose width is not `bits`; call once per distinct width. */
#define JQ_MOE_TILE_M 128

/* Upper bound of the number of row tiles jq_moe_sort can emit (sizes tile_expert/tile_row0). */
size_t jq_moe_sort_max_tiles(int64_t n_pairs, int num_experts, int tile_m);

/* Stable sort of the n_pairs = T*k (token, slot) pairs by expert id (dsv41/model.py:1207-1212:
 * order = argsort(flat idx), inv = argsort(order)).  Experts outside
 * [expert_base, expert_base + num_experts) (another rank's, under expert parallelism) are dropped:
 * inv = -1.  expert_offsets[num_experts + 1]; expert_offsets[num_experts] = kept pairs.  Also emits
 * the tile list of the grouped GEMM: tile t covers sorted rows tile_row0[t] .. of expert
 * tile_expert[t]; *num_tiles tiles.  All outputs are device arrays; nothing syncs. */
int jq_moe_sort(const int32_t* topk_idx, int64_t n_pairs, int num_experts, int expert_base,
                int32_t* order, int32_t* inv, int32_t* expert_offsets, int tile_m,
                int32_t* tile_expert, int32_t* tile_row0, int32_t* num_tiles, jq_stream_t stream);

/* dst[p, :] = src[order[p] / div, :] for p < min(*count, max_rows): the activation gather
 * x[order // topk] of dsv41/model.py:1210.  16-bit rows, 16-byte aligned. */
int jq_gather_rows(const void* src, int64_t src_ld, const int32_t* order, const int32_t* count,
                   int div, void* dst, int64_t dst_ld, int64_t cols, int64_t max_rows, int dtype,
                   jq_stream_t stream);

/* Grouped quantized GEMM over the expert-sorted rows (gather_qmm with sorted_indices=True):
 * y_sorted[p, :] = x_sorted[p, :] . deq(W[expert of row p])^T, on the tcgen05 tensor cores. */
int jq_moe_gemm(const void* x_sorted, int act_dtype, int64_t max_rows, int64_t ldx,
                const int32_t* expert_offsets, const int32_t* tile_expert, const int32_t* tile_row0,
                const int32_t* num_tiles, int64_t max_tiles, const uint32_t* const* codes_tab,
                const void* const* scales_tab, const void* const* biases_tab, const int32_t* bits_tab,
                int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y_sorted,
                int64_t ldy, jq_stream_t stream);
/* jq_moe_gemm over a tile list of tile_m rows per entry (the tile_m given to jq_moe_sort): 128, or 256 -- one CTA
 * then carries two 128-row accumulators and every dequantized weight tile feeds both, which pays once experts hold
 * more than 128 rows (bf16 activations and N >= 256 only; JQ_EUNSUPPORTED otherwise). */
int jq_moe_gemm_tiled(const void* x_sorted, int act_dtype, int64_t max_rows, int64_t ldx,
                      const int32_t* expert_offsets, const int32_t* tile_expert, const int32_t* tile_row0,
                      const int32_t* num_tiles, int64_t max_tiles, int tile_m, const uint32_t* const* codes_tab,
                      const void* const* scales_tab, const void* const* biases_tab, const int32_t* bits_tab,
                      int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y_sorted,
                      int64_t ldy, jq_stream_t stream);


/* jq_moe_gemm without any workspace.  No counterpart in the reference (MLX allocates inside
 * gather_qmm); it exists for callers that must not allocate device memory on the request path:
 * a serving process that gave its whole device budget to weight and KV-cache arenas at start-up
 * (a late allocation there can fail, fragment the pool, or stall the device), or a host runtime
 * that calls this library as a plug-in and does not lend its allocator to plug-ins.
 * The tile list that jq_moe_gemm reads from caller buffers is rebuilt here from expert_offsets
 * into a fixed array inside the library (about 12 KB per device, held until the process exits).
 * Limits: num_experts <= 1024 and max_rows <= 65536, otherwise JQ_EUNSUPPORTED.
 * The first call on a device looks the array's device address up; make that call during
 * start-up, before any stream capture.  All calls share the one array and every call rewrites
 * it, so two calls whose kernels may overlap on the GPU (different streams) race: serialise them.
 * Every call puts one small launch in front of the GEMM (one CTA, a thread per expert and a block-wide
 * scan) that rebuilds the tile list; jq_moe_gemm reuses the list jq_moe_sort made and has no such launch.
 * Same inputs and outputs as jq_moe_gemm otherwise; it calls no cudaMalloc/cudaFree. */
int jq_moe_gemm_static(const void* x_sorted, int act_dtype, int64_t max_rows, int64_t ldx,
                       const int32_t* expert_offsets, int num_experts,
                       const uint32_t* const* codes_tab, const void* const* scales_tab,
                       const void* const* biases_tab, const int32_t* bits_tab, int sidecar_dtype,
                       int64_t N, int64_t K, int bits, int group_size, void* y_sorted, int64_t ldy,
                       jq_stream_t stream);

/* h = silu(min(g, limit)) * clip(u, +-limit) * weights[pair] (dsv41/model.py:1216-1226; limit <= 0:
 * no clamp; weights NULL: 1).  pair = order[p] when order != NULL else p; rows p < *count when
 * count != NULL else p < max_rows. */
int jq_moe_swiglu(const void* gate, const void* up, int64_t ld_in, const float* weights,
                  const int32_t* order, const int32_t* count, void* h, int64_t ld_out, int64_t cols,
                  int64_t max_rows, float limit, int dtype, jq_stream_t stream);

/* out[t, :] = sum over the k slots, in slot order, f32: (weights ? weights[t*k+j] : 1) *
 * y[inv ? inv[t*k+j] : t*k+j, :] (dsv41/model.py:1230-1234, dots3/ops.py:223); slots with
 * inv < 0 are skipped.  Writes out (activation dtype) or, when out_f32 != NULL, f32 [T, D]. */
int jq_moe_combine(const void* y, int64_t ldy, const int32_t* inv, const float* weights, int64_t T,
                   int k, int64_t D, void* out, int64_t ldo, float* out_f32, int dtype,
                   jq_stream_t stream);

/* jq_moe_combine plus the always-on (shared) expert: after the slot sum, shared_y[t, :] (activation dtype,
 * [T, D] with leading dimension ld_shared; NULL: none) is added in f32 and the result rounded once --
 * `y + se.w2(...)` of jang_tools/dsv41/model.py:1237-1245, where the fused decode kernels treat the shared
 * expert as one more slot (dsv41/metal_decode.py:376-421). */
int jq_moe_combine_shared(const void* y, int64_t ldy, const int32_t* inv, const float* weights, int64_t T,
                          int k, int64_t D, const void* shared_y, int64_t ld_shared, void* out, int64_t ldo,
                          float* out_f32, int dtype, jq_stream_t stream);

/* Unsorted gather mat-vec for few pairs (the reference's path below its sort threshold of 64,
 * dsv41/model.py:1206, and its fused decode kernels): y[p, :] = deq(W[pair_expert[p]]) .
 * x[p / x_div, :], p < pairs.  Pairs whose expert is outside [0, num_experts) get a zero row. */
int jq_gather_qgemv(const void* x, int act_dtype, int64_t ldx, int x_div, const int32_t* pair_expert,
                    int64_t pairs, const uint32_t* const* codes_tab, const void* const* scales_tab,
                    const void* const* biases_tab, const int32_t* bits_tab, int num_experts,
                    int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size, void* y,
                    int64_t ldy, jq_stream_t stream);

/* The same over two expert banks of equal shape that read the same rows of x (gate and up of the
 * routed SwiGLU experts, dsv41/model.py:1216-1220) in one launch: y[p] from the first tables, y2[p]
 * from the second (all four second-bank arguments NULL: one bank).  pair_expert holds global expert ids
 * and the tables describe the experts [expert_base, expert_base + num_experts) (expert parallelism).
 * Pairs of other experts get a zero row here and in jq_gather_qgemv (the caller need not clear y).
 * flags as for jq_qgemv_ex. */
int jq_gather_qgemv2(const void* x, int act_dtype, int64_t ldx, int x_div, const int32_t* pair_expert,
                     int64_t pairs, const uint32_t* const* codes_tab, const void* const* scales_tab,
                     const void* const* biases_tab, const uint32_t* const* codes_tab2,
                     const void* const* scales_tab2, const void* const* biases_tab2,
                     const int32_t* bits_tab, int num_experts, int sidecar_dtype, int64_t N, int64_t K,
                     int bits, int group_size, void* y, void* y2, int64_t ldy, int expert_base, int flags,
                     jq_stream_t stream);

/* The down projection of the routed experts with the SwiGLU in front of it folded in (few pairs): the
 * reference's second fused decode dispatch, dsv41_moe_dn, reads the activations the first one wrote
 * (jang_tools/dsv41/metal_decode.py:334-421); here the two gather launches stay and the SwiGLU between them
 * disappears: y[p, :] = deq(W[pair_expert[p] - expert_base]) . h[p, :] with
 * h[p, :] = silu(min(g[p, :], limit)) * clip(u[p, :], +-limit) * weights[p], rounded to the activation type --
 * jq_moe_swiglu followed by jq_gather_qgemv2 with x_div = 1.  gate/up: [pairs, K] of the activation type, leading
 * dimension ld_in.  Up to 16 pairs of one width (2, 3, 4, 6 or 8 bits, bits_tab NULL) run as one launch and need no
 * scratch; any other case runs the two launches through h_scratch ([pairs, K], activation type; JQ_EWORKSPACE when
 * it is needed and NULL). */
int jq_gather_qgemv_swiglu(const void* gate, const void* up, int act_dtype, int64_t ld_in, const float* weights,
                           float limit, const int32_t* pair_expert, int64_t pairs, const uint32_t* const* codes_tab,
                           const void* const* scales_tab, const void* const* biases_tab, const int32_t* bits_tab,
                           int num_experts, int sidecar_dtype, int64_t N, int64_t K, int bits, int group_size,
                           void* y, int64_t ldy, int expert_base, int flags, void* h_scratch, jq_stream_t stream);

/* Router of the few-token (decode) path, one launch: logits = x . router_w^T (f32 accumulation,
 * rounded to the activation type), softmax over the experts in f32, the k largest scores with ties
 * to the lower expert id (jang_tools/dsv41/metal_decode.py:1141), weights p / (sum p + 1e-20) * scale
 * when renorm != 0, else p * scale (dots3/ops.py:149-162).  x [T, H] and router_w [num_experts, H]
 * are of the activation type; idx_out int32 [T, k], w_out f32 [T, k].  num_experts <= 1024.
 * counters: T device int32 that are zero when the call starts; the call leaves them zero (the CTAs of a
 * token count themselves in and the last one selects).  logits_ws: T*num_experts floats of scratch. */
int jq_moe_route(const void* x, int act_dtype, int64_t ldx, int64_t T, int64_t H, const void* router_w,
                 int num_experts, int k, int renorm, float scale, int32_t* idx_out, float* w_out,
                 int32_t* counters, float* logits_ws, jq_stream_t stream);

/* The selection half of the router for many tokens, where the logits come from a GEMM: softmax over the experts
 * in f32, the k largest scores with ties to the lower expert id, weights p / (sum p + 1e-20) * scale when
 * renorm != 0, else p * scale (dots3/ops.py:149-162; tie rule of jang_tools/dsv41/metal_decode.py:1141).
 * logits [T, ld >= num_experts], f32 or a 16-bit type; idx_out int32 [T, k], w_out f32 [T, k]; one warp per
 * token, one launch.  num_experts <= 1024. */
int jq_moe_topk(const void* logits, int logits_dtype, int64_t ld, int64_t T, int num_experts, int k, int renorm,
                float scale, int32_t* idx_out, float* w_out, jq_stream_t stream);

/* jq_moe_route with the residual + RMS norm in front of it folded in: x_out = rms_norm(x + res) (no weight, f32
 * arithmetic, rounded to the activation type; x, res, x_out: [T, H] contiguous, H <= 4096), then the router on
 * x_out.  One launch instead of jq_residual_rmsnorm + jq_moe_route in the synthetic decode stacks.
 * x_out must not overlap x or res (the CTAs of a token read both while one of them writes x_out): JQ_EINVAL.
 * counters and logits_ws belong to one stream at a time: calls on different streams need their own. */
int jq_moe_route_norm(const void* x, const void* res, int act_dtype, int64_t T, int64_t H, float eps, void* x_out,
                      const void* router_w, int num_experts, int k, int renorm, float scale, int32_t* idx_out,
                      float* w_out, int32_t* counters, float* logits_ws, jq_stream_t stream);

/* out[t, :] = v / sqrt(mean(v^2) + eps) with v = x[t, :] + sum_{j<k} y[t*k + j, :], f32 arithmetic,
 * activation type out; y is f32 when y_f32 != NULL (then k = 1), else of the activation type.  With k > 1
 * it is also the unweighted combine of the routed experts' k slot rows (their routing weights are applied
 * before the down projection, dsv41/model.py:1222-1226).  No counterpart in the reference's quantized
 * path: it is the residual + norm glue between the quantized blocks of the synthetic decode stacks
 * (jangq_b200/stacks.py), one launch instead of several.  H <= 4096. */
int jq_residual_rmsnorm(const void* x, const void* y, const float* y_f32, int k, int64_t T, int64_t H,
                        float eps, void* out, int act_dtype, jq_stream_t stream);

/* Activation-weighted affine quantizer: per group, `iterations` rounds of weighted least squares for scale and
 * bias (weights importance[k] ~ E[x_k^2]) and re-rounding of the codes, float64 arithmetic, float16 sidecars,
 * final codes from the stored sidecars.  Bit-identical to quantize_imatrix_affine_numpy
 * (jang_tools/affine.py:279-399) for the same float32 weights and the same FLOORED importance vector (the
 * caller applies the median floor of affine.py:310-312 on the host: it is a K-vector).  w: [rows, K] f32, f16 or
 * bf16 (read as float32); importance: K float32 > 0; codes: uint32 [rows, K*bits/32]; scales, biases: float16
 * [rows, K/group_size].  The reference's fourth return value (relative weighted error) is not computed. */
int jq_quantize_imatrix(const void* w, int w_dtype, const float* importance, int64_t rows, int64_t K, int bits,
                        int group_size, int iterations, uint32_t* codes, void* scales_f16, void* biases_f16,
                        jq_stream_t stream);

/* Randomized Hadamard rotation of rows: out[r] = H * diag(signs) * x[r], applied per power-of-two block of
 * the row (K = 11008 -> blocks 8192, 2048, 512, 256), each block normalised by 1/sqrt(block), float32
 * arithmetic in the reference's order.  Stands in for hadamard_rotate (jang_tools/turboquant/rotation.py:86-113):
 * weights before quantization (jang_tools/convert.py:1496-1512, rows of W along K) and the input of every rotated
 * linear layer at inference (jang_tools/loader.py:1763-1767).  signs: K float32 values +-1
 * (numpy default_rng(seed).choice, rotation.py:43-59).  x, out: [rows, K] f32/f16/bf16 with leading dimensions. */
int jq_hadamard_rotate(const void* x, int x_dtype, int64_t ldx, int64_t rows, int64_t K, const float* signs,
                       void* out, int out_dtype, int64_t ldo, jq_stream_t stream);

/* Quantized embedding lookup, out[t, :] = dequantize(row ids[t]) with jq_dequantize's arithmetic (two
 * roundings, q*s then +b).  Stands in for nn.QuantizedEmbedding's mx.dequantize(weight[ids], scales[ids],
 * biases[ids]) and for jang-runtime/Metal/JANGEmbedding.metal:57-98 (jang_embedding_dequant).  ids: T int32
 * on the device; an id outside [0, rows) yields a row of zeros.  out: [T, K] f32/f16/bf16, 16-byte aligned. */
int jq_embedding(const int32_t* ids, int64_t T, const uint32_t* codes, const void* scales, const void* biases,
                 int sidecar_dtype, int64_t rows, int64_t K, int bits, int group_size, void* out, int out_dtype,
                 jq_stream_t stream);

/* JANGTQ: rotated codebook weights (jang_tools/turboquant/linear.py:24-200; kernels
 * jang-runtime/Sources/JANGCoreMetal/JANGTQMatmul.metal:154-363).  Storage per stacked tensor: packed uint32
 * [E, N, ceil(K / (32 / bits))] holding 32 / bits codebook indices per word, LSB first (3-bit words hold 10 and
 * leave 2 bits unused: not the affine codec's continuous bitstream); norms float16 [E, N]; one codebook of
 * 2^bits float32 centroids per (K, bits); bits 2, 3 or 4.  Activations arrive already rotated,
 * x_rot = H diag(signs) x in float32 (jq_hadamard_rotate with out_dtype JQ_F32), outputs are float32, as in the
 * reference's kernels.
 *
 * jq_tq_gather_matmul (jangtq_gather_tq_matmul, metal:281-363):
 *     out[p, n] = norms[e, n] * sum_i codebook[idx[e, n, i]] * x_rot[p / x_div, i],   e = rhs_indices[p]
 *   x_div = 1: every pair has its own activation row (the down projection); x_div = k: the k pairs of a token
 *   share its row.  rhs_indices NULL: expert 0 for every pair (a plain TurboQuantLinear with E = 1).  Pairs whose
 *   expert is outside [0, num_experts) get a row of zeros.
 * jq_tq_fused_gate_up_swiglu (jangtq_fused_gate_up_swiglu, metal:154-262): gate and up of the same expert in one
 *   pass, out_act[p, n] = silu(min(g, limit)) * clip(u, +-limit) (limit <= 0: no clamp).
 * jq_tq_quantize (tq_quantize_weight, linear.py:137-178, after the rotation): per row of w_rot [rows, K] float32
 *   the L2 norm (float16 out, floored at 1e-10 for the division) and for every element the number of
 *   boundaries (midpoints of neighbouring centroids, 2^bits - 1 floats on the device) its normalised value
 *   exceeds, packed as above. */
int jq_tq_gather_matmul(const float* x_rot, int64_t ldx, int x_div, const int32_t* rhs_indices, int64_t pairs,
                        const uint32_t* packed, const void* norms, const float* codebook, int num_experts,
                        int64_t N, int64_t K, int bits, float* out, int64_t ldo, jq_stream_t stream);
int jq_tq_fused_gate_up_swiglu(const float* x_rot, int64_t ldx, int x_div, const int32_t* rhs_indices,
                               int64_t pairs, const uint32_t* packed_gate, const void* norms_gate,
                               const uint32_t* packed_up, const void* norms_up, const float* codebook,
                               int num_experts, int64_t N, int64_t K, int bits, float swiglu_limit,
                               float* out_act, int64_t ldo, jq_stream_t stream);
int jq_tq_quantize(const float* w_rot, int64_t rows, int64_t K, int bits, const float* boundaries,
                   uint32_t* packed, void* norms, jq_stream_t stream);

/* Expert-parallel prefill, dispatch side: the rows of this rank's (token, slot) pairs packed into fixed-capacity
 * slots per destination rank, ready for ONE equal-split all-to-all (the reference runs on one device; this is the
 * exchange step in front of its gather_qmm call sites, dots3/ops.py:168-192, when the experts are sharded
 * E / world per GPU).  send: [world * capacity] slot rows of H * 2 + 16 bytes -- H values of the activation type,
 * then int32 local expert id (-1: empty slot), float32 routing weight, 8 spare bytes.  Pair p = t * k + j goes to
 * rank idx[p] / (num_experts / world); slot_of_pair[p] receives its slot (dest * capacity + position) or -1 when
 * that destination was already full, in which case *overflow (device int32) becomes 1 -- read it after the step
 * and repeat the step with exact split sizes.  Which slot of its destination a pair gets depends on the launch;
 * no result does (slot rows are computed independently and added per token in slot order by jq_moe_combine with
 * inv = slot_of_pair).  counters: world device int32 of scratch.  Two launches, no host read-back. */
int jq_ep_pack_slots(const void* x, int64_t ldx, const int32_t* idx, const float* w, int64_t T, int k, int64_t H,
                     int num_experts, int world, int64_t capacity, void* send, int32_t* slot_of_pair,
                     int32_t* counters, int32_t* overflow, jq_stream_t stream);

/* Expert-parallel decode: sum of the ranks' partial expert outputs over NVLink peer memory fused with
 * the residual and the RMS norm that consume it (one launch per layer instead of an all-reduce plus
 * jq_residual_rmsnorm).  The reference runs on one device (its gather_qmm call sites,
 * jang_tools/dsv41/model.py:1205-1230, sum the k expert outputs of a token locally); this is the same sum with
 * the experts spread over `world` GPUs.  Every rank calls it with the same x[T,H] and its own y[T*k,H]
 * (rows of pairs owned by other ranks zero, as jq_gather_qgemv2 leaves them).  peer_bufs: host array of
 * `world` device addresses, entry p = rank p's exchange buffer of jq_ep_buffer_bytes(tcap, H) bytes,
 * zero-filled once before the first call and mapped for peer access (entry `rank` is the caller's own).
 * counters: tcap zero-initialised int32 on the device, private to the rank.  The wait for the peers is bounded
 * (2 s, or JANGQ_EP_WAIT_MS milliseconds); when it runs out the call's result is undefined, jq_device_status()
 * returns JQ_ETIMEOUT and later calls do not wait again until jq_device_status_clear().
 * CTA t of every rank waits for CTA t of its peers, so all T CTAs (1024 threads each) must be resident at
 * once: T above what one GPU holds (one or two per SM) is refused with JQ_EUNSUPPORTED.
 * emulate_ranks = world (with rank = 0) runs every rank in one cooperative launch on one GPU: x, y, out and
 * counters then hold the ranks' arrays back to back (testing without a second GPU). */
size_t jq_ep_buffer_bytes(int64_t tcap, int64_t H);
int jq_ep_combine_residual_rmsnorm(const void* x, const void* y, int k, int64_t T, int64_t H, float eps, void* out,
                                   int act_dtype, const uint64_t* peer_bufs, int rank, int world, int64_t tcap,
                                   int32_t* counters, int emulate_ranks, jq_stream_t stream);

/* Reads the device-side status word (synchronises the device).  JQ_ETIMEOUT when a
 * kernel's bounded wait on a copy in flight ran out since the library was loaded.
 * No counterpart in the reference: its Metal path has no device-side waits. */
int jq_device_status(void);

/* Clears the status word (synchronises the device): for a caller that has handled a JQ_ETIMEOUT, e.g. by
 * rebuilding its process group after a rank was lost.  No counterpart in the reference. */
int jq_device_status_clear(void);

#ifdef __cplusplus
}
#endif
#endif /* JANGQ_B200_H */
