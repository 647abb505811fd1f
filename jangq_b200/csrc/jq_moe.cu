// K4 support kernels for the routed-MoE path: stable sort of (token, slot) pairs by expert,
// row gather, SwiGLU with routing weight, and the top-k combine.  The matmuls themselves are the
// grouped mode of the tensor-core GEMM (jq_qgemm.cu) and the gather mode of the mat-vec
// (jq_qgemv.cu).  All of these are small, bandwidth-bound index/elementwise kernels.
#include "jq_mma.cuh"

namespace jq {

// The small kernels of the few-token path are launched with programmatic stream serialization: their CTAs
// may be scheduled while the predecessor still runs, and they touch memory only after griddepcontrol.wait
// (which returns once the predecessor has completed and flushed), so the launch latency of a chain of
// tiny dependent kernels overlaps.  The instruction is a no-op for a launch without the attribute.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int SORT_THREADS = 1024;
constexpr int SORT_WARPS = SORT_THREADS / 32;

// Stable counting sort of n = T*k expert ids, one CTA.
//   order[p]  = flat pair index (t*k + j) of the p-th pair in expert order (ties: ascending index)
//   inv[i]    = position of pair i in `order`, or -1 when its expert is outside [base, base+E)
//   offsets[e]= first position of local expert e, offsets[E] = number of kept pairs
//   tiles: for every local expert, ceil(count/tile_m) tiles (expert id, first sorted row); *num_tiles
// Shared memory: (SORT_WARPS + 1) * (E + 1) counters.
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int32_t* __restrict__ idx, int n, int E, int base, int32_t* __restrict__ order,
                int32_t* __restrict__ inv, int32_t* __restrict__ offsets, int tile_m, int32_t* __restrict__ tile_expert,
                int32_t* __restrict__ tile_row0, int32_t* __restrict__ num_tiles) {
    extern __shared__ int32_t sm[];
    const int EB = E + 1;                           // bucket E collects dropped pairs
    int32_t* cnt = sm;                              // [SORT_WARPS][EB] per-chunk counts, then running positions
    int32_t* start = sm + SORT_WARPS * EB;          // [EB] exclusive scan over experts
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (SORT_WARPS + 1) * EB; i += SORT_THREADS) sm[i] = 0;
    __syncthreads();
    // chunk of this warp: a contiguous range whose length is a multiple of 32
    const int per = ((n + SORT_WARPS - 1) / SORT_WARPS + 31) / 32 * 32;
    const int lo = min(n, warp * per), hi = min(n, lo + per);
    auto bucket = [&](int i) -> int {
        const int e = idx[i] - base;
        return (e >= 0 && e < E) ? e : E;
    };
    // pass 1: per-chunk histogram.  The ids of 16 steps are loaded up front (one round trip to memory instead
    // of sixteen dependent ones: the loop below synchronises the warp every step).
    constexpr int SORT_BATCH = 16;
    for (int j0 = lo; j0 < hi; j0 += 32 * SORT_BATCH) {
        int bk[SORT_BATCH];
#pragma unroll
        for (int q = 0; q < SORT_BATCH; ++q) {
            const int i = j0 + q * 32 + lane;
            bk[q] = i < hi ? bucket(i) : -1;
        }
#pragma unroll
        for (int q = 0; q < SORT_BATCH; ++q) {
            if (j0 + q * 32 >= hi) break;
            const int b = bk[q];
            const bool act = b >= 0;
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, b);
            if (act && (peers & ((1u << lane) - 1u)) == 0) cnt[warp * EB + b] += __popc(peers);
            __syncwarp();
        }
    }
    __syncthreads();
    // totals per bucket and exclusive scan over buckets (thread 0 .. E: serial scan is fine for E <= 1024)
    for (int b = threadIdx.x; b < EB; b += SORT_THREADS) {
        int tot = 0;
        for (int w = 0; w < SORT_WARPS; ++w) tot += cnt[w * EB + b];
        start[b] = tot;
    }
    __syncthreads();
    // Exclusive scan over the buckets of (pairs, tiles), 1024 buckets at a time with a carry: thread b owns bucket
    // b, a shuffle scan inside the warps and one over the warps' sums give its first position and its first tile;
    // every thread then writes the tiles of its own expert.
    {
        __shared__ int wsum_c[SORT_WARPS], wsum_t[SORT_WARPS], carry[2];
        if (threadIdx.x == 0) carry[0] = carry[1] = 0;
        __syncthreads();
        for (int b0 = 0; b0 < EB; b0 += SORT_THREADS) {
            const int b = b0 + threadIdx.x;
            const int c = b < EB ? start[b] : 0;
            const int tl = b < E ? (c + tile_m - 1) / tile_m : 0;
            int ic = c, it = tl;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int vc = __shfl_up_sync(0xFFFFFFFFu, ic, d), vt = __shfl_up_sync(0xFFFFFFFFu, it, d);
                if (lane >= d) { ic += vc; it += vt; }
            }
            if (lane == 31) { wsum_c[warp] = ic; wsum_t[warp] = it; }
            __syncthreads();
            if (warp == 0) {
                int vc = wsum_c[lane], vt = wsum_t[lane];
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int uc = __shfl_up_sync(0xFFFFFFFFu, vc, d), ut = __shfl_up_sync(0xFFFFFFFFu, vt, d);
                    if (lane >= d) { vc += uc; vt += ut; }
                }
                wsum_c[lane] = vc; wsum_t[lane] = vt;      // inclusive over the warps
            }
            __syncthreads();
            const int run = carry[0] + (warp > 0 ? wsum_c[warp - 1] : 0) + ic - c;
            int tile = carry[1] + (warp > 0 ? wsum_t[warp - 1] : 0) + it - tl;
            if (b < EB) start[b] = run;
            if (b < E) {
                offsets[b] = run;
                for (int r = 0; r < c; r += tile_m, ++tile) {
                    tile_expert[tile] = b;
                    tile_row0[tile] = run + r;
                }
            }
            if (b == E) offsets[E] = run;
            __syncthreads();
            if (threadIdx.x == 0) { carry[0] += wsum_c[SORT_WARPS - 1]; carry[1] += wsum_t[SORT_WARPS - 1]; }
            __syncthreads();
        }
        if (threadIdx.x == 0) *num_tiles = carry[1];
    }
    __syncthreads();
    // per-chunk base positions: start[b] + counts of earlier chunks
    for (int b = threadIdx.x; b < EB; b += SORT_THREADS) {
        int run = start[b];
        for (int w = 0; w < SORT_WARPS; ++w) {
            const int c = cnt[w * EB + b];
            cnt[w * EB + b] = run;
            run += c;
        }
    }
    __syncthreads();
    // pass 2: stable placement
    for (int j0 = lo; j0 < hi; j0 += 32 * SORT_BATCH) {
        int bk[SORT_BATCH];
#pragma unroll
        for (int q = 0; q < SORT_BATCH; ++q) {
            const int i = j0 + q * 32 + lane;
            bk[q] = i < hi ? bucket(i) : -1;
        }
#pragma unroll
        for (int q = 0; q < SORT_BATCH; ++q) {
            if (j0 + q * 32 >= hi) break;
            const int i = j0 + q * 32 + lane;
            const int b = bk[q];
            const bool act = b >= 0;
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, b);
            const int rank = __popc(peers & ((1u << lane) - 1u));
            int pos = 0;
            if (act) pos = cnt[warp * EB + b] + rank;
            __syncwarp();
            if (act && rank == 0) cnt[warp * EB + b] += __popc(peers);
            __syncwarp();
            if (act) {
                if (b < E) {
                    order[pos] = i;
                    inv[i] = pos;
                } else {
                    inv[i] = -1;
                }
            }
        }
    }
}

// ---- the same sort over several CTAs (n >= 2048 pairs, at most 1023 experts) ---------------------------------------
// One CTA's cost is its __match_any_sync steps (one per 32 pairs and pass, and a step costs about as many
// iterations as the warp holds distinct experts): 16384 pairs keep one SM busy for 40 us.  Here chunk c =
// pairs [1024 c, 1024 (c + 1)) (the last chunk also takes the remainder, so it holds 1024..2047 pairs) belongs to
// CTA c: (A) counts per bucket, (B) one CTA turns the counts into first positions per (chunk, bucket), offsets and
// the tile list, (C) stable placement inside the chunk.  The per-chunk tables live in the chunk's own stretch of
// `inv` (1024 entries >= buckets), which CTA c reads into shared memory before it writes its inv entries.
__device__ __forceinline__ int sort_bucket(const int32_t* idx, int i, int base, int E) {
    const int e = idx[i] - base;
    return (e >= 0 && e < E) ? e : E;
}

__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_count_kernel(const int32_t* __restrict__ idx, int n, int E, int base, int chunks, int32_t* __restrict__ inv) {
    extern __shared__ int32_t sm[];                   // [E + 1]
    const int EB = E + 1, c = blockIdx.x, lane = threadIdx.x & 31;
    const int lo = c * SORT_THREADS, hi = c == chunks - 1 ? n : lo + SORT_THREADS;
    for (int b = threadIdx.x; b < EB; b += SORT_THREADS) sm[b] = 0;
    __syncthreads();
    for (int i0 = lo; i0 < hi; i0 += SORT_THREADS) {
        const int i = i0 + threadIdx.x;
        const int b = i < hi ? sort_bucket(idx, i, base, E) : -1;
        const unsigned peers = __match_any_sync(0xFFFFFFFFu, b);
        if (b >= 0 && (peers & ((1u << lane) - 1u)) == 0) atomicAdd(sm + b, __popc(peers));
    }
    __syncthreads();
    for (int b = threadIdx.x; b < EB; b += SORT_THREADS) inv[lo + b] = sm[b];
}

__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_scan_kernel(int E, int chunks, int32_t* __restrict__ inv, int32_t* __restrict__ offsets, int tile_m,
                     int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_row0, int32_t* __restrict__ num_tiles) {
    __shared__ int wsum_c[SORT_WARPS], wsum_t[SORT_WARPS];
    const int EB = E + 1, b = threadIdx.x, warp = b >> 5, lane = b & 31;       // EB <= SORT_THREADS
    int c = 0;
    if (b < EB)
        for (int ch = 0; ch < chunks; ++ch) c += inv[ch * SORT_THREADS + b];
    const int tl = b < E ? (c + tile_m - 1) / tile_m : 0;
    int ic = c, it = tl;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int vc = __shfl_up_sync(0xFFFFFFFFu, ic, d), vt = __shfl_up_sync(0xFFFFFFFFu, it, d);
        if (lane >= d) { ic += vc; it += vt; }
    }
    if (lane == 31) { wsum_c[warp] = ic; wsum_t[warp] = it; }
    __syncthreads();
    if (warp == 0) {
        int vc = wsum_c[lane], vt = wsum_t[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int uc = __shfl_up_sync(0xFFFFFFFFu, vc, d), ut = __shfl_up_sync(0xFFFFFFFFu, vt, d);
            if (lane >= d) { vc += uc; vt += ut; }
        }
        wsum_c[lane] = vc; wsum_t[lane] = vt;
    }
    __syncthreads();
    int run = (warp > 0 ? wsum_c[warp - 1] : 0) + ic - c;
    int tile = (warp > 0 ? wsum_t[warp - 1] : 0) + it - tl;
    if (b < E) {
        offsets[b] = run;
        for (int r = 0; r < c; r += tile_m, ++tile) {
            tile_expert[tile] = b;
            tile_row0[tile] = run + r;
        }
    }
    if (b == E) offsets[E] = run;
    if (b == SORT_THREADS - 1) *num_tiles = wsum_t[SORT_WARPS - 1];
    if (b < EB)
        for (int ch = 0; ch < chunks; ++ch) {          // counts -> first position of (chunk, bucket)
            const int v = inv[ch * SORT_THREADS + b];
            inv[ch * SORT_THREADS + b] = run;
            run += v;
        }
}

__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_place_kernel(const int32_t* __restrict__ idx, int n, int E, int base, int chunks, int32_t* __restrict__ order,
                      int32_t* __restrict__ inv) {
    extern __shared__ int32_t sm[];                   // [SORT_WARPS + 1][E + 1]
    const int EB = E + 1, c = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* wpos = sm;                               // per warp of the round: count, then first position
    int32_t* next = sm + SORT_WARPS * EB;             // first free position of the bucket in this chunk
    const int lo = c * SORT_THREADS, hi = c == chunks - 1 ? n : lo + SORT_THREADS;
    for (int b = threadIdx.x; b < EB; b += SORT_THREADS) next[b] = inv[lo + b];
    __syncthreads();                                  // the chunk's table is read before its inv entries are written
    for (int i0 = lo; i0 < hi; i0 += SORT_THREADS) {
        for (int j = threadIdx.x; j < SORT_WARPS * EB; j += SORT_THREADS) wpos[j] = 0;
        __syncthreads();
        const int i = i0 + threadIdx.x;
        const int b = i < hi ? sort_bucket(idx, i, base, E) : -1;
        const unsigned peers = __match_any_sync(0xFFFFFFFFu, b);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (b >= 0 && rank == 0) wpos[warp * EB + b] = __popc(peers);
        __syncthreads();
        for (int bb = threadIdx.x; bb < EB; bb += SORT_THREADS) {
            int run = next[bb];
            for (int w = 0; w < SORT_WARPS; ++w) {
                const int v = wpos[w * EB + bb];
                wpos[w * EB + bb] = run;
                run += v;
            }
            next[bb] = run;
        }
        __syncthreads();
        if (b >= 0) {
            if (b < E) {
                const int pos = wpos[warp * EB + b] + rank;
                order[pos] = i;
                inv[i] = pos;
            } else {
                inv[i] = -1;
            }
        }
        __syncthreads();
    }
}

// dst[p, :] = src[order[p] / div, :] for p < *count (16-byte vectors; cols*2 % 16 == 0)
__global__ void gather_rows_kernel(const uint4* __restrict__ src, int64_t src_ld_vec, const int32_t* __restrict__ order,
                                   const int32_t* __restrict__ count, int div, uint4* __restrict__ dst,
                                   int64_t dst_ld_vec, int cols_vec, int max_rows) {
    const int n = min(*count, max_rows);
    for (int p = blockIdx.x; p < n; p += gridDim.x) {
        const int64_t s = order[p] / div;
        for (int c = threadIdx.x; c < cols_vec; c += blockDim.x) dst[p * dst_ld_vec + c] = __ldg(src + s * src_ld_vec + c);
    }
}

// h[p, i] = silu(min(g, lim)) * clip(u, -lim, lim) * w[pair(p)]   (dsv41/model.py:1216-1226)
// pair(p) = order[p] when `order` is given (sorted rows), else p.  lim <= 0 disables the clamp.
template <typename AT>
__global__ void swiglu_kernel(const AT* __restrict__ g, const AT* __restrict__ u, int64_t ld_in,
                              const float* __restrict__ w, const int32_t* __restrict__ order,
                              const int32_t* __restrict__ count, AT* __restrict__ h, int64_t ld_out, int cols, int max_rows,
                              float lim) {
    pdl_enter();
    const int n = count ? min(*count, max_rows) : max_rows;
    // rows of whole 16-byte vectors (the grouped-GEMM outputs): 8 elements per thread and step, same arithmetic
    const bool vec = (cols % 8 == 0) && (ld_in % 8 == 0) && (ld_out % 8 == 0) &&
                     ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(h)) % 16 == 0);
    for (int p = blockIdx.x; p < n; p += gridDim.x) {
        const float wt = w ? w[order ? order[p] : p] : 1.0f;
        if (vec) {
            for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
                const uint4 gq = __ldg(reinterpret_cast<const uint4*>(g + p * ld_in + c));
                const uint4 uq = __ldg(reinterpret_cast<const uint4*>(u + p * ld_in + c));
                const AT* ga = reinterpret_cast<const AT*>(&gq);
                const AT* ua = reinterpret_cast<const AT*>(&uq);
                uint4 hq;
                AT* ha = reinterpret_cast<AT*>(&hq);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float gv = Elt<AT>::to_f32(ga[j]), uv = Elt<AT>::to_f32(ua[j]);
                    if (lim > 0.f) {
                        gv = fminf(gv, lim);
                        uv = fminf(fmaxf(uv, -lim), lim);
                    }
                    const float sv = gv / (1.0f + __expf(-gv));
                    ha[j] = Elt<AT>::from_f32(sv * uv * wt);
                }
                *reinterpret_cast<uint4*>(h + p * ld_out + c) = hq;
            }
            continue;
        }
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            float gv = Elt<AT>::to_f32(g[p * ld_in + c]), uv = Elt<AT>::to_f32(u[p * ld_in + c]);
            if (lim > 0.f) {
                gv = fminf(gv, lim);
                uv = fminf(fmaxf(uv, -lim), lim);
            }
            const float s = gv / (1.0f + __expf(-gv));
            h[p * ld_out + c] = Elt<AT>::from_f32(s * uv * wt);
        }
    }
}

// out[t, :] = sum_j (w ? w[t*k+j] : 1) * y[inv ? inv[t*k+j] : t*k+j, :]  in f32, slots in order
// (dsv41/model.py:1230-1234); pairs with inv < 0 (experts of another rank) are skipped.  `shared`
// (optional, [T, D]) is the always-on expert's output, added to the routed sum in f32 (model.py:1237-1245).
template <typename AT>
__global__ void combine_kernel(const AT* __restrict__ y, int64_t ldy, const int32_t* __restrict__ inv,
                               const float* __restrict__ w, int T, int k, int D, AT* __restrict__ out, int64_t ldo,
                               float* __restrict__ out_f32, const AT* __restrict__ shared, int64_t ld_shared) {
    // rows of whole 16-byte vectors: 8 columns per thread, the same sums in the same (slot) order
    const bool vec = (D % 8 == 0) && (ldy % 8 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0) &&
                     (out_f32 ? reinterpret_cast<uintptr_t>(out_f32) % 16 == 0
                              : (ldo % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0)) &&
                     (!shared || (ld_shared % 8 == 0 && reinterpret_cast<uintptr_t>(shared) % 16 == 0));
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        if (vec) {
            for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                for (int j = 0; j < k; ++j) {
                    const int p = inv ? inv[t * k + j] : t * k + j;
                    if (p < 0) continue;
                    const float wj = w ? w[t * k + j] : 1.0f;
                    const uint4 q = __ldg(reinterpret_cast<const uint4*>(y + (int64_t)p * ldy + c));
                    const AT* ya = reinterpret_cast<const AT*>(&q);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = fmaf(wj, Elt<AT>::to_f32(ya[i]), acc[i]);
                }
                if (shared) {
                    const uint4 q = __ldg(reinterpret_cast<const uint4*>(shared + (int64_t)t * ld_shared + c));
                    const AT* sa = reinterpret_cast<const AT*>(&q);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += Elt<AT>::to_f32(sa[i]);
                }
                if (out_f32) {
                    float4* o = reinterpret_cast<float4*>(out_f32 + (int64_t)t * D + c);
                    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
                } else {
                    uint4 oq;
                    AT* oa = reinterpret_cast<AT*>(&oq);
#pragma unroll
                    for (int i = 0; i < 8; ++i) oa[i] = Elt<AT>::from_f32(acc[i]);
                    *reinterpret_cast<uint4*>(out + (int64_t)t * ldo + c) = oq;
                }
            }
            continue;
        }
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            float acc = 0.f;
            for (int j = 0; j < k; ++j) {
                const int p = inv ? inv[t * k + j] : t * k + j;
                if (p >= 0) acc = fmaf(w ? w[t * k + j] : 1.0f, Elt<AT>::to_f32(y[(int64_t)p * ldy + c]), acc);
            }
            if (shared) acc += Elt<AT>::to_f32(shared[(int64_t)t * ld_shared + c]);
            if (out_f32) out_f32[(int64_t)t * D + c] = acc;
            else out[(int64_t)t * ldo + c] = Elt<AT>::from_f32(acc);
        }
    }
}


// Router for few tokens (decode): logits[e] = x . Wr[e] in f32, rounded to the activation type (what
// x @ Wr^T returns there), softmax over the experts in f32, the k largest scores (ties to the lower
// id), w = p / (sum p + 1e-20) * scale  (dots3/ops.py:149-162; the plain softmax-top-k of the mlx-lm
// switch layers).  One CTA per token; warps split the experts, warp 0 selects.
constexpr int ROUTE_MAX_E = 1024;
// FUSED: the token is first formed as rms_norm(x + res) (no weight, f32, rounded to the activation type:
// residual_rmsnorm_kernel's arithmetic up to the order of the sum of squares), kept in shared memory for the
// dot products, and written to x_out by the CTAs of expert block 0 -- the residual + norm launch in front of
// the router disappears.
template <typename AT, bool FUSED>
__global__ void __launch_bounds__(256)
route_kernel(const AT* __restrict__ x, int64_t ldx, const AT* __restrict__ wr, int H, int E, int k, int renorm,
             float scale, int32_t* __restrict__ idx_out, float* __restrict__ w_out, float* __restrict__ ws_logits,
             int* __restrict__ ws_count, const AT* __restrict__ res, float eps, AT* __restrict__ x_out) {
    // grid (T, ceil(E / 8)): warp w of CTA (t, b) computes the logit of expert 8b + w; the CTA that finishes
    // last for its token (a counter, no waiting) runs the selection over all E logits
    __shared__ float p[ROUTE_MAX_E];
    __shared__ int is_last;
    __shared__ __align__(16) AT xn[FUSED ? 4096 : 8];
    __shared__ float part[8];
    pdl_enter();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.y * 8 + warp;
    uint4 wpre[FUSED ? 16 : 1];                            // FUSED: the expert's router row, requested before the norm
    if constexpr (FUSED) {
        if (e < E) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int c = lane * 8 + 256 * i;
                if (c < H) wpre[i] = __ldg(reinterpret_cast<const uint4*>(wr + (int64_t)e * H + c));
            }
        }
    }
    if constexpr (FUSED) {                                 // H <= 4096: 16 columns per thread
        float v[16];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c = threadIdx.x + i * 256;
            v[i] = 0.f;
            if (c < H) {
                v[i] = Elt<AT>::to_f32(x[(int64_t)t * ldx + c]) + Elt<AT>::to_f32(res[(int64_t)t * H + c]);
                ss = fmaf(v[i], v[i], ss);
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot += part[i];
        const float r = rsqrtf(tot / (float)H + eps);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c = threadIdx.x + i * 256;
            if (c < H) {
                const AT o = Elt<AT>::from_f32(v[i] * r);
                xn[c] = o;
                if (blockIdx.y == 0) x_out[(int64_t)t * H + c] = o;
            }
        }
        __syncthreads();
    }
    if (e < E) {
        const AT* xr = FUSED ? xn : x + (int64_t)t * ldx;
        const AT* wrow = wr + (int64_t)e * H;
        float acc = 0.f;
        auto dot8 = [&](const uint4& xv, const uint4& wv) {
            const AT* xa = reinterpret_cast<const AT*>(&xv);
            const AT* wa = reinterpret_cast<const AT*>(&wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(Elt<AT>::to_f32(xa[j]), Elt<AT>::to_f32(wa[j]), acc);
        };
        if constexpr (FUSED) {                             // H % 8 == 0, 16-byte loads
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int c = lane * 8 + 256 * i;
                if (c < H) dot8(*reinterpret_cast<const uint4*>(xr + c), wpre[i]);
            }
        } else {
            for (int c = lane * 8; c < H; c += 256)
                dot8(*reinterpret_cast<const uint4*>(xr + c), __ldg(reinterpret_cast<const uint4*>(wrow + c)));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, d);
        if (lane == 0) ws_logits[(int64_t)t * E + e] = Elt<AT>::to_f32(Elt<AT>::from_f32(acc));
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(ws_count + t, 1);
        is_last = prev == (int)gridDim.y - 1;
        if (is_last) ws_count[t] = 0;                      // left at zero for the next call
    }
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    for (int i = lane; i < E; i += 32) p[i] = __ldcg(ws_logits + (int64_t)t * E + i);
    __syncwarp();
    float mx = -INFINITY;
    for (int i = lane; i < E; i += 32) mx = fmaxf(mx, p[i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, d));
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float v = __expf(p[i] - mx);
        p[i] = v;
        sum += v;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    const float inv_sum = 1.0f / sum;
    __syncwarp();
    float top_sum = 0.f, my_w = 0.f;
    int my_idx = 0;
    for (int j = 0; j < k; ++j) {
        float bv = -1.f;
        int bi = 0x7FFFFFFF;
        for (int i = lane; i < E; i += 32) {
            const float v = p[i];
            if (v > bv) { bv = v; bi = i; }                // ascending i: the first maximum is the lowest id
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, d);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, d);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) p[bi] = -1.f;                       // taken
        __syncwarp();
        const float pv = bv * inv_sum;
        top_sum += pv;
        if (lane == j % 32) { my_w = pv; my_idx = bi; }
        if (j % 32 == 31 || j == k - 1) {                  // flush this batch of (up to 32) selections
            const int j0 = j - (j % 32);
            if (lane <= j - j0) {
                idx_out[(int64_t)t * k + j0 + lane] = my_idx;
                w_out[(int64_t)t * k + j0 + lane] = my_w;  // raw p: normalised below
            }
        }
    }
    __syncwarp();
    const float norm = renorm ? scale / (top_sum + 1e-20f) : scale;
    for (int j = lane; j < k; j += 32) w_out[(int64_t)t * k + j] *= norm;
}

// The fused router for up to 128 experts as ONE thread-block cluster per token (up to 8 CTAs x 16 experts): the
// logits meet in the shared memory of the cluster's first CTA (st.shared::cluster) and a cluster barrier replaces
// the fence + counter + re-read from global memory of route_kernel, whose hand-over costs about 2.5 us on a path
// that is a chain of dependent launches.  The router rows are requested before the dependency wait (static
// weights); x and res are read 16 bytes per thread.  Same arithmetic as route_kernel<AT, true>.
template <typename AT>
__global__ void __launch_bounds__(256)
route_cluster_kernel(const AT* __restrict__ x, const AT* __restrict__ wr, int H, int E, int k, int renorm, float scale,
                     int32_t* __restrict__ idx_out, float* __restrict__ w_out, const AT* __restrict__ res, float eps,
                     AT* __restrict__ x_out) {
    __shared__ float p[128];
    __shared__ __align__(16) AT xn[4096];
    __shared__ float part[8];
    const int t = blockIdx.x, rank = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // two experts per warp: their router rows, 8 columns per lane and 256-column step (H <= 4096: 16 steps)
    const int e0 = rank * 16 + warp * 2;
    uint4 wa[16], wb[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int c = lane * 8 + 256 * i;
        wa[i] = wb[i] = make_uint4(0u, 0u, 0u, 0u);
        if (c < H) {
            if (e0 < E) wa[i] = __ldg(reinterpret_cast<const uint4*>(wr + (int64_t)e0 * H + c));
            if (e0 + 1 < E) wb[i] = __ldg(reinterpret_cast<const uint4*>(wr + (int64_t)(e0 + 1) * H + c));
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // the token: rms_norm(x + res); thread j owns columns [8 j, 8 j + 8) and, for H > 2048, [2048 + 8 j, ...)
    float v[16];
    float ss = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int c = h * 2048 + threadIdx.x * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[h * 8 + j] = 0.f;
        if (c < H) {
            const uint4 xq = *reinterpret_cast<const uint4*>(x + (int64_t)t * H + c);
            const uint4 rq = *reinterpret_cast<const uint4*>(res + (int64_t)t * H + c);
            const AT* xa = reinterpret_cast<const AT*>(&xq);
            const AT* ra = reinterpret_cast<const AT*>(&rq);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[h * 8 + j] = Elt<AT>::to_f32(xa[j]) + Elt<AT>::to_f32(ra[j]);
                ss = fmaf(v[h * 8 + j], v[h * 8 + j], ss);
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float r = rsqrtf(tot / (float)H + eps);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int c = h * 2048 + threadIdx.x * 8;
        if (c < H) {
            uint4 oq;
            AT* oa = reinterpret_cast<AT*>(&oq);
#pragma unroll
            for (int j = 0; j < 8; ++j) oa[j] = Elt<AT>::from_f32(v[h * 8 + j] * r);
            *reinterpret_cast<uint4*>(xn + c) = oq;
            if (rank == 0) *reinterpret_cast<uint4*>(x_out + (int64_t)t * H + c) = oq;
        }
    }
    __syncthreads();
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int c = lane * 8 + 256 * i;
        if (c < H) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xn + c);
            const AT* xa = reinterpret_cast<const AT*>(&xv);
            const AT* a0 = reinterpret_cast<const AT*>(&wa[i]);
            const AT* a1 = reinterpret_cast<const AT*>(&wb[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float xf = Elt<AT>::to_f32(xa[j]);
                acc0 = fmaf(xf, Elt<AT>::to_f32(a0[j]), acc0);
                acc1 = fmaf(xf, Elt<AT>::to_f32(a1[j]), acc1);
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, d);
        acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, d);
    }
    if (lane < 2 && e0 + lane < E) {
        // the logit, rounded to the activation type, into p[] of the cluster's first CTA
        const float lv = Elt<AT>::to_f32(Elt<AT>::from_f32(lane == 0 ? acc0 : acc1));
        uint32_t local = (uint32_t)__cvta_generic_to_shared(p + e0 + lane), remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(lv) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank != 0 || warp != 0) return;
    float mx = -INFINITY;
    for (int i = lane; i < E; i += 32) mx = fmaxf(mx, p[i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, d));
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float pv = __expf(p[i] - mx);
        p[i] = pv;
        sum += pv;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    const float inv_sum = 1.0f / sum;
    __syncwarp();
    float top_sum = 0.f, my_w = 0.f;
    int my_idx = 0;
    for (int j = 0; j < k; ++j) {
        float bv = -1.f;
        int bi = 0x7FFFFFFF;
        for (int i = lane; i < E; i += 32) {
            const float pv = p[i];
            if (pv > bv) { bv = pv; bi = i; }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, d);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, d);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) p[bi] = -1.f;
        __syncwarp();
        const float pv = bv * inv_sum;
        top_sum += pv;
        if (lane == j % 32) { my_w = pv; my_idx = bi; }
        if (j % 32 == 31 || j == k - 1) {
            const int j0 = j - (j % 32);
            if (lane <= j - j0) {
                idx_out[(int64_t)t * k + j0 + lane] = my_idx;
                w_out[(int64_t)t * k + j0 + lane] = my_w;
            }
        }
    }
    __syncwarp();
    const float norm = renorm ? scale / (top_sum + 1e-20f) : scale;
    for (int j = lane; j < k; j += 32) w_out[(int64_t)t * k + j] *= norm;
}

// Router for many tokens (prefill): the logits come from a GEMM; one warp per token turns its row of logits
// (f32, or the activation type) into the softmax over the experts in f32, the k largest scores (ties to the
// lower id) and w = p / (sum p + 1e-20) * scale -- route_kernel's selection, one launch instead of the five or
// six of an eager softmax / top-k / normalise chain.  E <= 1024: a lane holds up to 32 logits in registers.
template <typename LT>
__global__ void __launch_bounds__(256)
topk_rows_kernel(const LT* __restrict__ logits, int64_t ld, int T, int E, int k, int renorm, float scale,
                 int32_t* __restrict__ idx_out, float* __restrict__ w_out) {
    const int lane = threadIdx.x & 31;
    const int t = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    if (t >= T) return;
    constexpr int PER = ROUTE_MAX_E / 32;
    float p[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        p[i] = -INFINITY;
        if (e < E) {
            if constexpr (sizeof(LT) == 4) p[i] = (float)logits[(int64_t)t * ld + e];
            else p[i] = Elt<LT>::to_f32(logits[(int64_t)t * ld + e]);
            mx = fmaxf(mx, p[i]);
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, d));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        p[i] = e < E ? __expf(p[i] - mx) : -1.f;
        if (e < E) sum += p[i];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
    const float inv_sum = 1.0f / sum;
    float top_sum = 0.f;
    for (int j = 0; j < k; ++j) {
        float bv = -1.f;
        int bi = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (p[i] > bv) { bv = p[i]; bi = lane + 32 * i; }       // ascending ids: the first maximum is the lowest id
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, d);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, d);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (bi == lane + 32 * i) p[i] = -1.f;                   // taken
        const float pv = bv * inv_sum;
        top_sum += pv;
        if (lane == 0) {
            idx_out[(int64_t)t * k + j] = bi;
            w_out[(int64_t)t * k + j] = pv;                         // raw p: normalised below
        }
    }
    __syncwarp();
    const float norm = renorm ? scale / (top_sum + 1e-20f) : scale;
    for (int j = lane; j < k; j += 32) w_out[(int64_t)t * k + j] *= norm;
}

// out[t, :] = rms_norm(x[t, :] + sum_j y[t*k + j, :]) without weight, in f32: v / sqrt(mean(v^2) + eps), rounded
// to the activation type; the k rows are added in slot order (k = 1: a plain residual).  Glue of the
// synthetic decode stacks (residual + norm between the quantized blocks; with k > 1 also the unweighted
// combine of the routed experts, whose routing weights were applied before the down projection); y is
// f32 (y_f32 != NULL, k = 1) or of the activation type.
template <typename AT>
__global__ void __launch_bounds__(1024)
residual_rmsnorm_kernel(const AT* __restrict__ x, const AT* __restrict__ y, const float* __restrict__ y_f32, int k, int H,
                        float eps, AT* __restrict__ out) {
    __shared__ float part[32];
    pdl_enter();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int PER = 4;                               // columns per thread held in registers (H <= 4096)
    float v[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * 1024;
        v[i] = 0.f;
        if (c < H) {
            float a = Elt<AT>::to_f32(x[(int64_t)t * H + c]);
            if (y_f32) a += y_f32[(int64_t)t * H + c];
            else
                for (int j = 0; j < k; ++j) a += Elt<AT>::to_f32(y[((int64_t)t * k + j) * H + c]);
            v[i] = a;
            ss = fmaf(a, a, ss);
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, d);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) tot += part[i];
    const float r = rsqrtf(tot / (float)H + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * 1024;
        if (c < H) out[(int64_t)t * H + c] = Elt<AT>::from_f32(v[i] * r);
    }
}

}  // namespace jq

extern "C" {

int jq_moe_route(const void* x, int act_dtype, int64_t ldx, int64_t T, int64_t H, const void* router_w, int num_experts,
                 int k, int renorm, float scale, int32_t* idx_out, float* w_out, int32_t* counters, float* logits_ws,
                 jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(T >= 0 && H > 0 && H % 8 == 0, JQ_EINVAL, "jq_moe_route needs H %% 8 == 0");
    JQ_REQUIRE(num_experts > 0 && num_experts <= ROUTE_MAX_E, JQ_EUNSUPPORTED, "jq_moe_route takes at most %d experts",
               ROUTE_MAX_E);
    JQ_REQUIRE(k > 0 && k <= num_experts, JQ_EINVAL, "k must be in [1, num_experts]");
    if (T == 0) return JQ_OK;
    JQ_REQUIRE(x && router_w && idx_out && w_out && counters && logits_ws, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(ldx >= H && ldx % 8 == 0 && aligned(x, 16) && aligned(router_w, 16), JQ_EINVAL,
               "x and the router weights must be 16-byte aligned with ldx %% 8 == 0");
    JQ_REQUIRE(T <= 65535, JQ_EUNSUPPORTED, "jq_moe_route is the few-token path");
    const dim3 grid((unsigned)T, (unsigned)((num_experts + 7) / 8));
    JQ_DISPATCH_DTYPE16(act_dtype, AT,
        JQ_CUDA_OK(launch_pdl(route_kernel<AT, false>, grid, dim3(256), 0, (cudaStream_t)stream, (const AT*)x, ldx,
                              (const AT*)router_w, (int)H, num_experts, k, renorm, scale, idx_out, w_out, logits_ws,
                              (int*)counters, (const AT*)nullptr, 0.f, (AT*)nullptr)))
    return JQ_OK;
}

int jq_moe_route_norm(const void* x, const void* res, int act_dtype, int64_t T, int64_t H, float eps, void* x_out,
                      const void* router_w, int num_experts, int k, int renorm, float scale, int32_t* idx_out,
                      float* w_out, int32_t* counters, float* logits_ws, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(T >= 0 && H > 0 && H % 8 == 0 && H <= 4096, JQ_EINVAL, "jq_moe_route_norm needs H %% 8 == 0, H <= 4096");
    JQ_REQUIRE(num_experts > 0 && num_experts <= ROUTE_MAX_E, JQ_EUNSUPPORTED, "jq_moe_route_norm takes at most %d experts",
               ROUTE_MAX_E);
    JQ_REQUIRE(k > 0 && k <= num_experts, JQ_EINVAL, "k must be in [1, num_experts]");
    if (T == 0) return JQ_OK;
    JQ_REQUIRE(x && res && x_out && router_w && idx_out && w_out && counters && logits_ws, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(aligned(router_w, 16), JQ_EINVAL, "the router weights must be 16-byte aligned");
    JQ_REQUIRE(T <= 65535, JQ_EUNSUPPORTED, "jq_moe_route_norm is the few-token path");
    {   // every CTA of a token re-reads x and res while the first one already writes x_out: no in-place update
        const char* o0 = (const char*)x_out;
        const char* o1 = o0 + (size_t)T * H * 2;
        const char* x0 = (const char*)x;
        const char* r0 = (const char*)res;
        const size_t nb = (size_t)T * H * 2;
        JQ_REQUIRE((o1 <= x0 || x0 + nb <= o0) && (o1 <= r0 || r0 + nb <= o0), JQ_EINVAL,
                   "jq_moe_route_norm: x_out must not overlap x or res");
    }
    if (num_experts <= 128 && aligned(x, 16) && aligned(res, 16) && aligned(x_out, 16)) {
        // one cluster of ceil(E / 16) <= 8 CTAs per token
        const unsigned cl = (unsigned)((num_experts + 15) / 16);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)T, cl);
        cfg.blockDim = dim3(256);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1; attr[1].val.clusterDim.y = cl; attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        const int Hi = (int)H;
        JQ_DISPATCH_DTYPE16(act_dtype, AT,
            JQ_CUDA_OK(cudaLaunchKernelEx(&cfg, route_cluster_kernel<AT>, (const AT*)x, (const AT*)router_w, Hi, num_experts, k,
                                          renorm, scale, idx_out, w_out, (const AT*)res, eps, (AT*)x_out)))
        return JQ_OK;
    }
    const dim3 grid((unsigned)T, (unsigned)((num_experts + 7) / 8));
    JQ_DISPATCH_DTYPE16(act_dtype, AT,
        JQ_CUDA_OK(launch_pdl(route_kernel<AT, true>, grid, dim3(256), 0, (cudaStream_t)stream, (const AT*)x, H,
                              (const AT*)router_w, (int)H, num_experts, k, renorm, scale, idx_out, w_out, logits_ws,
                              (int*)counters, (const AT*)res, eps, (AT*)x_out)))
    return JQ_OK;
}

int jq_moe_topk(const void* logits, int logits_dtype, int64_t ld, int64_t T, int num_experts, int k, int renorm, float scale,
                int32_t* idx_out, float* w_out, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(num_experts > 0 && num_experts <= ROUTE_MAX_E, JQ_EUNSUPPORTED, "jq_moe_topk takes at most %d experts", ROUTE_MAX_E);
    JQ_REQUIRE(k > 0 && k <= num_experts && T >= 0 && ld >= num_experts, JQ_EINVAL, "k in [1, num_experts], ld >= num_experts");
    JQ_REQUIRE(T < (1ll << 26), JQ_EUNSUPPORTED, "too many rows");
    if (T == 0) return JQ_OK;
    JQ_REQUIRE(logits && idx_out && w_out, JQ_EINVAL, "null pointer");
    const unsigned blocks = (unsigned)((T * 32 + 255) / 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (logits_dtype == JQ_F32)
        topk_rows_kernel<float><<<blocks, 256, 0, st>>>((const float*)logits, ld, (int)T, num_experts, k, renorm, scale, idx_out, w_out);
    else if (logits_dtype == JQ_BF16)
        topk_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)logits, ld, (int)T, num_experts, k, renorm,
                                                               scale, idx_out, w_out);
    else if (logits_dtype == JQ_F16)
        topk_rows_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)logits, ld, (int)T, num_experts, k, renorm, scale, idx_out,
                                                        w_out);
    else
        return fail(JQ_EINVAL, "logits must be f32, f16 or bf16");
    return check_launch("moe_topk");
}

int jq_residual_rmsnorm(const void* x, const void* y, const float* y_f32, int k, int64_t T, int64_t H, float eps, void* out,
                        int act_dtype, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(T >= 0 && H > 0 && H <= 4096, JQ_EUNSUPPORTED, "jq_residual_rmsnorm takes rows of at most 4096 elements");
    if (T == 0) return JQ_OK;
    JQ_REQUIRE(x && out && (y || y_f32), JQ_EINVAL, "null pointer");
    JQ_REQUIRE(k >= 1 && (y_f32 == nullptr || k == 1), JQ_EINVAL, "k >= 1; an f32 addend is a single row");
    JQ_REQUIRE(T <= 65535, JQ_EUNSUPPORTED, "at most 65535 rows");
    JQ_DISPATCH_DTYPE16(act_dtype, AT,
        JQ_CUDA_OK(launch_pdl(residual_rmsnorm_kernel<AT>, dim3((unsigned)T), dim3(1024), 0, (cudaStream_t)stream,
                              (const AT*)x, (const AT*)y, y_f32, k, (int)H, eps, (AT*)out)))
    return JQ_OK;
}


size_t jq_moe_sort_max_tiles(int64_t n_pairs, int num_experts, int tile_m) {
    if (n_pairs < 0 || num_experts < 0 || tile_m <= 0) return 0;
    return (size_t)(n_pairs / tile_m + num_experts);
}

int jq_moe_sort(const int32_t* topk_idx, int64_t n_pairs, int num_experts, int expert_base, int32_t* order,
                int32_t* inv, int32_t* expert_offsets, int tile_m, int32_t* tile_expert, int32_t* tile_row0,
                int32_t* num_tiles, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(n_pairs >= 0 && n_pairs < (1ll << 30), JQ_EINVAL, "bad pair count %lld", (long long)n_pairs);
    JQ_REQUIRE(num_experts > 0 && num_experts <= 4096, JQ_EUNSUPPORTED, "num_experts must be in 1..4096");
    JQ_REQUIRE(tile_m > 0, JQ_EINVAL, "tile_m must be positive");
    JQ_REQUIRE(order && inv && expert_offsets && tile_expert && tile_row0 && num_tiles, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(n_pairs == 0 || topk_idx, JQ_EINVAL, "null pointer");
    const size_t smem = (size_t)(SORT_WARPS + 1) * (num_experts + 1) * sizeof(int32_t);
    JQ_REQUIRE(smem <= 200 * 1024, JQ_EUNSUPPORTED, "too many experts for the single-CTA sort");
    static bool attr_done[64] = {};
    int dev = 0;
    JQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        JQ_CUDA_OK(cudaFuncSetAttribute(moe_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    if (n_pairs >= 2 * SORT_THREADS && num_experts + 1 <= SORT_THREADS) {
        // several CTAs: count, scan, place
        static bool attr2_done[64] = {};
        if (dev < 0 || dev >= 64 || !attr2_done[dev]) {
            JQ_CUDA_OK(cudaFuncSetAttribute(moe_sort_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            if (dev >= 0 && dev < 64) attr2_done[dev] = true;
        }
        const int chunks = (int)(n_pairs / SORT_THREADS);
        cudaStream_t st = (cudaStream_t)stream;
        moe_sort_count_kernel<<<chunks, SORT_THREADS, (size_t)(num_experts + 1) * sizeof(int32_t), st>>>(
            topk_idx, (int)n_pairs, num_experts, expert_base, chunks, inv);
        moe_sort_scan_kernel<<<1, SORT_THREADS, 0, st>>>(num_experts, chunks, inv, expert_offsets, tile_m, tile_expert,
                                                         tile_row0, num_tiles);
        moe_sort_place_kernel<<<chunks, SORT_THREADS, smem, st>>>(topk_idx, (int)n_pairs, num_experts, expert_base, chunks,
                                                                  order, inv);
        return check_launch("moe_sort");
    }
    moe_sort_kernel<<<1, SORT_THREADS, smem, (cudaStream_t)stream>>>(topk_idx, (int)n_pairs, num_experts, expert_base,
                                                                      order, inv, expert_offsets, tile_m, tile_expert,
                                                                      tile_row0, num_tiles);
    return check_launch("moe_sort");
}

int jq_gather_rows(const void* src, int64_t src_ld, const int32_t* order, const int32_t* count, int div, void* dst,
                   int64_t dst_ld, int64_t cols, int64_t max_rows, int dtype, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(dtype == JQ_BF16 || dtype == JQ_F16, JQ_EINVAL, "gather_rows takes 16-bit rows");
    JQ_REQUIRE(div > 0 && cols >= 0 && max_rows >= 0, JQ_EINVAL, "bad argument");
    if (max_rows == 0 || cols == 0) return JQ_OK;
    JQ_REQUIRE(src && dst && order && count, JQ_EINVAL, "null pointer");
    JQ_REQUIRE(cols % 8 == 0 && src_ld % 8 == 0 && dst_ld % 8 == 0 && aligned(src, 16) && aligned(dst, 16), JQ_EINVAL,
               "gather_rows needs 16-byte aligned rows");
    const int blocks = (int)(max_rows < 4 * 148 ? max_rows : 4 * 148);
    gather_rows_kernel<<<blocks, 128, 0, (cudaStream_t)stream>>>((const uint4*)src, src_ld / 8, order, count, div,
                                                                  (uint4*)dst, dst_ld / 8, (int)(cols / 8), (int)max_rows);
    return check_launch("gather_rows");
}

int jq_moe_swiglu(const void* gate, const void* up, int64_t ld_in, const float* weights, const int32_t* order,
                  const int32_t* count, void* h, int64_t ld_out, int64_t cols, int64_t max_rows, float limit, int dtype,
                  jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(max_rows >= 0 && cols >= 0, JQ_EINVAL, "bad argument");
    if (max_rows == 0 || cols == 0) return JQ_OK;
    JQ_REQUIRE(gate && up && h, JQ_EINVAL, "null pointer");
    const int blocks = (int)(max_rows < 8 * 148 ? max_rows : 8 * 148);
    JQ_DISPATCH_DTYPE16(dtype, T,
        JQ_CUDA_OK(launch_pdl(swiglu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)gate,
                              (const T*)up, ld_in, weights, order, count, (T*)h, ld_out, (int)cols, (int)max_rows, limit)))
    return JQ_OK;
}

int jq_moe_combine_shared(const void* y, int64_t ldy, const int32_t* inv, const float* weights, int64_t T, int k,
                          int64_t D, const void* shared_y, int64_t ld_shared, void* out, int64_t ldo, float* out_f32,
                          int dtype, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(T >= 0 && k > 0 && D >= 0, JQ_EINVAL, "bad argument");
    if (T == 0 || D == 0) return JQ_OK;
    JQ_REQUIRE(y && (out || out_f32), JQ_EINVAL, "null pointer");
    JQ_REQUIRE(shared_y == nullptr || ld_shared >= D, JQ_EINVAL, "leading dimension of the shared expert's rows too small");
    const int blocks = (int)(T < 8 * 148 ? T : 8 * 148);
    JQ_DISPATCH_DTYPE16(dtype, A,
        (combine_kernel<A><<<blocks, 256, 0, (cudaStream_t)stream>>>((const A*)y, ldy, inv, weights, (int)T, k, (int)D,
                                                                      (A*)out, ldo, out_f32, (const A*)shared_y,
                                                                      ld_shared)))
    return check_launch("moe_combine");
}

int jq_moe_combine(const void* y, int64_t ldy, const int32_t* inv, const float* weights, int64_t T, int k, int64_t D,
                   void* out, int64_t ldo, float* out_f32, int dtype, jq_stream_t stream) {
    return jq_moe_combine_shared(y, ldy, inv, weights, T, k, D, nullptr, 0, out, ldo, out_f32, dtype, stream);
}

}  // extern "C"
