// Expert-parallel decode, the exchange step fused with its consumer: sum of the ranks' partial expert
// outputs over NVLink peer memory + residual + RMS norm, one launch per layer and no library collective.
//
// Every rank holds the same tokens x[T,H] (replicated decode, jangq_b200/stacks.py) and the outputs of
// its own experts for them, y[T*k,H] (rows of pairs routed to other ranks' experts are zero).  CTA t of
// rank r:
//   1. sums its k slot rows of token t in f32 and PUSHES the row into row [t][r] of every rank's symmetric
//      buffer, its own included (plain stores over NVLink, posted; half s & 1 of a double buffer, s = the
//      launch's sequence number from a device counter);
//   2. release: writes s into flag [t][r] of every peer's buffer (st.release.sys after a system fence);
//   3. acquire: waits until its own flags [t][0..world) are >= s (ld.acquire.sys, bounded by a wall-clock
//      limit, after which the library's status word is set, the CTA carries on without hanging and no
//      later launch waits again);
//   4. reads rows [t][0..world) of its OWN buffer in rank order (the same order on every rank, so the
//      replicated x stays bit-identical), adds x, normalises, writes out[t].  The exchange crosses NVLink once
//      (stores and flags one way) instead of twice (flags, then loads and their replies).
// Double buffering needs no second barrier: a rank writes into half s & 1 of its peers only in launch s + 2,
// which it enters after launch s + 1, whose flags every peer sends only after it finished reading in launch s.
// Bytes over NVLink per rank and layer: (world - 1) * T * H * 4 written + (world - 1) * T * 4 of flags.
//
// The peers' buffers are plain device pointers (obtained by the caller, e.g. from torch's symmetric
// memory rendezvous); there is no TMA and no multicast in this file.
#include <cstdlib>

#include "jq_common.cuh"

namespace jq {

constexpr int EP_MAX_WORLD = 16;
constexpr int EP_PER = 4;                                // columns per thread (H <= 4096)
constexpr unsigned long long EP_WAIT_NS = 2000000000ull; // 2 s unless JANGQ_EP_WAIT_MS says otherwise

struct EpPeers {
    float* buf[EP_MAX_WORLD];       // [2][tcap][EP_MAX_WORLD][H] f32 (row of token t from rank r), then flags [tcap][EP_MAX_WORLD] u32
};

__device__ __forceinline__ unsigned long long ep_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void ep_store_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ep_load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ep_load_peer(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

// grid (T, ranks_in_launch): ranks_in_launch is 1 in production (rank = rank0) and the world size when one
// GPU plays every rank in a single cooperative launch (tests): then blockIdx.y is the rank and x, y, out,
// counters advance by their per-rank strides.
template <typename AT>
__global__ void __launch_bounds__(1024)
ep_combine_rmsnorm_kernel(const AT* __restrict__ x, const AT* __restrict__ y, int k, int H, float eps,
                          AT* __restrict__ out, EpPeers peers, int rank0, int world, int tcap, int32_t* counters,
                          int64_t x_rank_stride, int64_t y_rank_stride, int64_t ctr_rank_stride, int* status,
                          unsigned long long wait_ns) {
    __shared__ float part[32];
    __shared__ uint32_t seq_sh;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = blockIdx.x, rank = rank0 + (int)blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    x += (int64_t)blockIdx.y * x_rank_stride;
    out += (int64_t)blockIdx.y * x_rank_stride;
    y += (int64_t)blockIdx.y * y_rank_stride;
    counters += (int64_t)blockIdx.y * ctr_rank_stride;
    if (threadIdx.x == 0) seq_sh = (uint32_t)(++counters[t]);   // only this CTA touches counters[t]; launches are stream-ordered
    __syncthreads();
    const uint32_t s = seq_sh;
    const size_t half = (size_t)(s & 1u) * tcap * EP_MAX_WORLD * H;
    const size_t flags_off = (size_t)2 * tcap * EP_MAX_WORLD * H;       // in floats

    // 1. this rank's partial row, PUSHED into every rank's buffer (plain stores over NVLink, posted): the readers
    //    then find all rows in their own memory and the exchange costs one NVLink crossing instead of two
    const size_t my_row = half + ((size_t)t * EP_MAX_WORLD + rank) * H;
#pragma unroll
    for (int i = 0; i < EP_PER; ++i) {
        const int c = threadIdx.x + i * 1024;
        if (c < H) {
            float a = 0.f;
            for (int j = 0; j < k; ++j) a += Elt<AT>::to_f32(y[((int64_t)t * k + j) * H + c]);
            for (int p = 0; p < world; ++p) peers.buf[p][my_row + c] = a;
        }
    }
    __syncthreads();
    // 2. + 3. one thread per peer
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        __threadfence_system();
        uint32_t* theirs = reinterpret_cast<uint32_t*>(peers.buf[p] + flags_off) + (size_t)t * EP_MAX_WORLD + rank;
        ep_store_release_sys(theirs, s);
        const uint32_t* own = reinterpret_cast<const uint32_t*>(peers.buf[rank] + flags_off) + (size_t)t * EP_MAX_WORLD + p;
        const unsigned long long t0 = ep_now_ns();
        // after a peer failed to arrive once, no launch waits for peers again until the word is cleared
        bool ok = (*reinterpret_cast<volatile int*>(status) & JQ_STATUS_PEER_WAIT) == 0;
        while (ok && (int32_t)(ep_load_acquire_sys(own) - s) < 0) {
            __nanosleep(100);
            if (ep_now_ns() - t0 > wait_ns) ok = false;
        }
        if (!ok) atomicOr(status, JQ_STATUS_PEER_WAIT);
    }
    __syncthreads();
    // 4. sum in rank order + residual + RMS norm
    float v[EP_PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < EP_PER; ++i) {
        const int c = threadIdx.x + i * 1024;
        v[i] = 0.f;
        if (c < H) {
            float a = 0.f;                                 // rank order: the same x on every rank, bit for bit
            for (int p = 0; p < world; ++p)
                a += ep_load_peer(peers.buf[rank] + half + ((size_t)t * EP_MAX_WORLD + p) * H + c);
            a += Elt<AT>::to_f32(x[(int64_t)t * H + c]);
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
    for (int i = 0; i < EP_PER; ++i) {
        const int c = threadIdx.x + i * 1024;
        if (c < H) out[(int64_t)t * H + c] = Elt<AT>::from_f32(v[i] * r);
    }
}

// ---- sharded-token dispatch: rows into fixed-capacity slots per destination rank ------------------------------
// Slot row layout (row_bytes = H * 2 + 16): the H activation values, then int32 local expert id (-1: empty slot),
// float32 routing weight, 8 spare bytes.  ep_fill marks every slot empty and clears the per-destination
// counters; ep_pack gives pair p (token p / k, slot p % k) the next free slot of its destination rank
// (an atomic counter: the order of the slots inside a destination is whatever the launch makes it, which no
// result depends on -- every slot row is computed on its own and each token adds its k slots in slot order) and
// copies the row there; a pair that finds its destination full sets the overflow word and gets slot -1.
__global__ void ep_fill_kernel(uint8_t* __restrict__ send, int64_t row_bytes, int64_t slots, int H2,
                               int32_t* __restrict__ counters, int world, int32_t* __restrict__ overflow) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < slots) *reinterpret_cast<int32_t*>(send + i * row_bytes + H2) = -1;
    if (i < world) counters[i] = 0;
    if (i == 0) *overflow = 0;
}

__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint8_t* __restrict__ x, int64_t x_row_bytes, const int32_t* __restrict__ idx,
               const float* __restrict__ w, int64_t P, int k, int H2, int e_local, int world, int cap,
               uint8_t* __restrict__ send, int64_t row_bytes, int32_t* __restrict__ counters,
               int32_t* __restrict__ slot_of_pair, int32_t* __restrict__ overflow) {
    const int lane = threadIdx.x & 31;
    const int64_t p = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;      // one warp per pair
    if (p >= P) return;
    const int e = idx[p];
    int dest = e / e_local;
    dest = dest < 0 ? 0 : (dest >= world ? world - 1 : dest);
    int s = 0;
    if (lane == 0) {
        s = atomicAdd(counters + dest, 1);
        if (s >= cap) { atomicExch(overflow, 1); s = -1; }
        slot_of_pair[p] = s < 0 ? -1 : dest * cap + s;
    }
    s = __shfl_sync(0xFFFFFFFFu, s, 0);
    if (s < 0) return;
    uint8_t* dst = send + ((int64_t)dest * cap + s) * row_bytes;
    const uint8_t* src = x + (p / k) * x_row_bytes;
    for (int c = lane * 16; c < H2; c += 512) *reinterpret_cast<uint4*>(dst + c) = __ldg(reinterpret_cast<const uint4*>(src + c));
    if (lane == 0) {
        *reinterpret_cast<int32_t*>(dst + H2) = e - dest * e_local;
        *reinterpret_cast<float*>(dst + H2 + 4) = w[p];
    }
}

}  // namespace jq

extern "C" {

int jq_ep_pack_slots(const void* x, int64_t ldx, const int32_t* idx, const float* w, int64_t T, int k, int64_t H,
                     int num_experts, int world, int64_t capacity, void* send, int32_t* slot_of_pair,
                     int32_t* counters, int32_t* overflow, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(T >= 0 && k >= 1 && H > 0 && H % 8 == 0 && ldx >= H && ldx % 8 == 0, JQ_EINVAL,
               "rows of a multiple of 8 16-bit values");
    JQ_REQUIRE(world >= 1 && num_experts >= world && num_experts % world == 0, JQ_EINVAL, "experts must shard evenly");
    JQ_REQUIRE(capacity >= 1 && capacity * world < (1ll << 31) && T * k < (1ll << 31), JQ_EINVAL, "bad capacity");
    JQ_REQUIRE(send && slot_of_pair && counters && overflow && (T == 0 || (x && idx && w)), JQ_EINVAL, "null pointer");
    JQ_REQUIRE(aligned(x, 16) && aligned(send, 16), JQ_EINVAL, "x and the send buffer must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t slots = capacity * world, row_bytes = H * 2 + 16, P = T * k;
    ep_fill_kernel<<<(unsigned)((slots + 255) / 256), 256, 0, st>>>((uint8_t*)send, row_bytes, slots, (int)(H * 2), counters,
                                                                    world, overflow);
    int rc = check_launch("ep_fill");
    if (rc != JQ_OK || P == 0) return rc;
    ep_pack_kernel<<<(unsigned)((P * 32 + 255) / 256), 256, 0, st>>>((const uint8_t*)x, ldx * 2, idx, w, P, k, (int)(H * 2),
                                                                     num_experts / world, world, (int)capacity,
                                                                     (uint8_t*)send, row_bytes, counters, slot_of_pair,
                                                                     overflow);
    return check_launch("ep_pack");
}

size_t jq_ep_buffer_bytes(int64_t tcap, int64_t H) {
    if (tcap <= 0 || H <= 0) return 0;
    return (size_t)2 * tcap * jq::EP_MAX_WORLD * H * sizeof(float) + (size_t)tcap * jq::EP_MAX_WORLD * sizeof(uint32_t);
}

int jq_ep_combine_residual_rmsnorm(const void* x, const void* y, int k, int64_t T, int64_t H, float eps, void* out,
                                   int act_dtype, const uint64_t* peer_bufs, int rank, int world, int64_t tcap,
                                   int32_t* counters, int emulate_ranks, jq_stream_t stream) {
    using namespace jq;
    JQ_REQUIRE(act_dtype == JQ_BF16 || act_dtype == JQ_F16, JQ_EINVAL, "16-bit activations only");
    JQ_REQUIRE(T >= 0 && T <= tcap && H > 0 && H <= EP_PER * 1024 && k >= 1, JQ_EINVAL, "bad shape (T <= tcap, H <= 4096)");
    JQ_REQUIRE(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world, JQ_EINVAL, "bad rank/world");
    JQ_REQUIRE(emulate_ranks == 0 || (emulate_ranks == world && rank == 0), JQ_EINVAL,
               "emulation runs every rank of the world in one launch");
    if (T == 0) return JQ_OK;
    JQ_REQUIRE(x && y && out && peer_bufs && counters, JQ_EINVAL, "null pointer");
    EpPeers peers = {};
    for (int p = 0; p < world; ++p) {
        JQ_REQUIRE(peer_bufs[p] != 0 && peer_bufs[p] % 16 == 0, JQ_EINVAL, "peer buffer %d is null or unaligned", p);
        peers.buf[p] = reinterpret_cast<float*>(peer_bufs[p]);
    }
    int* status = status_word();
    JQ_REQUIRE(status != nullptr, JQ_ECUDA, "could not locate the device status word");
    const int ranks = emulate_ranks ? world : 1;
    const int k_i = k, H_i = (int)H, rank_i = rank, world_i = world, tcap_i = (int)tcap;
    const int64_t xs = emulate_ranks ? T * H : 0, ys = emulate_ranks ? T * k * H : 0, cs = emulate_ranks ? tcap : 0;
    unsigned long long wait_ns = EP_WAIT_NS;
    if (const char* e = getenv("JANGQ_EP_WAIT_MS")) {
        const long ms = atol(e);
        if (ms > 0 && ms <= 60000) wait_ns = (unsigned long long)ms * 1000000ull;
    }
    int rc = JQ_OK;
    JQ_DISPATCH_DTYPE16(act_dtype, AT, {
        const AT* xp = (const AT*)x;
        const AT* yp = (const AT*)y;
        AT* op = (AT*)out;
        void* args[] = {(void*)&xp, (void*)&yp, (void*)&k_i, (void*)&H_i, (void*)&eps, (void*)&op, (void*)&peers,
                        (void*)&rank_i, (void*)&world_i, (void*)&tcap_i, (void*)&counters, (void*)&xs, (void*)&ys,
                        (void*)&cs, (void*)&status, (void*)&wait_ns};
        const dim3 grid((unsigned)T, (unsigned)ranks);
        if (emulate_ranks) {
            // the ranks' CTAs wait on one another: a cooperative launch guarantees that they are co-resident
            JQ_REQUIRE((int64_t)T * ranks <= sm_count(), JQ_EINVAL, "emulation needs T * world <= number of SMs");
            JQ_CUDA_OK(cudaLaunchCooperativeKernel((const void*)ep_combine_rmsnorm_kernel<AT>, grid, dim3(1024), args, 0,
                                                   (cudaStream_t)stream));
        } else {
            // CTA t waits for CTA t of every peer: all T CTAs must be resident at once on every rank, or the
            // order in which the ranks' GPUs start their blocks decides whether the waits can finish
            int per_sm = 0;
            JQ_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ep_combine_rmsnorm_kernel<AT>, 1024, 0));
            JQ_REQUIRE(T <= (int64_t)per_sm * sm_count(), JQ_EUNSUPPORTED,
                       "T=%lld exceeds the %lld CTAs of this kernel one GPU holds at a time", (long long)T,
                       (long long)per_sm * sm_count());
            JQ_CUDA_OK(cudaLaunchKernel((const void*)ep_combine_rmsnorm_kernel<AT>, grid, dim3(1024), args, 0,
                                        (cudaStream_t)stream));
        }
    })
    return rc;
}

}  // extern "C"
