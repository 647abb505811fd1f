// Shared helpers for the jangq_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jangq_b200.h"

namespace jq {

// ---- host-side error plumbing ------------------------------------------------
void set_error(const char* fmt, ...);
int  fail(int status, const char* fmt, ...);   // records the message, returns status

#define JQ_REQUIRE(cond, status, ...)                     \
    do {                                                  \
        if (!(cond)) return ::jq::fail((status), __VA_ARGS__); \
    } while (0)

#define JQ_CUDA_OK(expr)                                                          \
    do {                                                                          \
        cudaError_t e__ = (expr);                                                 \
        if (e__ != cudaSuccess)                                                   \
            return ::jq::fail(JQ_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(JQ_ECUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    return JQ_OK;
}

inline bool valid_bits(int b) { return b == 2 || b == 3 || b == 4 || b == 5 || b == 6 || b == 8; }
inline bool valid_gs(int g) { return g == 32 || g == 64 || g == 128; }
inline bool valid_dtype(int d) { return d == JQ_F32 || d == JQ_F16 || d == JQ_BF16; }
inline size_t dtype_size(int d) { return d == JQ_F32 ? 4 : 2; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int check_quant_shape(int64_t rows, int64_t K, int bits, int group_size);

// cached per-device attributes (SM count); mutex-guarded, filled on first use
int sm_count();

// device address of the library's status word on the current device (nullptr on failure).
// Kernels with bounded waits OR a bit into it when a wait runs out; jq_device_status() reads it.
//   JQ_STATUS_LOCAL_WAIT  a wait inside one kernel's own pipeline (mbarrier, grid barrier) ran out
//   JQ_STATUS_PEER_WAIT   a rank of the expert-parallel exchange did not arrive; only this bit makes
//                         later exchange launches skip their cross-rank wait
constexpr int JQ_STATUS_LOCAL_WAIT = 1;
constexpr int JQ_STATUS_PEER_WAIT = 2;
int* status_word();

// ---- device-side scalar conversion -------------------------------------------
template <typename T> struct Elt;
template <> struct Elt<float> {
    static constexpr int id = JQ_F32;
    __device__ static __forceinline__ float to_f32(float v) { return v; }
    __device__ static __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elt<__half> {
    static constexpr int id = JQ_F16;
    __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elt<__nv_bfloat16> {
    static constexpr int id = JQ_BF16;
    __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// Call f.template operator()<T>() with the element type named by a JQ_* dtype id.
#define JQ_DISPATCH_DTYPE(id, T, ...)                              \
    switch (id) {                                                  \
        case JQ_F32:  { using T = float;          __VA_ARGS__; break; } \
        case JQ_F16:  { using T = __half;         __VA_ARGS__; break; } \
        case JQ_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; } \
        default: return ::jq::fail(JQ_EINVAL, "bad dtype id %d", (int)(id)); \
    }

#define JQ_DISPATCH_DTYPE16(id, T, ...)                            \
    switch (id) {                                                  \
        case JQ_F16:  { using T = __half;         __VA_ARGS__; break; } \
        case JQ_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; } \
        default: return ::jq::fail(JQ_EINVAL, "dtype id %d must be f16 or bf16 here", (int)(id)); \
    }

#define JQ_DISPATCH_BITS(bits, B, ...)                             \
    switch (bits) {                                                \
        case 2: { constexpr int B = 2; __VA_ARGS__; break; }       \
        case 3: { constexpr int B = 3; __VA_ARGS__; break; }       \
        case 4: { constexpr int B = 4; __VA_ARGS__; break; }       \
        case 5: { constexpr int B = 5; __VA_ARGS__; break; }       \
        case 6: { constexpr int B = 6; __VA_ARGS__; break; }       \
        case 8: { constexpr int B = 8; __VA_ARGS__; break; }       \
        default: return ::jq::fail(JQ_EUNSUPPORTED, "bits=%d", (int)(bits)); \
    }

}  // namespace jq
