// Library-wide plumbing: version, status strings, per-thread error text,
// shape validation shared by every entry point.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "jq_common.cuh"

namespace jq {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

int check_quant_shape(int64_t rows, int64_t K, int bits, int group_size) {
    JQ_REQUIRE(valid_bits(bits), JQ_EUNSUPPORTED, "unsupported bits=%d (allowed 2,3,4,5,6,8)", bits);
    JQ_REQUIRE(valid_gs(group_size), JQ_EUNSUPPORTED, "unsupported group_size=%d (allowed 32,64,128)",
               group_size);
    JQ_REQUIRE(rows >= 0 && K >= 0, JQ_EINVAL, "negative shape rows=%lld K=%lld", (long long)rows,
               (long long)K);
    JQ_REQUIRE(K % group_size == 0, JQ_EINVAL, "input dimension %lld is not divisible by group_size=%d",
               (long long)K, group_size);
    JQ_REQUIRE((K * bits) % 32 == 0, JQ_EINVAL, "packed row is not uint32-aligned: columns=%lld, bits=%d",
               (long long)K, bits);
    return JQ_OK;
}

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    static bool have[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lk(mu);
    if (!have[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
        have[dev] = true;
    }
    return cached[dev];
}

}  // namespace jq

extern "C" {

int jq_version(void) { return 100; }

const char* jq_status_string(int status) {
    switch (status) {
        case JQ_OK: return "ok";
        case JQ_EINVAL: return "invalid argument";
        case JQ_EUNSUPPORTED: return "unsupported configuration";
        case JQ_EWORKSPACE: return "workspace too small";
        case JQ_ECUDA: return "CUDA error";
        case JQ_ETIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

const char* jq_last_error(void) { return jq::g_err; }

}  // extern "C"
