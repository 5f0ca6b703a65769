// Status strings, thread-local error text and device queries of the bsi_b200 library.
#include "common.cuh"

#include <stdlib.h>

#include <stdarg.h>

#include <mutex>
#include <unordered_map>

namespace bsi {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

bool pdl_enabled() {
    static int cached = -1;
    if (cached < 0) {
        const char* e = getenv("BSI_B200_PDL");
        cached = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return cached == 1;
}

namespace {
std::mutex g_bounds_mu;
std::unordered_map<const void*, KeyBounds> g_bounds;
std::unordered_map<const void*, QueryBounds> g_query_bounds;
}  // namespace

bool lookup_query_bounds(const void* a8, QueryBounds* out) {
    std::lock_guard<std::mutex> lock(g_bounds_mu);
    auto it = g_query_bounds.find(a8);
    if (it == g_query_bounds.end()) return false;
    *out = it->second;
    return true;
}

bool lookup_key_bounds(const void* k8, KeyBounds* out) {
    const char* e = getenv("BSI_B200_EXACT_INT");      // 0 switches the integer accumulation off (A/B comparisons)
    if (e != nullptr && e[0] == '0') return false;
    std::lock_guard<std::mutex> lock(g_bounds_mu);
    auto it = g_bounds.find(k8);
    if (it == g_bounds.end()) return false;
    *out = it->second;
    return true;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int require_sm100() {
    static int cached[64] = {0};  // 0 unknown, 1 ok, 2 not sm_100
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        set_error("cudaGetDevice: %s", cudaGetErrorString(e));
        return BSI_ERR_CUDA;
    }
    if (dev < 0 || dev >= 64) return BSI_OK;
    if (cached[dev] == 0) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) {
            set_error("cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
            return BSI_ERR_CUDA;
        }
        cached[dev] = (major == 10) ? 1 : 2;
    }
    if (cached[dev] != 1) {
        set_error("bsi_b200 kernels are built for sm_100a only; current device is not compute capability 10.x");
        return BSI_ERR_DEVICE;
    }
    return BSI_OK;
}

}  // namespace bsi

extern "C" const char* bsi_b200_status_string(int status) {
    switch (status) {
        case BSI_OK: return "ok";
        case BSI_ERR_INVALID: return "invalid argument";
        case BSI_ERR_UNSUPPORTED: return "unsupported request";
        case BSI_ERR_CUDA: return "CUDA call failed";
        case BSI_ERR_DEVICE: return "not an sm_100 device";
        case BSI_ERR_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

extern "C" const char* bsi_b200_last_error(void) { return bsi::g_err; }

extern "C" int bsi_b200_version(void) { return BSI_B200_VERSION; }

extern "C" int bsi_b200_register_key_bounds(const int8_t* k8, const float* key_abs_sum, int64_t R, int query_abs_max) {
    using namespace bsi;
    if (k8 == nullptr || key_abs_sum == nullptr || R <= 0 || query_abs_max <= 0 || query_abs_max > 128) {
        set_error("register_key_bounds: bad argument");
        return BSI_ERR_INVALID;
    }
    std::lock_guard<std::mutex> lock(g_bounds_mu);
    g_bounds[k8] = KeyBounds{key_abs_sum, R, static_cast<float>(query_abs_max)};
    return BSI_OK;
}

extern "C" int bsi_b200_unregister_key_bounds(const int8_t* k8) {
    using namespace bsi;
    std::lock_guard<std::mutex> lock(g_bounds_mu);
    g_bounds.erase(k8);
    return BSI_OK;
}

extern "C" int bsi_b200_register_query_bounds(const int8_t* a8, const float* sq_norms, int64_t stride) {
    using namespace bsi;
    if (a8 == nullptr || sq_norms == nullptr || stride <= 0) {
        set_error("register_query_bounds: bad argument");
        return BSI_ERR_INVALID;
    }
    std::lock_guard<std::mutex> lock(g_bounds_mu);
    g_query_bounds[a8] = QueryBounds{sq_norms, stride};
    return BSI_OK;
}

extern "C" int bsi_b200_unregister_query_bounds(const int8_t* a8) {
    using namespace bsi;
    std::lock_guard<std::mutex> lock(g_bounds_mu);
    g_query_bounds.erase(a8);
    return BSI_OK;
}
