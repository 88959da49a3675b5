// Error reporting, dtype table, device properties.
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace dx {

static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

bool pdl_enabled() {
    static const bool on = [] { const char *e = std::getenv("DX_PDL"); return !(e && e[0] == '0'); }();
    return on;
}

int check_launch(const char *what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DX_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return DX_OK;
}

int sm_count() {
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] { std::memset(cached, 0, sizeof(cached)); });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace dx

extern "C" const char *dx_last_error(void) { return dx::g_err; }

extern "C" int dx_dtype_size(int dtype) {
    switch (dtype) {
        case DX_F64: case DX_I64: return 8;
        case DX_F32: case DX_I32: return 4;
        case DX_F16: case DX_BF16: case DX_I16: return 2;
        case DX_I8: case DX_BOOL: return 1;
        default: return 0;
    }
}

extern "C" int dx_sm_count(void) { return dx::sm_count(); }

extern "C" unsigned long long dx_launch_count(void) { return dx::g_launches.load(std::memory_order_relaxed); }
