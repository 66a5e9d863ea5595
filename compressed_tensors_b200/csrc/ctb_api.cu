// Library-wide host state: version, thread-local error text, launch counter, device properties.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "ctb_common.cuh"

namespace ctb {

static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int after_launch(const char *what) {
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(CTB_ECUDA, "%s: %s", what, cudaGetErrorString(e));
    return CTB_OK;
}

int sm_count() {
    // one cached value per device index
    static std::atomic<int> cached[64];  // zero-initialised; two threads racing on a first call store the same value
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace ctb

extern "C" const char *ctb_version(void) { return "ctb200 0.1.0 (sm_100a)"; }
extern "C" const char *ctb_last_error_string(void) { return ctb::g_err; }
extern "C" int64_t ctb_launch_count(void) { return ctb::g_launches.load(); }

// ---- page-locked host memory for the staging buffers of the host <-> device pipeline ---------------------------
// Plain wrappers over cudaHostAlloc / cudaFreeHost (portable: page-locked for every context of the process), so
// that the host layer can keep its own pool of staging blocks and decide itself when one is reused.
extern "C" int ctb_pinned_alloc(int64_t nbytes, void **out) {
    if (!out || nbytes <= 0) return ctb::fail(CTB_EINVAL_NULL, "ctb_pinned_alloc needs a size and a place for the pointer");
    void *p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, (size_t)nbytes, cudaHostAllocPortable);
    if (e != cudaSuccess) return ctb::fail(CTB_ECUDA, "cudaHostAlloc(%lld): %s", (long long)nbytes, cudaGetErrorString(e));
    *out = p;
    return CTB_OK;
}

extern "C" int ctb_pinned_free(void *p) {
    if (!p) return CTB_OK;
    cudaError_t e = cudaFreeHost(p);
    if (e != cudaSuccess) return ctb::fail(CTB_ECUDA, "cudaFreeHost: %s", cudaGetErrorString(e));
    return CTB_OK;
}
