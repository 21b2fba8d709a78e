// Error plumbing, device queries and launch accounting of the C ABI.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <cstdlib>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

bool pdl_enabled() {
    static const int v = [] {
        const char *e = getenv("B200_PDL");
        return (e && atoi(e) == 0) ? 0 : 1;
    }();
    return v == 1;
}

int pdl_early_rows() {
    static const int v = [] {
        const char *e = getenv("B200_PDL_EARLY_ROWS");
        return e ? atoi(e) : 1;
    }();
    return v;
}

void count_launch(int n) { g_launches.fetch_add((uint64_t) n, std::memory_order_relaxed); }

int check_launch(const char *what) {
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(B200_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_abi_version(void) { return B200_ABI_VERSION; }

const char *b200_last_error(void) { return b200::g_err; }

uint64_t b200_launch_count(void) { return b200::g_launches.load(); }

int b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ok = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ok++;
    }
    return ok == n ? n : 0;  // every visible device must be sm_100: the kernels are built for nothing else
}

int b200_device_info(int device, char *name, size_t name_len, size_t *free_bytes, size_t *total_bytes, int *sm_count) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return b200::set_error(B200_E_NODEVICE, "no CUDA device %d", device);
    if (name && name_len) {
        strncpy(name, p.name, name_len - 1);
        name[name_len - 1] = 0;
    }
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (free_bytes || total_bytes) {
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(device);
        size_t f = 0, t = 0;
        cudaError_t e = cudaMemGetInfo(&f, &t);
        cudaSetDevice(cur);
        if (e != cudaSuccess) return b200::set_error(B200_E_CUDA, "cudaMemGetInfo: %s", cudaGetErrorString(e));
        if (free_bytes) *free_bytes = f;
        if (total_bytes) *total_bytes = t;
    }
    return B200_OK;
}

}  // extern "C"
