// Error record shared by every launcher, and small device queries.
#include "common.cuh"
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include <atomic>

static thread_local char g_error[1024] = {0};
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_pdl{-1};

// Programmatic dependent launch is on unless INFERO_PDL=0 (or infero_set_pdl(0)).
int infero_pdl_enabled() {
    int v = g_pdl.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("INFERO_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
        g_pdl.store(v, std::memory_order_relaxed);
    }
    return v;
}

void infero_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// Launch errors only (invalid configuration and the like); asynchronous faults surface
// at the caller's next synchronisation.
int infero_check_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        infero_set_error("%s: %s", what, cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

extern "C" {

const char* infero_last_error() { return g_error; }

int infero_abi_version() { return 1; }

// Kernels launched by this library since it was loaded (one per successful or failed launch
// check; a launch recorded into a CUDA graph counts once, at capture).
void infero_set_pdl(int on) { g_pdl.store(on ? 1 : 0, std::memory_order_relaxed); }

long long infero_launch_count() { return g_launches.load(std::memory_order_relaxed); }

int infero_device_info(int device, int* sm_count, int* cc_major, int* cc_minor, int* smem_optin) {
    cudaDeviceProp p;
    cudaError_t e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) {
        infero_set_error("device_info: %s", cudaGetErrorString(e));
        return 1;
    }
    *sm_count = p.multiProcessorCount;
    *cc_major = p.major;
    *cc_minor = p.minor;
    *smem_optin = (int)p.sharedMemPerBlockOptin;
    return 0;
}

}  // extern "C"
