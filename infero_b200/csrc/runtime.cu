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

// Multiprocessors of the current device (asked once per device; the B200's 148 if the query fails).
int infero_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        cached[dev] = sms;
    }
    return cached[dev];
}

// How decode attention cuts the keys of a step into splits: (keys per split, number of splits) such
// that the splits cover max_visible keys and the grid of n_tok x n_kv x ceil(group / 16) x splits CTAs
// has about two CTAs per multiprocessor; a split has at least INFERO_DECODE_MIN_CHUNK keys (256) and
// there are at most 256 splits (the merge keeps one weight per split in shared memory).  The one
// statement of the plan: the Python parts, the native launcher of a block and the scratch sizing all
// call this.
void infero_attn_plan_decode(int n_tok, int n_kv, int group, int max_visible, int sm_count, int* chunk, int* splits) {
    static int min_chunk = -1;
    if (min_chunk < 0) {
        const char* e = getenv("INFERO_DECODE_MIN_CHUNK");
        min_chunk = e && atoi(e) > 0 ? atoi(e) : 256;
    }
    const int target = 2 * (sm_count > 0 ? sm_count : infero_sm_count()), max_splits = 256;
    const int per_split = n_tok * n_kv * ((group + 15) / 16) > 0 ? n_tok * n_kv * ((group + 15) / 16) : 1;
    const int want = target / per_split > 0 ? target / per_split : 1;
    if (max_visible < 16) max_visible = 16;
    int c = (max_visible + want - 1) / want;
    c = (c + 15) / 16 * 16;
    if (c < min_chunk) c = min_chunk;
    int sp = (max_visible + c - 1) / c;
    if (sp > max_splits) {
        c = ((max_visible + max_splits - 1) / max_splits + 15) / 16 * 16;
        sp = (max_visible + c - 1) / c;
    }
    *chunk = c;
    *splits = sp;
}

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
