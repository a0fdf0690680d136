// infero_attn_decode_static: decode attention whose split-context scratch is a fixed array
// in this library, for callers that cannot allocate device memory (see no_alloc.h).
#include "common.cuh"
#include "no_alloc.h"
#include <mutex>

extern "C" int infero_attn_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                                  const void* v_cache, const int* block_table, int max_blocks, const int* tok_entry,
                                  const int* positions, int tok_first, int n_tok, int n_heads, int n_kv,
                                  int head_dim, int page_size, int window, float scale, int chunk, int n_splits,
                                  void* scratch, cudaStream_t stream);
extern "C" long long infero_attn_decode_scratch(int n_tok, int n_heads, int head_dim, int n_splits);

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's symbol
// calls, never a device address: the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[INFERO_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_setup_mutex;

// Device address of the array on the current device (looked up on the first call there).
int static_scratch(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        infero_set_error("attn_decode_static: cannot tell the current device (%s)", cudaGetErrorString(e));
        return 1;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            infero_set_error("attn_decode_static: no device address for the scratch array on device %d (%s)", dev,
                             cudaGetErrorString(e));
            return 1;
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int infero_attn_decode_static(const void* q, int q_stride, void* out, int out_stride,
                                         const void* k_cache, const void* v_cache, const int* block_table,
                                         int max_blocks, const int* tok_entry, const int* positions, int tok_first,
                                         int n_tok, int n_heads, int n_kv, int head_dim, int page_size, int window,
                                         float scale, int chunk, int n_splits, cudaStream_t stream) {
    if (n_tok == 0) return 0;
    INFERO_REQUIRE(n_tok > 0 && n_heads > 0 && head_dim > 0 && n_splits > 0,
                   "attn_decode_static: bad sizes n_tok=%d n_heads=%d head_dim=%d n_splits=%d", n_tok, n_heads,
                   head_dim, n_splits);
    const long long need = infero_attn_decode_scratch(n_tok, n_heads, head_dim, n_splits);
    INFERO_REQUIRE(need <= INFERO_STATIC_SCRATCH_BYTES,
                   "attn_decode_static: %lld bytes of scratch needed (%d tokens x %d heads x %d splits), the fixed "
                   "array holds %lld; use fewer splits or tokens per call, or infero_attn_decode with your own scratch",
                   need, n_tok, n_heads, n_splits, (long long)INFERO_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (static_scratch(&scratch)) return 1;
    return infero_attn_decode(q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_blocks, tok_entry,
                              positions, tok_first, n_tok, n_heads, n_kv, head_dim, page_size, window, scale, chunk,
                              n_splits, scratch, stream);
}
