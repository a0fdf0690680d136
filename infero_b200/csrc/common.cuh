// Shared device helpers: element types, 32-bit conversions, block reductions and the
// error record that every launcher of this library reports through.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

// Element type tags passed across the C boundary.
enum : int { INFERO_F32 = 0, INFERO_BF16 = 1 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Read element i of a vector whose type is only known at run time (norm weights and
// biases keep the width they were stored in).
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    return dtype == INFERO_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on blockDim, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? smem32[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

// ---- programmatic dependent launch --------------------------------------------------------
// A kernel launched through launch_pdl may start while the kernel before it in the stream is
// still running.  Such a kernel calls pdl_launch_dependents() first (its successor may then be
// scheduled as soon as every block of this grid has started) and pdl_wait() before it reads
// anything an earlier kernel wrote or writes anything at all; what lies before pdl_wait()
// (barrier set-up, prefetch of weights) overlaps the tail of the predecessor.  Launched the
// ordinary way, both calls do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

int infero_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = infero_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- timeline (only in a library built with -DINFERO_TIMELINE) -----------------------------
// The reference times its kernels one by one with events (crates/cuda/src/profile.rs:28-130).  Under
// programmatic dependent launch neighbours overlap, and what a kernel costs in place is not what it
// takes alone; a library built with INFERO_TIMELINE=1 therefore lets every block of the instrumented
// kernels leave (kind, grid size, block, multiprocessor, first and last nanosecond of the global
// timer) in a log that tools/timeline.py attaches and reads.  The ordinary build compiles none of it.
enum : int { TL_EMBED = 1, TL_NORM = 2, TL_GEMM = 3, TL_ROPE = 4, TL_ATTN_DECODE = 5, TL_ARGMAX = 6,
              TL_ARGMAX_FINAL = 7, TL_KEEP = 8, TL_SWIGLU = 9, TL_ATTN_PREFILL = 10 };
#ifdef INFERO_TIMELINE
struct InferoTlRecord { unsigned long long t0, t1; int kind, grid, block, sm; };
struct InferoTlLog { unsigned int cursor, capacity; unsigned long long pad; InferoTlRecord rec[1]; };
static __device__ InferoTlLog* infero_tl_log = nullptr;          // one per translation unit
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void tl_end(int kind, unsigned long long t0) {
    InferoTlLog* log = infero_tl_log;
    if (!log) return;
    const unsigned int i = atomicAdd(&log->cursor, 1u);
    if (i >= log->capacity) return;
    unsigned int sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    InferoTlRecord r;
    r.t0 = t0, r.t1 = tl_now(), r.kind = kind, r.grid = (int)(gridDim.x * gridDim.y * gridDim.z);
    r.block = (int)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x), r.sm = (int)sm;
    log->rec[i] = r;
}
#define TL_BEGIN() const unsigned long long tl_t0 = tl_now()
#define TL_END_IF(cond, kind) do { if (cond) tl_end(kind, tl_t0); } while (0)
#define INFERO_TL_UNIT(name)                                                                       \
    extern "C" int infero_tl_attach_##name(void* log) {                                            \
        return cudaMemcpyToSymbol(infero_tl_log, &log, sizeof(log)) != cudaSuccess;                \
    }
#else
#define TL_BEGIN() do { } while (0)
#define TL_END_IF(cond, kind) do { } while (0)
#define INFERO_TL_UNIT(name)
#endif
#define TL_END(kind) TL_END_IF(threadIdx.x == 0 && threadIdx.y == 0, kind)
// a mark inside a kernel: a record of its own kind (50 and above) that ends where the mark stands
#define TL_MARK(kind) TL_END(kind)

// ---- error reporting -------------------------------------------------------------------
// Launchers return 0 on success.  On failure they return non-zero and leave a message
// that infero_last_error() hands to the caller.
void infero_set_error(const char* fmt, ...);
int infero_check_launch(const char* what);

#define INFERO_REQUIRE(cond, ...)                 \
    do {                                          \
        if (!(cond)) {                            \
            infero_set_error(__VA_ARGS__);        \
            return 1;                             \
        }                                         \
    } while (0)
