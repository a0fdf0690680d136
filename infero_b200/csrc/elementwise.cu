// Embedding gather, RMSNorm (with the residual add fused in), SwiGLU product.
//
// The residual stream x is kept in 32-bit in both precisions; what a kernel hands to a
// matrix product is written in the activation type (float, or bf16 in the serving
// precision).  All statistics and the residual sum are 32-bit.
//
// Formulas as in the reference: crates/kernels/src/cu/quant.cu:138-150 (gather),
// crates/kernels/src/cu/ops.cu:44-62 (x * rsqrt(mean(x^2)+eps) * w; multiply by the
// scale first, then by w), ops.cu:111-133 (g / (1 + exp(-g)) * u).
#include "common.cuh"

namespace {

template <typename TE>
__global__ void embed_gather_kernel(const TE* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ x, int d, int vocab, float scale) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // ids are validated on the host
    const TE* row = table + (size_t)id * d;
    float* o = x + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32(row[i]) * scale;
}

// One block per output row.
//   src row  = rows ? rows[blockIdx.x] : blockIdx.x
//   v        = x[src] (+ delta[src])            (32-bit)
//   if !rows: x[src] = v                        (the residual stream moves on)
//   out[blockIdx.x] = v * rsqrt(mean(v^2)+eps) * w
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                   const void* __restrict__ w, int wdtype, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    TO* orow = out + (size_t)r * d;
    extern __shared__ float vbuf[];      // d floats: the summed row, read twice
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (dr) v += to_f32(dr[i]);
        vbuf[i] = v;
        if (!rows && dr) xr[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = vbuf[i] * s;
        orow[i] = from_f32<TO>(v * load_any(w, wdtype, i));
    }
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int ff, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t t = i / ff;
    int j = (int)(i - t * ff);
    float g = to_f32(gu[t * 2 * (size_t)ff + j]);
    float u = to_f32(gu[t * 2 * (size_t)ff + ff + j]);
    float h = g / (1.0f + expf(-g)) * u;
    out[i] = from_f32<T>(h);
}

// x[t,:] += delta[t,:]   (used when no norm follows)
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] += to_f32(delta[i]);
}

}  // namespace

extern "C" {

int infero_embed_gather(const void* table, int table_dtype, const int* ids, float* x,
                        int n_tokens, int d, int vocab, float scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(d > 0 && vocab > 0, "embed_gather: bad sizes d=%d vocab=%d", d, vocab);
    const int threads = d >= 256 ? 256 : 64;
    if (table_dtype == INFERO_F32)
        embed_gather_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)table, ids, x, d, vocab, scale);
    else
        embed_gather_kernel<bf16><<<n_tokens, threads, 0, stream>>>((const bf16*)table, ids, x, d, vocab, scale);
    return infero_check_launch("embed_gather");
}

// delta may be null (plain norm); rows may be null (all rows, residual written back).
int infero_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w, int w_dtype,
                       float eps, void* out, int out_dtype, const int* rows, int n_rows, int d,
                       cudaStream_t stream) {
    if (n_rows == 0) return 0;
    INFERO_REQUIRE(d > 0 && (size_t)d * 4 <= 160 * 1024, "add_rmsnorm: width %d not supported (1..40960)", d);
    const size_t smem = (size_t)d * sizeof(float);
    const int threads = 256;
#define LAUNCH(TD, TO)                                                                          \
    do {                                                                                        \
        auto k = add_rmsnorm_kernel<TD, TO>;                                                    \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        k<<<n_rows, threads, smem, stream>>>(x, (const TD*)delta, w, w_dtype, eps, (TO*)out,    \
                                             rows, d);                                          \
    } while (0)
    if (delta_dtype == INFERO_F32 && out_dtype == INFERO_F32) LAUNCH(float, float);
    else if (delta_dtype == INFERO_BF16 && out_dtype == INFERO_BF16) LAUNCH(bf16, bf16);
    else if (delta_dtype == INFERO_F32 && out_dtype == INFERO_BF16) LAUNCH(float, bf16);
    else LAUNCH(bf16, float);
#undef LAUNCH
    return infero_check_launch("add_rmsnorm");
}

int infero_swiglu(const void* gate_up, void* out, int dtype, int n_tokens, int ff, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * ff;
    if (total == 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == INFERO_F32)
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, ff, total);
    else
        swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, ff, total);
    return infero_check_launch("swiglu");
}

int infero_residual_add(float* x, const void* delta, int delta_dtype, int n_tokens, int d, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * d;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (delta_dtype == INFERO_F32)
        residual_add_kernel<float><<<blocks, 256, 0, stream>>>(x, (const float*)delta, total);
    else
        residual_add_kernel<bf16><<<blocks, 256, 0, stream>>>(x, (const bf16*)delta, total);
    return infero_check_launch("residual_add");
}

}  // extern "C"
