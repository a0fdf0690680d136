// Attention over the paged cache for any batch of tokens: one warp per (token, query head).
//
// For token t of request entry e at position p, head h (kv head h / group):
//   s_j = (q . K[j]) * scale   for lo <= j <= p,  lo = window ? max(0, p - window + 1) : 0
//   out = sum_j softmax(s)_j V[j]
// (crates/kernels/src/cu/ops.cu:709-811 is the reference's three-kernel statement; its
// fused decode kernel is ops.cu:1773-2075.  Contiguous head groups: kv head = h / group.)
//
// Keys are visited in ascending order in chunks of 32 aligned to absolute positions, with a
// running maximum and sum (all 32-bit, accurate expf).  The arithmetic done for a token
// depends only on its own position and window, never on how the step was cut or on what
// else is in the batch.  It takes every head size up to 256 and every group size; it is the
// whole of attention on the 32-bit path and the fallback of the bf16 path.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ tok_entry, const int* __restrict__ positions,
                         int n_tokens, int n_heads, int n_kv, int head_dim, int page_size,
                         int window, float scale) {
    __shared__ float q_s[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const int group = n_heads / n_kv;
    const int kvh = h / group;
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_entry[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_s[warp][i] = to_f32(qrow[i]);
    __syncwarp();

    float m = -CUDART_INF_F, l = 0.f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

    for (int j0 = (lo / 32) * 32; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= lo && j <= pos;
        long long row = -1;
        float s = -CUDART_INF_F;
        if (valid) {
            const int page = table[j / page_size];
            if (page >= 0) {
                row = (((long long)page * n_kv + kvh) * page_size + (j % page_size)) * head_dim;
                const T* kr = k_cache + row;
                float d = 0.f;
                for (int i = 0; i < head_dim; ++i) d = fmaf(q_s[warp][i], to_f32(kr[i]), d);
                s = d * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -CUDART_INF_F) continue;         // no readable key in this chunk
        const float p = (row >= 0) ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);          // first chunk: exp(-inf) = 0
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (rj < 0) continue;                      // uniform across the warp
            const T* vr = v_cache + rj;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int dd = i * 32 + lane;
                if (dd < head_dim) acc[i] = fmaf(pj, to_f32(vr[dd]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * head_dim;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int dd = i * 32 + lane;
        if (dd < head_dim) orow[dd] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace

extern "C" {

int infero_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                             const void* v_cache, int dtype, const int* block_table, int max_blocks,
                             const int* tok_entry, const int* positions, int n_tokens, int n_heads,
                             int n_kv, int head_dim, int page_size, int window, float scale,
                             cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(head_dim >= 1 && head_dim <= MAX_D, "attention: head_dim %d outside 1..%d", head_dim, MAX_D);
    INFERO_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads not a multiple of %d kv heads", n_heads, n_kv);
    const long long items = (long long)n_tokens * n_heads;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (dtype == INFERO_F32)
        attention_generic_kernel<float><<<blocks, WARPS * 32, 0, stream>>>((const float*)q, q_stride, (float*)out,
            out_stride, (const float*)k_cache, (const float*)v_cache, block_table, max_blocks, tok_entry,
            positions, n_tokens, n_heads, n_kv, head_dim, page_size, window, scale);
    else
        attention_generic_kernel<bf16><<<blocks, WARPS * 32, 0, stream>>>((const bf16*)q, q_stride, (bf16*)out,
            out_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, tok_entry,
            positions, n_tokens, n_heads, n_kv, head_dim, page_size, window, scale);
    return infero_check_launch("attention_generic");
}

}  // extern "C"
