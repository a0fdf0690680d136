// Rotary position encoding of q and k (NeoX pairing) fused with the append of k and v to
// the paged cache.
//
// qkv is one row per token: [q heads | k heads | v heads], each head head_dim wide.
// For i < rotary_dim/2:  ang = pos * inv_freq[i];  (a, b) = (x[i], x[i + rotary_dim/2]);
// x[i] = a cos - b sin;  x[i + half] = a sin + b cos.  Dimensions >= rotary_dim and v are
// untouched (crates/kernels/src/cu/ops.cu:488-523; crates/kernels/src/cpu/mod.rs:275-314).
// The reference then stores k and v in a second kernel (ops.cu:661-685) and scatters a slot
// table in a third (:693-701); here the page of a token is looked up in the request's block
// table: page = table[entry][pos / page_size], row = pos % page_size.
//
// Angles, sine and cosine are 32-bit with the accurate sincosf.  inv_freq comes from the
// host, so the device's pow never enters.
#include "common.cuh"

namespace {

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                  const int* __restrict__ tok_entry, const int* __restrict__ block_table,
                                  int max_blocks, const float* __restrict__ inv_freq, int rotary_dim,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size,
                                  int n_heads, int n_kv, int head_dim, int write_cache) {
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int h = blockIdx.y;                 // [0,n_heads): q   [n_heads, +n_kv): k   then v
    const int pos = positions[t];
    T* row = qkv + (size_t)t * row_stride + (size_t)h * head_dim;
    const int half = rotary_dim >> 1;
    const bool is_q = h < n_heads;
    const bool is_k = !is_q && h < n_heads + n_kv;
    T* dst = nullptr;
    if (!is_q) {
        if (!write_cache) return;
        const int kvh = is_k ? h - n_heads : h - n_heads - n_kv;
        const int page = block_table[(size_t)tok_entry[t] * max_blocks + pos / page_size];
        if (page < 0) return;     // never for a token of this step; guards a bad table
        T* base = is_k ? k_cache : v_cache;
        dst = base + (((size_t)page * n_kv + kvh) * page_size + (pos % page_size)) * head_dim;
    }
    if (is_q || is_k) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float s, c;
            sincosf((float)pos * inv_freq[i], &s, &c);
            const float a = to_f32(row[i]), b = to_f32(row[i + half]);
            const T ra = from_f32<T>(a * c - b * s), rb = from_f32<T>(a * s + b * c);
            if (is_q) { row[i] = ra; row[i + half] = rb; }
            else      { dst[i] = ra; dst[i + half] = rb; }
        }
        if (is_k)
            for (int i = rotary_dim + threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = row[i];
    } else {
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = row[i];
    }
    TL_END(TL_ROPE);
}

// bf16, many tokens: one block per token.  The sines and cosines of the token's position are
// worked out once (they are the same for every head) and kept in shared memory; then every
// thread moves 8 + 8 elements at a time: rotate q in place, rotate k into its page, copy v.
// Needs rotary_dim % 16 == 0, head_dim % 8 == 0 and 16-byte aligned rows.
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(bf16* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                      const int* __restrict__ tok_entry, const int* __restrict__ block_table, int max_blocks,
                      const float* __restrict__ inv_freq, int rotary_dim, bf16* __restrict__ k_cache,
                      bf16* __restrict__ v_cache, int page_size, int n_heads, int n_kv, int head_dim,
                      int write_cache) {
    extern __shared__ float2 sc[];                 // [rotary_dim / 2] (sin, cos)
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        sc[i] = make_float2(sn, cs);
    }
    __syncthreads();
    bf16* row = qkv + (size_t)t * row_stride;
    const int page = write_cache ? block_table[(size_t)tok_entry[t] * max_blocks + pos / page_size] : -1;
    const size_t in_page = (size_t)(pos % page_size) * head_dim;
    const int hc = half >> 3;                      // chunks of 8 pairs per head
    const int rot_items = (n_heads + n_kv) * hc;
    for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
        const int h = it / hc, c = it - h * hc;
        const bf16* src = row + (size_t)h * head_dim + c * 8;
        bf16* dst;
        if (h < n_heads) {
            dst = row + (size_t)h * head_dim + c * 8;
        } else {
            if (page < 0) continue;
            dst = k_cache + ((size_t)page * n_kv + (h - n_heads)) * page_size * head_dim + in_page + c * 8;
        }
        uint4 ua = *reinterpret_cast<const uint4*>(src), ub = *reinterpret_cast<const uint4*>(src + half);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
        uint4 oa, ob;
        __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
        __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 s0 = sc[c * 8 + 2 * k], s1 = sc[c * 8 + 2 * k + 1];
            const float a0 = __low2float(pa[k]), a1 = __high2float(pa[k]);
            const float b0 = __low2float(pb[k]), b1 = __high2float(pb[k]);
            qa[k] = __floats2bfloat162_rn(a0 * s0.y - b0 * s0.x, a1 * s1.y - b1 * s1.x);
            qb[k] = __floats2bfloat162_rn(a0 * s0.x + b0 * s0.y, a1 * s1.x + b1 * s1.y);
        }
        *reinterpret_cast<uint4*>(dst) = oa;
        *reinterpret_cast<uint4*>(dst + half) = ob;
    }
    if (page < 0) return;
    // what is not rotated: the tail of every k head beyond rotary_dim, and v
    const int tail = (head_dim - rotary_dim) >> 3, dc = head_dim >> 3;
    const int copy_items = n_kv * (tail + dc);
    for (int it = threadIdx.x; it < copy_items; it += blockDim.x) {
        const int kvh = it / (tail + dc), c = it - kvh * (tail + dc);
        const bf16* src;
        bf16* dst;
        if (c < tail) {
            src = row + (size_t)(n_heads + kvh) * head_dim + rotary_dim + c * 8;
            dst = k_cache + ((size_t)page * n_kv + kvh) * page_size * head_dim + in_page + rotary_dim + c * 8;
        } else {
            src = row + (size_t)(n_heads + n_kv + kvh) * head_dim + (c - tail) * 8;
            dst = v_cache + ((size_t)page * n_kv + kvh) * page_size * head_dim + in_page + (c - tail) * 8;
        }
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
    TL_END(TL_ROPE);
}

// The same, reading q, k and v as the sum of 32-bit partial products (+ bias) that the
// few-token matrix kernel leaves behind: value(t, c) = sum_s partial[s][t][c] + bias[c], s
// ascending.  Rotated q goes to q_out [T, n_heads * head_dim]; k and v go to their pages.
template <typename T>
__global__ void rope_cache_partials_kernel(const float* __restrict__ partial, int splits, long long split_stride,
                                           int row_width, const void* __restrict__ bias, int bias_dtype,
                                           T* __restrict__ q_out, int q_stride, const int* __restrict__ positions,
                                           const int* __restrict__ tok_entry, const int* __restrict__ block_table,
                                           int max_blocks, const float* __restrict__ inv_freq, int rotary_dim,
                                           T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size,
                                           int n_heads, int n_kv, int head_dim, int write_cache) {
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int h = blockIdx.y;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    const bool is_q = h < n_heads;
    const bool is_k = !is_q && h < n_heads + n_kv;
    const size_t col0 = (size_t)h * head_dim;
    const float* src = partial + (size_t)t * row_width + col0;
    auto value = [&](int i) {
        float v = 0.f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s) v += src[(size_t)s * split_stride + i];
        if (bias) v += load_any(bias, bias_dtype, col0 + i);
        return v;
    };
    T* dst;
    if (is_q) {
        dst = q_out + (size_t)t * q_stride + col0;
    } else {
        if (!write_cache) return;
        const int kvh = is_k ? h - n_heads : h - n_heads - n_kv;
        const int page = block_table[(size_t)tok_entry[t] * max_blocks + pos / page_size];
        if (page < 0) return;
        T* base = is_k ? k_cache : v_cache;
        dst = base + (((size_t)page * n_kv + kvh) * page_size + (pos % page_size)) * head_dim;
    }
    if (is_q || is_k) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float a = value(i), b = value(i + half);
            dst[i] = from_f32<T>(a * cs - b * sn);
            dst[i + half] = from_f32<T>(a * sn + b * cs);
        }
        for (int i = rotary_dim + threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = from_f32<T>(value(i));
    } else {
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = from_f32<T>(value(i));
    }
    TL_END(TL_ROPE);
}

// The same for bf16 outputs with vector loads: one block per token, sines and cosines shared by
// all heads, every thread sums 4 + 4 columns over the splits, rotates and stores.
// Needs rotary_dim % 8 == 0, head_dim % 4 == 0 and 16-byte aligned rows of the partial sums.
__global__ void __launch_bounds__(256)
rope_cache_partials_vec_kernel(const float* __restrict__ partial, int splits, long long split_stride, int row_width,
                               const void* __restrict__ bias, int bias_dtype, bf16* __restrict__ q_out, int q_stride,
                               const int* __restrict__ positions, const int* __restrict__ tok_entry,
                               const int* __restrict__ block_table, int max_blocks,
                               const float* __restrict__ inv_freq, int rotary_dim, bf16* __restrict__ k_cache,
                               bf16* __restrict__ v_cache, int page_size, int n_heads, int n_kv, int head_dim,
                               int write_cache) {
    extern __shared__ float2 sc[];
    TL_BEGIN();
    pdl_launch_dependents();
    // positions and block tables are set before the step's first kernel: the sines can be worked
    // out while the product in front is still running
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        sc[i] = make_float2(sn, cs);
    }
    const int page = write_cache ? block_table[(size_t)tok_entry[t] * max_blocks + pos / page_size] : -1;
    __syncthreads();
    pdl_wait();
    const float* src_row = partial + (size_t)t * row_width;
    const size_t in_page = (size_t)(pos % page_size) * head_dim;
    auto sum4 = [&](size_t col, float* v) {
        v[0] = v[1] = v[2] = v[3] = 0.f;
        // eight splits' loads in flight at a time; added in ascending order
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float4 f[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (s0 + k < splits) f[k] = *reinterpret_cast<const float4*>(src_row + (size_t)(s0 + k) * split_stride + col);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (s0 + k < splits) { v[0] += f[k].x; v[1] += f[k].y; v[2] += f[k].z; v[3] += f[k].w; }
        }
        if (bias) {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] += load_any(bias, bias_dtype, col + k);
        }
    };
    auto store4bf = [](bf16* p, const float* v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    };
    // work items: rotated chunks of q and k heads, unrotated tails, chunks of v; the blocks of a
    // token (gridDim.y of them) share the items so that every thread has about one
    const int hc = half >> 2;                      // chunks of 4 pairs per head
    const int rot_items = (n_heads + n_kv) * hc;
    const int tail = (head_dim - rotary_dim) >> 2, dc = head_dim >> 2;
    const int tail_items = (n_heads + n_kv) * tail;
    const int v_items = n_kv * dc;
    const int total = rot_items + tail_items + v_items;
    for (int it0 = blockIdx.y * blockDim.x + threadIdx.x; it0 < total; it0 += gridDim.y * blockDim.x) {
        if (it0 < rot_items) {
            const int h = it0 / hc, c = it0 - h * hc;
            bf16* dst;
            if (h < n_heads) {
                dst = q_out + (size_t)t * q_stride + (size_t)h * head_dim + c * 4;
            } else {
                if (page < 0) continue;
                dst = k_cache + ((size_t)page * n_kv + (h - n_heads)) * page_size * head_dim + in_page + c * 4;
            }
            float a[4], b[4], ra[4], rb[4];
            sum4((size_t)h * head_dim + c * 4, a);
            sum4((size_t)h * head_dim + half + c * 4, b);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 s1 = sc[c * 4 + k];
                ra[k] = a[k] * s1.y - b[k] * s1.x;
                rb[k] = a[k] * s1.x + b[k] * s1.y;
            }
            store4bf(dst, ra);
            store4bf(dst + half, rb);
        } else if (it0 < rot_items + tail_items) {
            const int it = it0 - rot_items;
            const int h = it / tail, c = it - h * tail;
            bf16* dst;
            if (h < n_heads) {
                dst = q_out + (size_t)t * q_stride + (size_t)h * head_dim + rotary_dim + c * 4;
            } else {
                if (page < 0) continue;
                dst = k_cache + ((size_t)page * n_kv + (h - n_heads)) * page_size * head_dim + in_page + rotary_dim + c * 4;
            }
            float v[4];
            sum4((size_t)h * head_dim + rotary_dim + c * 4, v);
            store4bf(dst, v);
        } else {
            if (page < 0) continue;
            const int it = it0 - rot_items - tail_items;
            const int kvh = it / dc, c = it - kvh * dc;
            float v[4];
            sum4((size_t)(n_heads + n_kv + kvh) * head_dim + c * 4, v);
            store4bf(v_cache + ((size_t)page * n_kv + kvh) * page_size * head_dim + in_page + c * 4, v);
        }
    }
    TL_END(TL_ROPE);
}

}  // namespace

extern "C" {

int infero_rope_cache(void* qkv, int dtype, int row_stride, const int* positions, const int* tok_entry,
                      const int* block_table, int max_blocks, const float* inv_freq, int rotary_dim,
                      void* k_cache, void* v_cache, int page_size, int n_tokens, int n_heads, int n_kv,
                      int head_dim, int write_cache, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim,
                   "rope_cache: rotary_dim %d must be even and <= head_dim %d", rotary_dim, head_dim);
    INFERO_REQUIRE(n_heads + 2 * n_kv <= 65535, "rope_cache: too many heads (%d)", n_heads + 2 * n_kv);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (dtype == INFERO_BF16 && n_tokens >= 16 && rotary_dim % 16 == 0 && rotary_dim > 0 && head_dim % 8 == 0 &&
        row_stride % 8 == 0 && al16(qkv) && al16(k_cache) && al16(v_cache)) {
        launch_pdl(rope_cache_vec_kernel, dim3(n_tokens), dim3(256), (size_t)(rotary_dim / 2) * sizeof(float2), stream,
                   (bf16*)qkv, row_stride, positions, tok_entry, block_table, max_blocks, inv_freq, rotary_dim,
                   (bf16*)k_cache, (bf16*)v_cache, page_size, n_heads, n_kv, head_dim, write_cache);
        return infero_check_launch("rope_cache_vec");
    }
    dim3 grid(n_tokens, n_heads + 2 * n_kv);
    const int threads = head_dim >= 128 ? 64 : 32;
    if (dtype == INFERO_F32)
        launch_pdl(rope_cache_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, row_stride, positions, tok_entry,
            block_table, max_blocks, inv_freq, rotary_dim, (float*)k_cache, (float*)v_cache, page_size,
            n_heads, n_kv, head_dim, write_cache);
    else
        launch_pdl(rope_cache_kernel<bf16>, grid, dim3(threads), 0, stream, (bf16*)qkv, row_stride, positions, tok_entry,
            block_table, max_blocks, inv_freq, rotary_dim, (bf16*)k_cache, (bf16*)v_cache, page_size,
            n_heads, n_kv, head_dim, write_cache);
    return infero_check_launch("rope_cache");
}


// partial: splits arrays of [n_tokens, (n_heads + 2 n_kv) * head_dim] float, split_stride
// elements apart; bias nullable.  q_out and the caches have type dtype.
int infero_rope_cache_partials(const float* partial, int splits, long long split_stride, const void* bias,
                               int bias_dtype, void* q_out, int q_stride, int dtype, const int* positions,
                               const int* tok_entry, const int* block_table, int max_blocks,
                               const float* inv_freq, int rotary_dim, void* k_cache, void* v_cache, int page_size,
                               int n_tokens, int n_heads, int n_kv, int head_dim, int write_cache,
                               cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim,
                   "rope_cache: rotary_dim %d must be even and <= head_dim %d", rotary_dim, head_dim);
    INFERO_REQUIRE(n_heads + 2 * n_kv <= 65535, "rope_cache: too many heads (%d)", n_heads + 2 * n_kv);
    INFERO_REQUIRE(splits >= 1, "rope_cache: %d splits", splits);
    const int width = (n_heads + 2 * n_kv) * head_dim;
    auto al = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    if (dtype == INFERO_BF16 && rotary_dim % 8 == 0 && head_dim % 4 == 0 && q_stride % 4 == 0 && width % 4 == 0 &&
        split_stride % 4 == 0 && al(partial, 16) && al(q_out, 8) && al(k_cache, 8) && al(v_cache, 8)) {
        const int items = (n_heads + n_kv) * (head_dim / 4) + n_kv * (head_dim / 4) - (n_heads + n_kv) * (rotary_dim / 8);
        int by = (items + 255) / 256;
        if (by > 16) by = 16;
        if (by < 1) by = 1;
        launch_pdl(rope_cache_partials_vec_kernel, dim3(n_tokens, by), dim3(256), (size_t)(rotary_dim / 2) * sizeof(float2),
                   stream, partial, splits, split_stride, width, bias, bias_dtype, (bf16*)q_out, q_stride, positions,
                   tok_entry, block_table, max_blocks, inv_freq, rotary_dim, (bf16*)k_cache, (bf16*)v_cache, page_size,
                   n_heads, n_kv, head_dim, write_cache);
        return infero_check_launch("rope_cache_partials_vec");
    }
    dim3 grid(n_tokens, n_heads + 2 * n_kv);
    const int threads = head_dim >= 128 ? 64 : 32;
    if (dtype == INFERO_F32)
        launch_pdl(rope_cache_partials_kernel<float>, grid, dim3(threads), 0, stream, partial, splits, split_stride, width, bias,
            bias_dtype, (float*)q_out, q_stride, positions, tok_entry, block_table, max_blocks, inv_freq, rotary_dim,
            (float*)k_cache, (float*)v_cache, page_size, n_heads, n_kv, head_dim, write_cache);
    else
        launch_pdl(rope_cache_partials_kernel<bf16>, grid, dim3(threads), 0, stream, partial, splits, split_stride, width, bias,
            bias_dtype, (bf16*)q_out, q_stride, positions, tok_entry, block_table, max_blocks, inv_freq, rotary_dim,
            (bf16*)k_cache, (bf16*)v_cache, page_size, n_heads, n_kv, head_dim, write_cache);
    return infero_check_launch("rope_cache_partials");
}

}  // extern "C"

INFERO_TL_UNIT(rope_cache)
