// Embedding gather, RMSNorm (with the residual add fused in), SwiGLU product.
//
// The residual stream x is kept in 32-bit in both precisions; what a kernel hands to a
// matrix product is written in the activation type (float, or bf16 in the serving
// precision).  All statistics and the residual sum are 32-bit.
//
// Formulas as in the reference: crates/kernels/src/cu/quant.cu:138-150 (gather),
// crates/kernels/src/cu/ops.cu:44-62 (x * rsqrt(mean(x^2)+eps) * w; multiply by the
// scale first, then by w), ops.cu:111-133 (g / (1 + exp(-g)) * u).
#include "tc_common.cuh"
#include <cstdlib>

namespace {

template <typename TE>
__global__ void embed_gather_kernel(const TE* __restrict__ table, const int* __restrict__ ids,
                                    const int* __restrict__ device_tokens, float* __restrict__ x, int d, int vocab,
                                    float scale) {
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    // a negative id -(s + 1) stands for "the token the sampler left in device_tokens[s]": the step
    // was launched before the host had seen that token
    if (id < 0 && device_tokens) id = device_tokens[-id - 1];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // ids are validated on the host
    const TE* row = table + (size_t)id * d;
    float* o = x + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32(row[i]) * scale;
    TL_END(TL_EMBED);
}

// 4 consecutive elements as 32-bit values (p must be aligned to 4 elements).
__device__ __forceinline__ void load4(const float* p, float* v) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void load4(const bf16* p, float* v) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void load4_any(const void* p, int dtype, size_t i, float* v) {
    if (dtype == INFERO_F32) load4(reinterpret_cast<const float*>(p) + i, v);
    else load4(reinterpret_cast<const bf16*>(p) + i, v);
}
__device__ __forceinline__ void store4(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

// One block per output row.
//   src row  = rows ? rows[blockIdx.x] : blockIdx.x
//   v        = x[src] + sum_s delta[s][src] (+ dbias)      (32-bit; s ascending)
//   if !rows: x[src] = v                                   (the residual stream moves on)
//   out[blockIdx.x] = v * rsqrt(mean(v^2)+eps) * w
// delta may come as several 32-bit partial sums (the split-K products of the few-token
// matrix kernel), split_stride elements apart.  VEC = 4 needs d % 4 == 0.
template <typename TD, typename TO, int VEC>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int splits,
                                   long long split_stride, const void* __restrict__ dbias, int dbias_dtype,
                                   const void* __restrict__ w, int wdtype, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float red[32];
    TL_BEGIN();
    pdl_launch_dependents();
    // the norm's weights do not come from the kernel in front: the thread's first vector of them
    // is fetched before the wait
    float w_first[4] = {0.f, 0.f, 0.f, 0.f};
    if (VEC == 4 && (int)threadIdx.x * 4 < d) load4_any(w, wdtype, threadIdx.x * 4, w_first);
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    TO* orow = out + (size_t)r * d;
    extern __shared__ float vbuf[];      // d floats: the summed row, read twice
    float ss = 0.f;
    // first loop: loads only (global stores wait for the second loop, so that the loads of all
    // of a thread's vectors can be in flight together)
    if (VEC == 4) {
#pragma unroll 2
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float v[4];
            load4(xr + i, v);
            if (dr) {
                // eight partial sums' loads in flight at a time; added in ascending order
                for (int s0 = 0; s0 < splits; s0 += 8) {
                    float t[8][4];
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (s0 + k < splits) load4(dr + (size_t)(s0 + k) * split_stride + i, t[k]);
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (s0 + k < splits) { v[0] += t[k][0]; v[1] += t[k][1]; v[2] += t[k][2]; v[3] += t[k][3]; }
                }
                if (dbias) {
                    float t[4];
                    load4_any(dbias, dbias_dtype, i, t);
                    v[0] += t[0]; v[1] += t[1]; v[2] += t[2]; v[3] += t[3];
                }
            }
            store4(vbuf + i, v);
            ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float v = xr[i];
            if (dr) {
                for (int s = 0; s < splits; ++s) v += to_f32(dr[(size_t)s * split_stride + i]);
                if (dbias) v += load_any(dbias, dbias_dtype, i);
            }
            vbuf[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)d + eps);
    const bool write_x = dr && !rows;
    if (VEC == 4) {
#pragma unroll 4
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float v[4], ww[4];
            load4(vbuf + i, v);
            if (write_x) store4(xr + i, v);
            if (i == (int)threadIdx.x * 4) { ww[0] = w_first[0]; ww[1] = w_first[1]; ww[2] = w_first[2]; ww[3] = w_first[3]; }
            else load4_any(w, wdtype, i, ww);
            v[0] = v[0] * sc * ww[0]; v[1] = v[1] * sc * ww[1]; v[2] = v[2] * sc * ww[2]; v[3] = v[3] * sc * ww[3];
            store4(orow + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v0 = vbuf[i];
            if (write_x) xr[i] = v0;
            orow[i] = from_f32<TO>(v0 * sc * load_any(w, wdtype, i));
        }
    }
    TL_END(TL_NORM);
}

// Many rows, one vector per thread: a block walks over rows blockIdx.x, + gridDim.x, ... and
// has the next row's loads in flight while it reduces and writes the current one.  Thread t
// owns elements 4t .. 4t+3 of every row and the block size is the same as in the kernel above,
// so each row is computed by exactly the same operations in the same order.
template <typename TD, typename TO>
__global__ void __launch_bounds__(1024, 2) add_rmsnorm_rows_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                        const void* __restrict__ dbias, int dbias_dtype,
                                        const void* __restrict__ w, int wdtype, float eps,
                                        TO* __restrict__ out, int n_rows, int d) {
    __shared__ float red[32];
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int i = threadIdx.x * 4;
    const bool mine = i < d;
    float ww[4] = {0.f, 0.f, 0.f, 0.f}, bb[4] = {0.f, 0.f, 0.f, 0.f};
    if (mine) {
        load4_any(w, wdtype, i, ww);
        if (dbias) load4_any(dbias, dbias_dtype, i, bb);
    }
    float xv[4] = {0.f, 0.f, 0.f, 0.f}, dv[4] = {0.f, 0.f, 0.f, 0.f};
    int r = blockIdx.x;
    if (r < n_rows && mine) {
        load4(x + (size_t)r * d + i, xv);
        if (delta) load4(delta + (size_t)r * d + i, dv);
    }
    for (; r < n_rows; r += gridDim.x) {
        float v[4] = {xv[0], xv[1], xv[2], xv[3]};
        if (delta) {
            v[0] += dv[0]; v[1] += dv[1]; v[2] += dv[2]; v[3] += dv[3];
            if (dbias) { v[0] += bb[0]; v[1] += bb[1]; v[2] += bb[2]; v[3] += bb[3]; }
        }
        const int rn = r + gridDim.x;
        if (rn < n_rows && mine) {                   // the next row, before this one is reduced
            load4(x + (size_t)rn * d + i, xv);
            if (delta) load4(delta + (size_t)rn * d + i, dv);
        }
        float ss = 0.f;
        if (mine) {
            ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
        }
        ss = block_sum(ss, red);
        const float sc = 1.0f / sqrtf(ss / (float)d + eps);
        if (mine) {
            if (delta) store4(x + (size_t)r * d + i, v);
            v[0] = v[0] * sc * ww[0]; v[1] = v[1] * sc * ww[1]; v[2] = v[2] * sc * ww[2]; v[3] = v[3] * sc * ww[3];
            store4(out + (size_t)r * d + i, v);
        }
    }
    TL_END(TL_NORM);
}

// The same rows through a ring in shared memory: one thread asks for whole rows (x and delta, one
// bulk copy each, RING rows ahead), so a block has RING rows on their way instead of two and the
// loads no longer wait on the block-wide sum of the row before.  The arithmetic per row is the
// kernel's above, operation for operation.  Needs rows that are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tc::smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
                 : "memory");
}

template <typename TD, typename TO>
__global__ void __launch_bounds__(1024, 2) add_rmsnorm_ring_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                                                   const void* __restrict__ dbias, int dbias_dtype,
                                                                   const void* __restrict__ w, int wdtype, float eps,
                                                                   TO* __restrict__ out, int n_rows, int d, int ring,
                                                                   int* __restrict__ err_flag) {
    extern __shared__ __align__(16) uint8_t ring_mem[];
    __shared__ float red[32];
    __shared__ uint64_t full[8];
    __shared__ int abort_flag;
    const uint32_t x_bytes = (uint32_t)d * 4u, d_bytes = delta ? (uint32_t)d * (uint32_t)sizeof(TD) : 0u;
    const uint32_t row_bytes = x_bytes + d_bytes;
    TL_BEGIN();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < ring; ++s) tc::mbar_init(&full[s], 1);
        abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    const int i = threadIdx.x * 4;
    const bool mine = i < d;
    float ww[4] = {0.f, 0.f, 0.f, 0.f}, bb[4] = {0.f, 0.f, 0.f, 0.f};
    if (mine) {
        load4_any(w, wdtype, i, ww);
        if (dbias) load4_any(dbias, dbias_dtype, i, bb);
    }
    __syncthreads();
    pdl_wait();
    auto ask = [&](int r, int s) {                  // (thread 0) row r into stage s
        uint8_t* st = ring_mem + (size_t)s * row_bytes;
        tc::mbar_expect_tx(&full[s], row_bytes);
        bulk_load(st, x + (size_t)r * d, x_bytes, &full[s]);
        if (delta) bulk_load(st + x_bytes, delta + (size_t)r * d, d_bytes, &full[s]);
    };
    if (threadIdx.x == 0)
        for (int s = 0; s < ring; ++s) {
            const int r = (int)blockIdx.x + s * (int)gridDim.x;
            if (r < n_rows) ask(r, s);
        }
    int k = 0;
    bool ok = true;
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x, ++k) {
        const int s = k % ring;
        // (every thread watches the barrier itself, and the block agrees on the outcome before it goes on)
        ok = __syncthreads_and(tc::mbar_wait(&full[s], (uint32_t)(k / ring) & 1u, &abort_flag) ? 1 : 0) != 0;
        if (!ok) break;
        const uint8_t* st = ring_mem + (size_t)s * row_bytes;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (mine) {
            load4(reinterpret_cast<const float*>(st) + i, v);
            if (delta) {
                float dv[4];
                load4(reinterpret_cast<const TD*>(st + x_bytes) + i, dv);
                v[0] += dv[0]; v[1] += dv[1]; v[2] += dv[2]; v[3] += dv[3];
                if (dbias) { v[0] += bb[0]; v[1] += bb[1]; v[2] += bb[2]; v[3] += bb[3]; }
            }
        }
        float ss = 0.f;
        if (mine) {
            ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
        }
        ss = block_sum(ss, red);                    // (its barriers: every thread has read the stage by now)
        if (threadIdx.x == 0) {
            const int rn = r + ring * (int)gridDim.x;
            if (rn < n_rows) {
                tc::fence_proxy_async();            // the stage was read through ordinary loads
                ask(rn, s);
            }
        }
        const float sc = 1.0f / sqrtf(ss / (float)d + eps);
        if (mine) {
            if (delta) store4(x + (size_t)r * d + i, v);
            v[0] = v[0] * sc * ww[0]; v[1] = v[1] * sc * ww[1]; v[2] = v[2] * sc * ww[2]; v[3] = v[3] * sc * ww[3];
            store4(out + (size_t)r * d + i, v);
        }
    }
    if (!ok) {
        // a row never arrived (the wait is bounded): report it; what thread 0 asked for and has not been
        // waited for is given the same bounded time to land before the block's shared memory goes away
        if (threadIdx.x == 0) {
            abort_flag = 1;
            atomicExch(err_flag, 8);
        }
    }
    __syncthreads();
    if (!ok && threadIdx.x == 0) {
        int never = 0;
        int kk = k;
        for (int r = (int)blockIdx.x + k * (int)gridDim.x, n = 0; r < n_rows && n < ring; r += gridDim.x, ++n, ++kk)
            tc::mbar_wait(&full[kk % ring], (uint32_t)(kk / ring) & 1u, &never);
    }
    TL_END(TL_NORM);
}

// out[t, j] = silu(g) * u with g = sum_s gu[s][t, 2j], u = sum_s gu[s][t, 2j + 1] (s ascending):
// gate and up alternate along a row, as the stacked weight's rows do.  VEC = 4 outputs per thread.
template <typename T, int VEC>
__global__ void swiglu_kernel(const T* __restrict__ gu, int splits, long long split_stride, T* __restrict__ out_same,
                              bf16* __restrict__ out_bf16, int ff, size_t total) {
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= total) return;
    size_t t = i / ff;
    int j = (int)(i - t * ff);
    const T* row = gu + t * 2 * (size_t)ff + 2 * (size_t)j;
    float p[2 * VEC], h[VEC];
#pragma unroll
    for (int k = 0; k < 2 * VEC; ++k) p[k] = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
        const T* rs = row + (size_t)s * split_stride;
        if (VEC == 4) {
            float a[4], b[4];
            load4(rs, a);
            load4(rs + 4, b);
#pragma unroll
            for (int k = 0; k < 4; ++k) { p[k] += a[k]; p[4 + k] += b[k]; }
        } else {
            p[0] += to_f32(rs[0]);
            p[1] += to_f32(rs[1]);
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) h[k] = p[2 * k] / (1.0f + expf(-p[2 * k])) * p[2 * k + 1];
    if (VEC == 4) {
        if (out_bf16) store4(out_bf16 + i, h);
        else store4(out_same + i, h);
    } else {
        if (out_bf16) out_bf16[i] = __float2bfloat16_rn(h[0]);
        else out_same[i] = from_f32<T>(h[0]);
    }
    TL_END(TL_SWIGLU);
}

// x[t,:] += delta[t,:]   (used when no norm follows)
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] += to_f32(delta[i]);
}

}  // namespace

extern "C" {

int infero_embed_gather(const void* table, int table_dtype, const int* ids, const int* device_tokens, float* x,
                        int n_tokens, int d, int vocab, float scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(d > 0 && vocab > 0, "embed_gather: bad sizes d=%d vocab=%d", d, vocab);
    const int threads = d >= 256 ? 256 : 64;
    if (table_dtype == INFERO_F32)
        launch_pdl(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, device_tokens, x, d, vocab, scale);
    else
        launch_pdl(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, device_tokens, x, d, vocab, scale);
    return infero_check_launch("embed_gather");
}

// delta may be null (plain norm); rows may be null (all rows, residual written back).
// delta: delta_splits arrays of [rows of x, d], split_stride elements apart, summed in
// ascending order, plus dbias (nullable) -- the few-token matrix kernel's partial products.
int infero_add_rmsnorm(float* x, const void* delta, int delta_dtype, int delta_splits, long long split_stride,
                       const void* dbias, int dbias_dtype, const void* w, int w_dtype,
                       float eps, void* out, int out_dtype, const int* rows, int n_rows, int d,
                       cudaStream_t stream) {
    if (n_rows == 0) return 0;
    INFERO_REQUIRE(d > 0 && (size_t)d * 4 <= 160 * 1024, "add_rmsnorm: width %d not supported (1..40960)", d);
    INFERO_REQUIRE(delta_splits >= 1, "add_rmsnorm: %d splits", delta_splits);
    const size_t smem = (size_t)d * sizeof(float);
    auto al = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    const bool vec = d % 4 == 0 && al(x, 16) && al(out, 16) && al(w, 16) && (!delta || al(delta, 16)) &&
                     (!dbias || al(dbias, 16)) && split_stride % 4 == 0;
    // one vector per thread where the width allows it: with few rows (decode) the kernel is one
    // round trip to memory, and all of a row's loads are in flight together.  The block size
    // depends on the width only, so a row's arithmetic (and its rounding) does not depend on
    // how many rows the step has.
    int threads = vec ? (d / 4 + 31) / 32 * 32 : 256;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    if (vec && !rows && delta_splits == 1 && n_rows >= 256 && d <= 4 * threads) {
        // many rows (prompt portions): the pipelined kernel, same arithmetic per row
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int per_sm = 2048 / threads;
        if (per_sm > 8) per_sm = 8;
        if (per_sm < 1) per_sm = 1;
        int blocks = sms * per_sm;
        if (blocks > n_rows) blocks = n_rows;
        // rows through a ring of bulk copies where a row is a multiple of 16 bytes and two or more fit
        const size_t delta_row = delta ? (size_t)d * (delta_dtype == INFERO_F32 ? 4 : 2) : 0;
        const size_t row_bytes = (size_t)d * 4 + delta_row;
        int ring = (int)((96 * 1024) / row_bytes);
        if (ring > 4) ring = 4;
        static const bool ring_off = getenv("INFERO_NORM_RING") && atoi(getenv("INFERO_NORM_RING")) == 0;
        if (!ring_off && ring >= 2 && delta_row % 16 == 0 && ((size_t)d * 4) % 16 == 0) {
            int* err;
            if (infero_tc_err_flag(&err)) return 1;
            const size_t ring_bytes = (size_t)ring * row_bytes;
#define LAUNCH_RING(TD, TO)                                                                      \
            do {                                                                                 \
                auto k = add_rmsnorm_ring_kernel<TD, TO>;                                        \
                if (ring_bytes > 48 * 1024)                                                      \
                    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring_bytes); \
                launch_pdl(k, dim3(blocks), dim3(threads), ring_bytes, stream, x, (const TD*)delta, dbias, dbias_dtype, \
                           w, w_dtype, eps, (TO*)out, n_rows, d, ring, err);                      \
            } while (0)
            if (delta_dtype == INFERO_F32 && out_dtype == INFERO_F32) LAUNCH_RING(float, float);
            else if (delta_dtype == INFERO_BF16 && out_dtype == INFERO_BF16) LAUNCH_RING(bf16, bf16);
            else if (delta_dtype == INFERO_F32 && out_dtype == INFERO_BF16) LAUNCH_RING(float, bf16);
            else LAUNCH_RING(bf16, float);
#undef LAUNCH_RING
            return infero_check_launch("add_rmsnorm_ring");
        }
#define LAUNCH_ROWS(TD, TO)                                                                      \
        launch_pdl(add_rmsnorm_rows_kernel<TD, TO>, dim3(blocks), dim3(threads), 0, stream, x, (const TD*)delta, dbias, \
                   dbias_dtype, w, w_dtype, eps, (TO*)out, n_rows, d)
        if (delta_dtype == INFERO_F32 && out_dtype == INFERO_F32) LAUNCH_ROWS(float, float);
        else if (delta_dtype == INFERO_BF16 && out_dtype == INFERO_BF16) LAUNCH_ROWS(bf16, bf16);
        else if (delta_dtype == INFERO_F32 && out_dtype == INFERO_BF16) LAUNCH_ROWS(float, bf16);
        else LAUNCH_ROWS(bf16, float);
#undef LAUNCH_ROWS
        return infero_check_launch("add_rmsnorm_rows");
    }
#define LAUNCH(TD, TO)                                                                          \
    do {                                                                                        \
        if (vec) {                                                                              \
            auto k = add_rmsnorm_kernel<TD, TO, 4>;                                             \
            if (smem > 48 * 1024)                                                               \
                cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            launch_pdl(k, dim3(n_rows), dim3(threads), smem, stream, x, (const TD*)delta, delta_splits,   \
                       split_stride, dbias, dbias_dtype, w, w_dtype, eps, (TO*)out, rows, d);            \
        } else {                                                                                \
            auto k = add_rmsnorm_kernel<TD, TO, 1>;                                             \
            if (smem > 48 * 1024)                                                               \
                cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            launch_pdl(k, dim3(n_rows), dim3(threads), smem, stream, x, (const TD*)delta, delta_splits,   \
                       split_stride, dbias, dbias_dtype, w, w_dtype, eps, (TO*)out, rows, d);            \
        }                                                                                       \
    } while (0)
    if (delta_dtype == INFERO_F32 && out_dtype == INFERO_F32) LAUNCH(float, float);
    else if (delta_dtype == INFERO_BF16 && out_dtype == INFERO_BF16) LAUNCH(bf16, bf16);
    else if (delta_dtype == INFERO_F32 && out_dtype == INFERO_BF16) LAUNCH(float, bf16);
    else LAUNCH(bf16, float);
#undef LAUNCH
    return infero_check_launch("add_rmsnorm");
}

// gate_up: splits arrays of [n_tokens, 2 * ff] (dtype, gate and up alternating), split_stride elements apart.  out has
// gate_up's type, or bf16 when out_bf16 is set (32-bit partial products in, bf16 out).
int infero_swiglu(const void* gate_up, int splits, long long split_stride, void* out, int dtype, int out_bf16,
                  int n_tokens, int ff, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * ff;
    if (total == 0) return 0;
    INFERO_REQUIRE(splits >= 1, "swiglu: %d splits", splits);
    const int threads = 256;
    auto al = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    const bool vec = ff % 4 == 0 && al(gate_up, 16) && al(out, 16) && split_stride % 4 == 0;
    const size_t work = vec ? total / 4 : total;
    const unsigned blocks = (unsigned)((work + threads - 1) / threads);
    bf16* ob = out_bf16 ? (bf16*)out : nullptr;
    if (dtype == INFERO_F32) {
        if (vec) launch_pdl(swiglu_kernel<float, 4>, dim3(blocks), dim3(threads), 0, stream, (const float*)gate_up, splits, split_stride, (float*)out, ob, ff, total);
        else launch_pdl(swiglu_kernel<float, 1>, dim3(blocks), dim3(threads), 0, stream, (const float*)gate_up, splits, split_stride, (float*)out, ob, ff, total);
    } else {
        if (vec) launch_pdl(swiglu_kernel<bf16, 4>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)gate_up, splits, split_stride, (bf16*)out, nullptr, ff, total);
        else launch_pdl(swiglu_kernel<bf16, 1>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)gate_up, splits, split_stride, (bf16*)out, nullptr, ff, total);
    }
    return infero_check_launch("swiglu");
}

int infero_residual_add(float* x, const void* delta, int delta_dtype, int n_tokens, int d, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * d;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (delta_dtype == INFERO_F32)
        launch_pdl(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (const float*)delta, total);
    else
        launch_pdl(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (const bf16*)delta, total);
    return infero_check_launch("residual_add");
}

}  // extern "C"

INFERO_TL_UNIT(elementwise)
