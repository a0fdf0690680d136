// Decode attention over the paged cache, fed by TMA.
//
// One CTA = one token, one kv head (its group of query heads fills the 16 rows of the MMA,
// 16 at a time) and one split of the context.  Each of the four warps walks its own 16-key
// slices (warp w takes slices w, w + 4, ...) through a ring of shared-memory stages of its
// own: lane 0 looks the slice's page up in the block table and issues tiled TMA loads
// (cp.async.bulk.tensor, 128-byte swizzle) for the slice's keys and values, which complete
// on an mbarrier; the warp waits for the stage, runs the 16-key step of the online softmax
// on mma.sync (s = q k^T, p = 2^(s - m), o += p v) and refills the stage.  Nothing but the
// TMA issue touches addresses, so the loop is a few hundred instructions per 8 KB of cache.
// The four warps are merged in shared memory and the CTA writes an unnormalised partial
// result (o, m, l) per query head; the CTA that arrives last for a (token, kv head) merges the
// splits (attn_combine does when there are more groups of splits than arrival counters).
// In steps of single tokens a second instance of the kernel (FUSED) also finishes the q/k/v
// product in front of it: bias, rotary positions and the cache append (see the kernel).
//
// The cache of one layer is seen as a matrix [pages * kv_heads * page_size, head_dim]; a slice
// of 16 keys is 16 consecutive rows of it (page_size is a multiple of 16).  Head sizes: 64 and
// 128 (whole 128-byte swizzle blocks); other sizes stay with the cp.async kernel in
// attention_mma.cu.  Reference: crates/kernels/src/cu/ops.cu:1773-2075 (fused decode attention
// with split context), :1465-1494 (merge).
#include "attn_common.cuh"
#include "tc_common.cuh"

extern "C" int infero_attn_decode_tma_supported(int head_dim, int page_size);

namespace {

using namespace attn;

constexpr int TD_WARPS = 4, TD_THREADS = TD_WARPS * 32;

template <int D>
struct TdPlan {
    static constexpr int STAGES = D == 128 ? 3 : 4;
    static constexpr int HALF_BYTES = 16 * D * 2;                 // keys (or values) of one slice
    static constexpr int STAGE_BYTES = 2 * HALF_BYTES;
    static constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
    static constexpr int TILES_BYTES = TD_WARPS * WARP_BYTES;
    static constexpr int RED_STRIDE = D + 8;                        // floats; the pad keeps the warps' row stores off each other's banks
    static constexpr int RED_BYTES = TD_WARPS * 16 * (RED_STRIDE + 3) * 4;
    static constexpr int DATA_BYTES = TILES_BYTES > RED_BYTES ? TILES_BYTES : RED_BYTES;
    static constexpr int BAR_OFFSET = DATA_BYTES;
    // the fused kernel's own: sines and cosines, the 16 rotated query rows, the token's new key and value
    static constexpr int Q_STRIDE = D + 8;
    static constexpr int FUSED_OFFSET = (BAR_OFFSET + TD_WARPS * STAGES * 8 + 16 + 15) / 16 * 16;
    static constexpr int FUSED_BYTES = (D / 2) * 8 + 16 * Q_STRIDE * 2 + 2 * D * 2;
    static constexpr int TOTAL = DATA_BYTES + TD_WARPS * STAGES * 8 + 16 + 1024;
    static constexpr int TOTAL_FUSED = FUSED_OFFSET + FUSED_BYTES + 1024;
};

// What the fused kernel takes in place of finished queries: the q/k/v product of the step's tokens as
// the few-token product kernel leaves it (32-bit partial sums [splits][token][(heads + 2 kv heads) * D],
// bias not yet added), and what the rotary-and-append kernel would have needed to finish it.
struct FusedQkv {
    const float* partial;
    long long split_stride;
    const void* bias;
    const float* inv_freq;
    bf16* k_cache;
    bf16* v_cache;
    int splits, row_width, bias_dtype, rotary_dim, write_cache;
    // The product's input may still lack its norm's scalar (the norm folded into the products around it,
    // gemm_tc.cu): then every summed value of token t is multiplied by
    // rsqrt(sum_{tile < in_tiles} sumsq_in[tile * 256 + t] * inv_d + eps) before the bias is added.
    const float* sumsq_in;
    int in_tiles;
    float inv_d, eps;
};

// The CTA that finishes last among the splits of one (token, kv head, group tile) merges them:
// out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M = max_s m_s.  Every CTA of the
// launch calls this after its partial result is written; `counter` counts the arrivals and is
// set back to zero by the last one, so the same (zeroed once) array serves every launch.
// Splits without keys wrote (m, l) = (-inf, 0) and no output: they are left out, not multiplied
// by zero (what lies in the scratch there may be NaN).
template <int D>
__device__ __forceinline__ void merge_if_last(int* counter, float* wbuf, const float* po_base, const float* pml_base,
                                              int n_splits, int valid, bf16* out_rows) {
    __shared__ int s_last;
    __syncthreads();                                   // every thread's partial results are written ...
    if (threadIdx.x == 0) {
        // ... and one release-and-acquire count publishes them and takes in those of the blocks before
        // (a release by one thread after a barrier covers what the block's other threads wrote)
        int old;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
        s_last = old == n_splits - 1;
        if (s_last) *counter = 0;
    }
    __syncthreads();
    if (!s_last) return;
    if (n_splits <= 16 && (reinterpret_cast<uintptr_t>(out_rows) & 15u) == 0) {
        // Up to 16 splits: one round of loads.  Every thread takes eight columns of a row and asks for the
        // row's (m, l) of every split and for its columns of every split's partial result at once, works the
        // weights out itself (the threads of a row all do, from the same values) and sums in ascending order.
        for (int idx = threadIdx.x; idx < valid * (D / 8); idx += TD_THREADS) {
            const int r = idx / (D / 8), d = (idx - r * (D / 8)) * 8;
            const float2* ml = reinterpret_cast<const float2*>(pml_base) + (size_t)r * n_splits;
            const float* pob = po_base + (size_t)r * n_splits * D + d;
            float2 mls[16];
            float4 v[16][2];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                if (k < n_splits) {
                    mls[k] = __ldcg(ml + k);
                    v[k][0] = __ldcg(reinterpret_cast<const float4*>(pob + (size_t)k * D));
                    v[k][1] = __ldcg(reinterpret_cast<const float4*>(pob + (size_t)k * D + 4));
                } else {
                    mls[k] = make_float2(-CUDART_INF_F, 0.f);
                    v[k][0] = v[k][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            float M = -CUDART_INF_F;
#pragma unroll
            for (int k = 0; k < 16; ++k) M = fmaxf(M, mls[k].x);
            float L = 0.f, a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                // a split without keys wrote (-inf, 0) and no result: left out, not multiplied by zero
                const float ws = (k >= n_splits || mls[k].x == -CUDART_INF_F) ? 0.f : exp2f(mls[k].x - M);
                if (ws != 0.f) {
                    L = fmaf(mls[k].y, ws, L);
                    a[0] = fmaf(v[k][0].x, ws, a[0]); a[1] = fmaf(v[k][0].y, ws, a[1]);
                    a[2] = fmaf(v[k][0].z, ws, a[2]); a[3] = fmaf(v[k][0].w, ws, a[3]);
                    a[4] = fmaf(v[k][1].x, ws, a[4]); a[5] = fmaf(v[k][1].y, ws, a[5]);
                    a[6] = fmaf(v[k][1].z, ws, a[6]); a[7] = fmaf(v[k][1].w, ws, a[7]);
                }
            }
            const float inv = 1.0f / L;
            uint4 w4;
            w4.x = pack_bf16(a[0] * inv, a[1] * inv);
            w4.y = pack_bf16(a[2] * inv, a[3] * inv);
            w4.z = pack_bf16(a[4] * inv, a[5] * inv);
            w4.w = pack_bf16(a[6] * inv, a[7] * inv);
            *reinterpret_cast<uint4*>(out_rows + (size_t)r * D + d) = w4;
        }
        return;
    }
    // Everything below waits on reads from L2, so each phase issues all of its loads at once.
    // (m, l) of every row and split in one go
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_ml = valid * n_splits;
    float* sm_m = wbuf;                                // [valid][n_splits]
    float* sm_l = wbuf + 16 * n_splits;
    float* sm_w = wbuf + 32 * n_splits;
    float* linv = wbuf + 48 * n_splits;                // [16]
    for (int i = threadIdx.x; i < n_ml; i += TD_THREADS) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(pml_base) + i);     // rows are n_splits pairs apart
        sm_m[i] = v.x;
        sm_l[i] = v.y;
    }
    __syncthreads();
    for (int r = warp; r < valid; r += TD_WARPS) {
        float M = -CUDART_INF_F;
        for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, sm_m[r * n_splits + s]);
        M = warp_max(M);
        float L = 0.f;
        for (int s = lane; s < n_splits; s += 32) {
            const float ms = sm_m[r * n_splits + s];
            const float w = ms == -CUDART_INF_F ? 0.f : exp2f(ms - M);
            sm_w[r * n_splits + s] = w;
            L += sm_l[r * n_splits + s] * w;
        }
        L = warp_sum(L);
        if (lane == 0) linv[r] = 1.0f / L;
    }
    __syncthreads();
    // four columns per thread, sixteen splits' loads in flight at a time; the sum stays in order
    for (int idx = threadIdx.x; idx < valid * (D / 4); idx += TD_THREADS) {
        const int r = idx / (D / 4), d = (idx - r * (D / 4)) * 4;
        const float* pob = po_base + (size_t)r * n_splits * D + d;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 16) {
            float4 v[16];
#pragma unroll
            for (int k = 0; k < 16; ++k)
                v[k] = s0 + k < n_splits ? __ldcg(reinterpret_cast<const float4*>(pob + (size_t)(s0 + k) * D))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const float ws = s0 + k < n_splits ? sm_w[r * n_splits + s0 + k] : 0.f;
                if (ws != 0.f) {
                    a0 = fmaf(v[k].x, ws, a0);
                    a1 = fmaf(v[k].y, ws, a1);
                    a2 = fmaf(v[k].z, ws, a2);
                    a3 = fmaf(v[k].w, ws, a3);
                }
            }
        }
        const float inv = linv[r];
        uint2 w2;
        w2.x = pack_bf16(a0 * inv, a1 * inv);
        w2.y = pack_bf16(a2 * inv, a3 * inv);
        *reinterpret_cast<uint2*>(out_rows + (size_t)r * D + d) = w2;
    }
}

// partial_o [n_tok, n_heads, n_splits, D] float (unnormalised), partial_ml [n_tok, n_heads, n_splits, 2].
//
// FUSED: the kernel also does what the rotary-and-append kernel does for a step of single tokens, so
// that a layer has one launch (and one wait for the kernel in front) fewer.  Every CTA adds up the
// partial sums of its own query heads, adds the bias, rotates them and keeps them in shared memory
// (the same operations in the same order as rope_cache_partials_vec_kernel, so the same bf16 values);
// the CTA whose split holds the token's own position does the same for the key and the value of its
// kv head, writes them to the cache for the steps to come and puts them into the row of its own tile
// that the bulk load filled from the cache before they were there.
template <int D, bool FUSED>
__global__ void __launch_bounds__(TD_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const bf16* __restrict__ q, int q_stride, const int* __restrict__ block_table,
                       int max_blocks, const int* __restrict__ tok_entry, const int* __restrict__ positions,
                       int tok_first, int n_heads, int n_kv, int page_size, int window, float scale_log2,
                       int chunk, int n_splits, float* __restrict__ partial_o, float* __restrict__ partial_ml,
                       bf16* __restrict__ out, int out_stride, int* __restrict__ counters,
                       int* __restrict__ err_flag, const FusedQkv fq) {
    using Plan = TdPlan<D>;
    using Layout = Swizzled128<D, 16>;
    constexpr int STAGES = Plan::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = tc::smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFFSET);       // [warp][stage]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + TD_WARPS * STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    TL_BEGIN();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        tc::prefetch_tensormap(&map_k);
        tc::prefetch_tensormap(&map_v);
        for (int i = 0; i < TD_WARPS * STAGES; ++i) tc::mbar_init(&bars[i], 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    // positions and block tables are set before the step's first kernel, and every cached key
    // but the token's own was written by earlier steps: all of that may be read before the
    // kernel in front (which writes q and the token's own key and value) has finished
    const int split = blockIdx.x;
    const int group = n_heads / n_kv;
    const int gtiles = (group + 15) / 16;
    const int kvh = blockIdx.y / gtiles, gt = blockIdx.y % gtiles;
    const int ti = blockIdx.z;
    const int t = tok_first + ti;
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_entry[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int base = (lo / KEYS16) * KEYS16;
    const int k_begin = base + split * chunk;
    const int k_end = min(pos + 1, k_begin + chunk);                  // exclusive
    const int h0 = kvh * group + gt * 16;
    const int valid = min(16, group - gt * 16);
    float* po = partial_o + (((size_t)ti * n_heads + h0) * n_splits + split) * D;
    float* pml = partial_ml + (((size_t)ti * n_heads + h0) * n_splits + split) * 2;
    if (k_begin >= k_end) {
        // nothing in this split: leave (m, l) = (-inf, 0) so the merge skips it
        pdl_wait();
        for (int r = threadIdx.x; r < valid; r += TD_THREADS) {
            pml[(size_t)r * n_splits * 2] = -CUDART_INF_F;
            pml[(size_t)r * n_splits * 2 + 1] = 0.f;
        }
        if (counters)
            merge_if_last<D>(counters + (size_t)ti * gridDim.y + blockIdx.y, reinterpret_cast<float*>(smem),
                             po - (size_t)split * D, pml - (size_t)split * 2, n_splits, valid,
                             out + (size_t)t * out_stride + (size_t)h0 * D);
        return;
    }
    float2* sc = reinterpret_cast<float2*>(smem + Plan::FUSED_OFFSET);            // [rotary_dim / 2] (sine, cosine)
    bf16* q_rows = reinterpret_cast<bf16*>(sc + D / 2);                            // [16][Q_STRIDE]
    bf16* k_new = q_rows + 16 * Plan::Q_STRIDE;                                    // [D]
    bf16* v_new = k_new + D;                                                       // [D]
    __syncthreads();

    uint8_t* my = smem + (size_t)warp * Plan::WARP_BYTES;
    uint64_t* my_bar = bars + warp * STAGES;
    const int n_slices = (k_end - k_begin + KEYS16 - 1) / KEYS16;
    const int my_slices = n_slices > warp ? (n_slices - warp + TD_WARPS - 1) / TD_WARPS : 0;
    const uint64_t policy = tc::policy_evict_first();                 // the cache is read once per step
    // The pages of the warp's slices, 32 at a time: lane l holds the page of slice base + l, so that the
    // look-ups in the block table are one round of loads, not one dependent load in front of every issue.
    int pages_base = 0;
    auto load_pages = [&](int base_slice) {
        const int i = base_slice + lane;
        int pg = -1;
        if (i < my_slices) pg = table[(k_begin + (warp + i * TD_WARPS) * KEYS16) / page_size];
        pages_base = base_slice;
        return pg;
    };
    int my_page = load_pages(0);
    // lane 0 issues the loads of the warp's i-th slice into stage i % STAGES
    auto issue = [&](int i) {
        if (i >= my_slices) return;                                   // (uniform over the warp)
        if (i >= pages_base + 32) my_page = load_pages(i);
        const int page = __shfl_sync(0xffffffffu, my_page, i - pages_base);
        if (lane == 0) {
            const int key0 = k_begin + (warp + i * TD_WARPS) * KEYS16;
            const int row = (page < 0 ? 0 : (page * n_kv + kvh) * page_size) + key0 % page_size;
            uint8_t* st = my + (size_t)(i % STAGES) * Plan::STAGE_BYTES;
            uint64_t* bar = &my_bar[i % STAGES];
            tc::mbar_expect_tx(bar, Plan::STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < D / 64; ++b) {
                tc::tma_load_2d_hint(st + b * 2048, &map_k, b * 64, row, bar, policy);
                tc::tma_load_2d_hint(st + Plan::HALF_BYTES + b * 2048, &map_v, b * 64, row, bar, policy);
            }
        }
    };
    // a slice that ends before the token's own position holds nothing of this step
    auto old_keys_only = [&](int i) { return k_begin + (warp + i * TD_WARPS) * KEYS16 + KEYS16 <= pos; };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i)
        if (old_keys_only(i)) issue(i);
    if (FUSED) {
        // the angles depend on the position alone: worked out while the first loads are on their way
        // (and, if this block could start early, while the product in front still runs)
        for (int i = threadIdx.x; i < (fq.rotary_dim >> 1); i += TD_THREADS) {
            float sn, cs;
            sincosf((float)pos * fq.inv_freq[i], &sn, &cs);
            sc[i] = make_float2(sn, cs);
        }
        __syncthreads();
    }
    pdl_wait();                                        // q and this step's key and value
    TL_MARK(51);
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i)
        if (!old_keys_only(i)) issue(i);

    uint32_t qf[D / 16][4];
    // does this CTA's split hold the token's own position?  Then the key and value of this step are its job.
    const bool own = FUSED && fq.write_cache && pos >= k_begin && pos < k_end;
    if (FUSED) {
        const float* src_row = fq.partial + (size_t)t * fq.row_width;
        float rstd = 1.0f;
        if (fq.sumsq_in) {
            // the tiles' sums in one round of loads: a lane per tile, added up across the warp
            float ss = 0.f;
            for (int tl = lane; tl < fq.in_tiles; tl += 32) ss += __ldcg(fq.sumsq_in + (size_t)tl * 256 + t);
            ss = warp_sum(ss);
            rstd = 1.0f / sqrtf(ss * fq.inv_d + fq.eps);
        }
        auto sum4 = [&](size_t col, float* v) {
            v[0] = v[1] = v[2] = v[3] = 0.f;
            // eight splits' loads in flight at a time; added in ascending order
            for (int s0 = 0; s0 < fq.splits; s0 += 8) {
                float4 f[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < fq.splits) f[k] = *reinterpret_cast<const float4*>(src_row + (size_t)(s0 + k) * fq.split_stride + col);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < fq.splits) { v[0] += f[k].x; v[1] += f[k].y; v[2] += f[k].z; v[3] += f[k].w; }
            }
            if (fq.sumsq_in) { v[0] *= rstd; v[1] *= rstd; v[2] *= rstd; v[3] *= rstd; }
            if (fq.bias) {
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += load_any(fq.bias, fq.bias_dtype, col + k);
            }
        };
        auto store4bf = [](bf16* p, const float* v) {
            uint2 u;
            u.x = pack_bf16(v[0], v[1]);
            u.y = pack_bf16(v[2], v[3]);
            *reinterpret_cast<uint2*>(p) = u;
        };
        // the two halves of a rotated chunk at once: all loads of both (and of their bias) are on their way
        // before the first addition, the additions in the same order as sum4's
        auto sum4x2 = [&](size_t col_a, size_t col_b, float* a, float* b) {
            float bias_a[4] = {0.f, 0.f, 0.f, 0.f}, bias_b[4] = {0.f, 0.f, 0.f, 0.f};
            if (fq.bias) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    bias_a[k] = load_any(fq.bias, fq.bias_dtype, col_a + k);
                    bias_b[k] = load_any(fq.bias, fq.bias_dtype, col_b + k);
                }
            }
            a[0] = a[1] = a[2] = a[3] = b[0] = b[1] = b[2] = b[3] = 0.f;
            for (int s0 = 0; s0 < fq.splits; s0 += 8) {
                float4 fa[8], fb[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < fq.splits) {
                        fa[k] = __ldcg(reinterpret_cast<const float4*>(src_row + (size_t)(s0 + k) * fq.split_stride + col_a));
                        fb[k] = __ldcg(reinterpret_cast<const float4*>(src_row + (size_t)(s0 + k) * fq.split_stride + col_b));
                    }
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < fq.splits) {
                        a[0] += fa[k].x; a[1] += fa[k].y; a[2] += fa[k].z; a[3] += fa[k].w;
                        b[0] += fb[k].x; b[1] += fb[k].y; b[2] += fb[k].z; b[3] += fb[k].w;
                    }
            }
            if (fq.sumsq_in) {
#pragma unroll
                for (int k = 0; k < 4; ++k) { a[k] *= rstd; b[k] *= rstd; }
            }
            if (fq.bias) {
#pragma unroll
                for (int k = 0; k < 4; ++k) { a[k] += bias_a[k]; b[k] += bias_b[k]; }
            }
        };
        const int half = fq.rotary_dim >> 1, hc = half >> 2, tail = (D - fq.rotary_dim) >> 2, per_head = hc + tail;
        const int n_q = valid * per_head, n_k = own ? per_head : 0, n_v = own ? D / 4 : 0;
        const int page = own ? table[pos / page_size] : -1;
        // (only one of the CTAs that share a kv head writes the cache; all of them need the values)
        const size_t cache_row = ((size_t)(page < 0 ? 0 : page) * n_kv + kvh) * page_size * D + (size_t)(pos % page_size) * D;
        const bool to_cache = own && page >= 0 && gt == 0;
        for (int it = threadIdx.x; it < n_q + n_k + n_v; it += TD_THREADS) {
            if (it < n_q + n_k) {
                const bool is_q = it < n_q;
                const int r = is_q ? it / per_head : 0, c = (is_q ? it : it - n_q) - r * per_head;
                const size_t col0 = (size_t)(is_q ? h0 + r : n_heads + kvh) * D;
                bf16* dst = is_q ? q_rows + r * Plan::Q_STRIDE : k_new;
                if (c < hc) {
                    float a[4], b[4], ra[4], rb[4];
                    sum4x2(col0 + c * 4, col0 + half + c * 4, a, b);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 s1 = sc[c * 4 + k];
                        ra[k] = a[k] * s1.y - b[k] * s1.x;
                        rb[k] = a[k] * s1.x + b[k] * s1.y;
                    }
                    store4bf(dst + c * 4, ra);
                    store4bf(dst + half + c * 4, rb);
                    if (!is_q && to_cache) {
                        store4bf(fq.k_cache + cache_row + c * 4, ra);
                        store4bf(fq.k_cache + cache_row + half + c * 4, rb);
                    }
                } else {
                    float v[4];
                    const int d0 = fq.rotary_dim + (c - hc) * 4;
                    sum4(col0 + d0, v);
                    store4bf(dst + d0, v);
                    if (!is_q && to_cache) store4bf(fq.k_cache + cache_row + d0, v);
                }
            } else {
                const int c = it - n_q - n_k;
                float v[4];
                sum4((size_t)(n_heads + n_kv + kvh) * D + c * 4, v);
                store4bf(v_new + c * 4, v);
                if (to_cache) store4bf(fq.v_cache + cache_row + c * 4, v);
            }
        }
        __syncthreads();
        TL_MARK(52);
        load_q<D>(qf, q_rows, (size_t)Plan::Q_STRIDE, valid, lane);
    } else {
        load_q<D>(qf, q + (size_t)t * q_stride + (size_t)h0 * D, (size_t)D, valid, lane);
    }
    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    bool ok = true;
    int waited = 0;
    for (int i = 0; i < my_slices; ++i) {
        issue(i + STAGES - 1);                                        // the stage the last iteration left
        if (!tc::mbar_wait(&my_bar[i % STAGES], (uint32_t)(i / STAGES) & 1u, abort_flag)) { ok = false; break; }
        waited = i + 1;
        const bf16* kt = reinterpret_cast<const bf16*>(my + (size_t)(i % STAGES) * Plan::STAGE_BYTES);
        const bf16* vt = kt + 16 * D;
        const int kb = k_begin + (warp + i * TD_WARPS) * KEYS16;
        if (own && pos >= kb && pos < kb + KEYS16) {
            // the slice with the token's own position came from the cache before this step's key and
            // value were there: put them into its row (the layout the bulk load leaves, 16 bytes per lane)
            const int row = pos - kb;
            if (lane < D / 8) {
                *reinterpret_cast<uint4*>(const_cast<bf16*>(kt) + (size_t)Layout::chunk(row, lane) * 8) =
                    *reinterpret_cast<const uint4*>(k_new + lane * 8);
                *reinterpret_cast<uint4*>(const_cast<bf16*>(vt) + (size_t)Layout::chunk(row, lane) * 8) =
                    *reinterpret_cast<const uint4*>(v_new + lane * 8);
            }
            __syncwarp();
        }
        slice16<D, Layout>(qf, kt, vt, 0, kb, lo, pos, lo, pos, scale_log2, m, l, o, lane);
        __syncwarp();
    }
    if (!ok) {
        // a load never arrived: report, and let what is still in flight land before the block
        // (and its shared memory) goes away
        if (lane == 0) {
            *abort_flag = 1;
            atomicExch(err_flag, 4);
        }
        volatile int never = 0;
        const int issued = min(my_slices, waited + STAGES);
        for (int i = waited; i < issued; ++i)
            tc::mbar_wait(&my_bar[i % STAGES], (uint32_t)(i / STAGES) & 1u, &never);
    }
    TL_MARK(53);
    // ---- merge the four warps ----------------------------------------------------------------------
    float l0 = l[0], l1 = l[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();                                   // every warp is done with its stages
    constexpr int RS = Plan::RED_STRIDE;
    float* red_o = reinterpret_cast<float*>(smem);                    // [4 warps][16 rows][RS]
    float* red_ml = red_o + TD_WARPS * 16 * RS;                       // [4 warps][16 rows][2]
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int d = nt * 8 + c * 2;
        float* r0 = red_o + ((size_t)warp * 16 + g) * RS + d;
        float* r1 = red_o + ((size_t)warp * 16 + g + 8) * RS + d;
        *reinterpret_cast<float2*>(r0) = make_float2(o[nt][0], o[nt][1]);
        *reinterpret_cast<float2*>(r1) = make_float2(o[nt][2], o[nt][3]);
    }
    if (c == 0) {
        red_ml[((size_t)warp * 16 + g) * 2] = m[0];
        red_ml[((size_t)warp * 16 + g) * 2 + 1] = l0;
        red_ml[((size_t)warp * 16 + g + 8) * 2] = m[1];
        red_ml[((size_t)warp * 16 + g + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    // per row: the common maximum and each warp's factor 2^(m_w - max); every thread works them out for the
    // row of its own columns (four values from shared memory), the thread at the row's first columns also
    // writes the row's (m, l)
    for (int idx = threadIdx.x; idx < valid * (D / 4); idx += TD_THREADS) {
        const int r = idx / (D / 4), d = (idx - r * (D / 4)) * 4;
        float mw[TD_WARPS], f[TD_WARPS], mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < TD_WARPS; ++w) {
            mw[w] = red_ml[((size_t)w * 16 + r) * 2];
            mm = fmaxf(mm, mw[w]);
        }
#pragma unroll
        for (int w = 0; w < TD_WARPS; ++w) f[w] = mw[w] == -CUDART_INF_F ? 0.f : exp2f(mw[w] - mm);
        if (d == 0) {
            float ll = 0.f;
#pragma unroll
            for (int w = 0; w < TD_WARPS; ++w) ll += red_ml[((size_t)w * 16 + r) * 2 + 1] * f[w];
            pml[(size_t)r * n_splits * 2] = mm;
            pml[(size_t)r * n_splits * 2 + 1] = ll;
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < TD_WARPS; ++w) {
            const float4 v = *reinterpret_cast<const float4*>(red_o + ((size_t)w * 16 + r) * RS + d);
            acc.x += v.x * f[w]; acc.y += v.y * f[w]; acc.z += v.z * f[w]; acc.w += v.w * f[w];
        }
        *reinterpret_cast<float4*>(po + (size_t)r * n_splits * D + d) = acc;
    }
    TL_MARK(54);
    if (counters)                                      // (its first barrier also ends the reads of red_o above)
        merge_if_last<D>(counters + (size_t)ti * gridDim.y + blockIdx.y, reinterpret_cast<float*>(smem),
                         po - (size_t)split * D, pml - (size_t)split * 2, n_splits, valid,
                         out + (size_t)t * out_stride + (size_t)h0 * D);
    TL_END(TL_ATTN_DECODE);
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M = max_s m_s; splits in
// ascending order.  One warp per (token, head): the weights of the splits are worked out once
// (lanes over splits), then every lane sums its columns with the loads of all splits in flight.
constexpr int COMBINE_MAX_SPLITS = 256;
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                    bf16* __restrict__ out, int out_stride, int tok_first, int n_tok, int n_heads,
                    int n_splits, int head_dim) {
    __shared__ float wsm[4][COMBINE_MAX_SPLITS];
    pdl_launch_dependents();
    pdl_wait();
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warp = blockIdx.x * 4 + wib;
    if (warp >= n_tok * n_heads) return;
    const int ti = warp / n_heads, h = warp % n_heads;
    const float* ml = partial_ml + (size_t)warp * n_splits * 2;
    const float* po = partial_o + (size_t)warp * n_splits * head_dim;
    float* wgt = wsm[wib];
    float M = -CUDART_INF_F;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, ml[s * 2]);
    M = warp_max(M);
    for (int s = lane; s < n_splits; s += 32) {
        const float ms = ml[s * 2];
        wgt[s] = ms == -CUDART_INF_F ? 0.f : exp2f(ms - M);
    }
    __syncwarp();
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) L += ml[s * 2 + 1] * wgt[s];    // ascending, same in every lane (l is written for every split)
    const float inv = 1.0f / L;
    bf16* orow = out + (size_t)(tok_first + ti) * out_stride + (size_t)h * head_dim;
    for (int d = lane * 2; d < head_dim; d += 64) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) {
            // a split without keys has weight 0 and wrote no partial output: what lies there is
            // whatever the memory held (possibly NaN), so it is left out, not multiplied by 0
            const float ws = wgt[s];
            float2 v = *reinterpret_cast<const float2*>(po + (size_t)s * head_dim + d);
            if (ws == 0.f) v = make_float2(0.f, 0.f);
            a0 = fmaf(v.x, ws, a0);
            a1 = fmaf(v.y, ws, a1);
        }
        *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16(a0 * inv, a1 * inv);
    }
}

template <int D, bool FUSED>
int launch_tma(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_stride, const int* block_table,
               int max_blocks, const int* tok_entry, const int* positions, int tok_first, int n_tok, int n_heads,
               int n_kv, int page_size, int window, float scale_log2, int chunk, int n_splits, float* po, float* pml,
               void* out, int out_stride, int* counters, int* err, const FusedQkv& fq, cudaStream_t stream) {
    using Plan = TdPlan<D>;
    constexpr int SMEM = FUSED ? Plan::TOTAL_FUSED : Plan::TOTAL;
    auto kern = attn_decode_tma_kernel<D, FUSED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) {
            infero_set_error("attn_decode_tma: cannot get %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
            return 1;
        }
        configured = true;
    }
    const int group = n_heads / n_kv;
    dim3 grid(n_splits, n_kv * ((group + 15) / 16), n_tok);
    launch_pdl(kern, grid, dim3(TD_THREADS), SMEM, stream, mk, mv, (const bf16*)q, q_stride, block_table,
               max_blocks, tok_entry, positions, tok_first, n_heads, n_kv, page_size, window, scale_log2, chunk,
               n_splits, po, pml, (bf16*)out, out_stride, counters, err, fq);
    return infero_check_launch(FUSED ? "attn_decode_tma_fused" : "attn_decode_tma");
}

// Checks, maps and the launch shared by the two entry points below (fq.partial null: finished queries in q).
int decode_tma(const void* q, int q_stride, const FusedQkv& fq, void* out, int out_stride, const void* k_cache,
               const void* v_cache, int num_pages, const int* block_table, int max_blocks, const int* tok_entry,
               const int* positions, int tok_first, int n_tok, int n_heads, int n_kv, int head_dim, int page_size,
               int window, float scale, int chunk, int n_splits, void* scratch, int* counters, int n_counters,
               cudaStream_t stream) {
    if (n_tok == 0) return 0;
    INFERO_REQUIRE(infero_attn_decode_tma_supported(head_dim, page_size),
                   "attn_decode_tma: head_dim %d / page_size %d not supported", head_dim, page_size);
    INFERO_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attn_decode_tma: bad head counts %d / %d", n_heads, n_kv);
    INFERO_REQUIRE(chunk > 0 && chunk % 16 == 0 && n_splits >= 1 && n_splits <= COMBINE_MAX_SPLITS,
                   "attn_decode_tma: bad split plan chunk=%d splits=%d", chunk, n_splits);
    INFERO_REQUIRE(n_tok <= 65535 && (long long)num_pages * n_kv * page_size < (1ll << 31),
                   "attn_decode_tma: %d tokens / %d pages in one call", n_tok, num_pages);
    INFERO_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0, "attn_decode_tma: odd row stride");
    CUtensorMap mk, mv;
    const int rows = num_pages * n_kv * page_size;
    if (infero_tensor_map_bf16(k_cache, rows, head_dim, head_dim, 16, &mk)) return 1;
    if (infero_tensor_map_bf16(v_cache, rows, head_dim, head_dim, 16, &mv)) return 1;
    int* err;
    if (infero_tc_err_flag(&err)) return 1;
    if (counters) {
        // more groups of splits than counters: the separate merge kernel does it
        const long long groups = (long long)n_tok * n_kv * ((n_heads / n_kv + 15) / 16);
        if (groups > n_counters) counters = nullptr;
    }
    const float sl2 = scale * 1.4426950408889634f;
    float* po = (float*)scratch;
    float* pml = po + (size_t)n_tok * n_heads * n_splits * head_dim;
    int rc;
#define GO(D_, F_)                                                                                                   \
    rc = launch_tma<D_, F_>(mk, mv, q, q_stride, block_table, max_blocks, tok_entry, positions, tok_first, n_tok,   \
                            n_heads, n_kv, page_size, window, sl2, chunk, n_splits, po, pml, out, out_stride,       \
                            counters, err, fq, stream)
    if (head_dim == 128) {
        if (fq.partial) GO(128, true); else GO(128, false);
    } else {
        if (fq.partial) GO(64, true); else GO(64, false);
    }
#undef GO
    if (rc || counters) return rc;                     // merged by the last CTA of every group
    const int warps = n_tok * n_heads;
    launch_pdl(attn_combine_kernel, dim3((warps + 3) / 4), dim3(128), 0, stream, (const float*)po, (const float*)pml,
               (bf16*)out, out_stride, tok_first, n_tok, n_heads, n_splits, head_dim);
    return infero_check_launch("attn_combine");
}

}  // namespace

extern "C" {

int infero_attn_decode_tma_supported(int head_dim, int page_size) {
    return (head_dim == 64 || head_dim == 128) && page_size % 16 == 0;
}

// The same contract as infero_attn_decode (attention_mma.cu), plus num_pages: the caches are
// [num_pages, n_kv, page_size, head_dim] bf16, contiguous and 16-byte aligned.  n_splits is
// at most 256.  scratch: infero_attn_decode_scratch bytes.  counters: n_counters ints, zero before the
// first call (each launch leaves them zero again); with n_tok * n_kv * ceil(group / 16) of them or more
// the last CTA of every group of splits merges the group; with fewer, or none (null), a second kernel does.
int infero_attn_decode_tma(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                           const void* v_cache, int num_pages, const int* block_table, int max_blocks,
                           const int* tok_entry, const int* positions, int tok_first, int n_tok, int n_heads,
                           int n_kv, int head_dim, int page_size, int window, float scale, int chunk, int n_splits,
                           void* scratch, int* counters, int n_counters, cudaStream_t stream) {
    FusedQkv none = {};
    return decode_tma(q, q_stride, none, out, out_stride, k_cache, v_cache, num_pages, block_table, max_blocks, tok_entry,
                      positions, tok_first, n_tok, n_heads, n_kv, head_dim, page_size, window, scale, chunk, n_splits,
                      scratch, counters, n_counters, stream);
}

// Can the kernel below finish the q/k/v product itself?  (The vector widths its loads and stores use.)
int infero_attn_decode_fused_supported(const float* partial, long long split_stride, int n_heads, int n_kv,
                                       int head_dim, int page_size, int rotary_dim, const void* k_cache,
                                       const void* v_cache) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return infero_attn_decode_tma_supported(head_dim, page_size) && rotary_dim >= 0 && rotary_dim % 8 == 0 &&
           rotary_dim <= head_dim && split_stride % 4 == 0 && al16(partial) && al16(k_cache) && al16(v_cache) &&
           n_kv > 0 && n_heads % n_kv == 0;
}

// Rotary positions, cache append and decode attention of a step's single tokens in one launch.  Takes
// the q/k/v product as the few-token product kernel leaves it: partial[s][t][(n_heads + 2 n_kv) * head_dim]
// 32-bit, s < splits, split_stride elements apart, rows indexed by the token's place in the step; bias
// (bias_dtype) may be null.  The queries are rotated and used, never written; with write_cache the keys
// and values of the tokens are appended to the cache as infero_rope_cache_partials appends them (the same
// bf16 values).  sumsq (may be null): the product's input lacked its norm's scalar, see FusedQkv.
// Everything else as infero_attn_decode_tma.
int infero_attn_decode_tma_fused(const float* partial, int splits, long long split_stride, const void* bias,
                                 int bias_dtype, const float* inv_freq, int rotary_dim, int write_cache, void* out,
                                 int out_stride, void* k_cache, void* v_cache, int num_pages, const int* block_table,
                                 int max_blocks, const int* tok_entry, const int* positions, int tok_first, int n_tok,
                                 int n_heads, int n_kv, int head_dim, int page_size, int window, float scale, int chunk,
                                 int n_splits, void* scratch, int* counters, int n_counters, const float* sumsq,
                                 int sumsq_tiles, float inv_d, float eps, cudaStream_t stream) {
    INFERO_REQUIRE(partial && splits >= 1, "attn_decode_tma_fused: no partial sums (%d splits)", splits);
    INFERO_REQUIRE(infero_attn_decode_fused_supported(partial, split_stride, n_heads, n_kv, head_dim, page_size, rotary_dim,
                                                      k_cache, v_cache),
                   "attn_decode_tma_fused: head_dim %d / rotary_dim %d / split stride %lld not supported", head_dim,
                   rotary_dim, split_stride);
    FusedQkv fq;
    fq.partial = partial, fq.split_stride = split_stride, fq.bias = bias, fq.inv_freq = inv_freq;
    fq.k_cache = (bf16*)k_cache, fq.v_cache = (bf16*)v_cache, fq.splits = splits;
    fq.row_width = (n_heads + 2 * n_kv) * head_dim, fq.bias_dtype = bias_dtype, fq.rotary_dim = rotary_dim;
    fq.write_cache = write_cache;
    fq.sumsq_in = sumsq, fq.in_tiles = sumsq_tiles, fq.inv_d = inv_d, fq.eps = eps;
    return decode_tma(nullptr, 0, fq, out, out_stride, k_cache, v_cache, num_pages, block_table, max_blocks, tok_entry,
                      positions, tok_first, n_tok, n_heads, n_kv, head_dim, page_size, window, scale, chunk, n_splits,
                      scratch, counters, n_counters, stream);
}

}  // extern "C"

INFERO_TL_UNIT(attention_decode)
