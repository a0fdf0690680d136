// bf16 attention over the paged cache on the warp-level tensor cores (mma.sync m16n8k16),
// in two kernels that share their inner pieces:
//
//   attn_prefill: one CTA = 64 consecutive query tokens of one request and one head.  Four
//     warps own 16 query rows each; key/value tiles of 64 positions are gathered page by page
//     into shared memory with cp.async (two stages) and shared by the four warps.
//   attn_decode: one CTA = one token, one kv head (its whole group of query heads forms the
//     16 rows of the MMA) and one split of the context.  Each warp walks its own 16-key
//     slices with its own cp.async ring; the four warps are merged in shared memory and the
//     CTA writes an unnormalised partial result (o, m, l) that attn_combine merges over the
//     splits.  The grid depends on the batch size and a context bound only, so a decode step
//     can be replayed as a CUDA graph while the requests grow.
//
// Both follow the same formula as the generic kernel (attention_generic.cu): scores
// q.k * scale over lo <= j <= pos with lo = max(0, pos - window + 1), softmax with running
// maximum and sum in 32-bit, weighted sum of v.  Scores and statistics are 32-bit; the
// probabilities are rounded to bf16 for the second product, as the keys and values are.
// Reference: crates/kernels/src/cu/ops.cu:1773-2075 (fused decode with split context),
// :1465-1494 (merge of the splits), attn_prefill_mma_ws4 (kernels/src/lib.rs:3717).
//
// Head sizes: multiples of 16 up to 128 (template instances); anything else is refused and
// the caller falls back to the generic kernel.  Any number of heads and any group size.
#include "attn_common.cuh"

namespace {

using namespace attn;

// ---- prefill -------------------------------------------------------------------------------------
constexpr int PF_ROWS = 64, PF_KEYS = 64, PF_THREADS = 128;

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                    const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ entry_q_start,
                    const int* __restrict__ entry_q_len, const int* __restrict__ entry_pos0, int n_entries,
                    int first_entry, int n_heads, int n_kv, int page_size, int window, float scale_log2) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    bf16* tiles = reinterpret_cast<bf16*>(smem_raw);          // [2 stages][K | V][64 rows][D]
    constexpr int TILE = tile_elems<D>(PF_KEYS);

    // which request and which block of 64 query rows is this CTA's?
    int e = -1, tile_in_e = 0;
    {
        int left = blockIdx.x;
        for (int i = first_entry; i < n_entries; ++i) {
            const int ql = entry_q_len[i];
            const int nt = (ql + PF_ROWS - 1) / PF_ROWS;
            if (left < nt) { e = i; tile_in_e = left; break; }
            left -= nt;
        }
    }
    if (e < 0) return;
    const int h = blockIdx.y, kvh = h / (n_heads / n_kv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int q_len = entry_q_len[e], pos0 = entry_pos0[e], tok0 = entry_q_start[e];
    const int* table = block_table + (size_t)e * max_blocks;
    const int row_first = tile_in_e * PF_ROWS;                        // first query row of the CTA (within the request's portion)
    const int rows_here = min(PF_ROWS, q_len - row_first);
    const int wrow = row_first + warp * 16;                           // first row of the warp
    const int wvalid = max(0, min(16, q_len - wrow));

    uint32_t qf[D / 16][4];
    load_q<D>(qf, q + (size_t)(tok0 + wrow) * q_stride + (size_t)h * D, (size_t)q_stride, wvalid, lane);

    // visible keys of the thread's two rows
    const int p0 = pos0 + wrow + g, p1 = p0 + 8;
    const int hi0 = (g < wvalid) ? p0 : -1, hi1 = (g + 8 < wvalid) ? p1 : -1;
    const int lo0 = window > 0 ? max(0, p0 - window + 1) : 0, lo1 = window > 0 ? max(0, p1 - window + 1) : 0;
    // keys the CTA needs: from the first row's window start to the last row's position
    const int cta_hi = pos0 + row_first + rows_here - 1;              // inclusive
    const int cta_lo = window > 0 ? max(0, pos0 + row_first - window + 1) : 0;
    const int key_begin = (cta_lo / PF_KEYS) * PF_KEYS;
    const int n_tiles = (cta_hi - key_begin) / PF_KEYS + 1;
    const int warp_hi = pos0 + wrow + wvalid - 1;                     // last key any row of this warp sees
    const int warp_lo = window > 0 ? max(0, pos0 + wrow - window + 1) : 0;

    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    auto issue = [&](int t) {
        bf16* kt = tiles + (size_t)(t & 1) * 2 * TILE;
        const int key0 = key_begin + t * PF_KEYS;
        gather_rows<D>(kt, k_cache, table, key0, PF_KEYS, cta_hi + 1, n_kv, kvh, page_size, threadIdx.x, PF_THREADS);
        gather_rows<D>(kt + TILE, v_cache, table, key0, PF_KEYS, cta_hi + 1, n_kv, kvh, page_size, threadIdx.x, PF_THREADS);
        cp_async_commit();
    };
    issue(0);
    for (int t = 0; t < n_tiles; ++t) {
        if (t + 1 < n_tiles) issue(t + 1);
        else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kt = tiles + (size_t)(t & 1) * 2 * TILE;
        const int key0 = key_begin + t * PF_KEYS;
        if (wvalid > 0 && key0 <= warp_hi && key0 + PF_KEYS > warp_lo) {
#pragma unroll 1
            for (int sl = 0; sl < PF_KEYS / KEYS16; ++sl) {
                const int kb = key0 + sl * KEYS16;
                if (kb > warp_hi || kb + KEYS16 <= warp_lo) continue;
                slice16<D>(qf, kt, kt + TILE, sl * KEYS16, kb, lo0, hi0, lo1, hi1, scale_log2, m, l, o, lane);
            }
        }
        __syncthreads();
    }
    // ---- write: o / l -----------------------------------------------------------------------------
    float l0 = l[0], l1 = l[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
    bf16* orow0 = out + (size_t)(tok0 + wrow + g) * out_stride + (size_t)h * D;
    bf16* orow1 = orow0 + (size_t)8 * out_stride;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int d = nt * 8 + c * 2;
        if (g < wvalid) *reinterpret_cast<uint32_t*>(orow0 + d) = pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
        if (g + 8 < wvalid) *reinterpret_cast<uint32_t*>(orow1 + d) = pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
    }
}

// ---- decode ----------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 4, DEC_THREADS = DEC_WARPS * 32, DEC_STAGES = 2;

// partial_o [n_tok, n_heads, n_splits, D] float (unnormalised), partial_ml [n_tok, n_heads, n_splits, 2].
template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                   const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ tok_entry, const int* __restrict__ positions, int tok_first,
                   int n_heads, int n_kv, int page_size, int window, float scale_log2, int chunk,
                   int n_splits, float* __restrict__ partial_o, float* __restrict__ partial_ml) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int TILE = tile_elems<D>(KEYS16);                       // elements of one 16-key slice
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int split = blockIdx.x;
    const int group = n_heads / n_kv;
    const int gtiles = (group + 15) / 16;
    const int kvh = blockIdx.y / gtiles, gt = blockIdx.y % gtiles;
    const int ti = blockIdx.z;                                        // index among this launch's tokens
    const int t = tok_first + ti;
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_entry[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int base = (lo / KEYS16) * KEYS16;                          // splits start at the window's first slice
    const int k_begin = base + split * chunk;
    const int k_end = min(pos + 1, k_begin + chunk);                  // exclusive
    const int h0 = kvh * group + gt * 16;                             // first query head of the CTA
    const int valid = min(16, group - gt * 16);
    float* po = partial_o + (((size_t)ti * n_heads + h0) * n_splits + split) * D;
    float* pml = partial_ml + (((size_t)ti * n_heads + h0) * n_splits + split) * 2;
    if (k_begin >= k_end) {
        // nothing in this split: leave (m, l) = (-inf, 0) so the merge skips it
        for (int r = threadIdx.x; r < valid; r += DEC_THREADS) {
            pml[(size_t)r * n_splits * 2] = -CUDART_INF_F;
            pml[(size_t)r * n_splits * 2 + 1] = 0.f;
        }
        return;
    }
    bf16* my = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * DEC_STAGES * 2 * TILE;

    uint32_t qf[D / 16][4];
    load_q<D>(qf, q + (size_t)t * q_stride + (size_t)h0 * D, (size_t)D, valid, lane);
    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const int n_slices = (k_end - k_begin + KEYS16 - 1) / KEYS16;
    // warp w takes slices w, w + 4, ...
    auto issue = [&](int i) {
        const int sl = warp + i * DEC_WARPS;
        if (sl < n_slices) {
            bf16* kt = my + (size_t)(i % DEC_STAGES) * 2 * TILE;
            const int key0 = k_begin + sl * KEYS16;
            gather_rows<D>(kt, k_cache, table, key0, KEYS16, pos + 1, n_kv, kvh, page_size, lane, 32);
            gather_rows<D>(kt + TILE, v_cache, table, key0, KEYS16, pos + 1, n_kv, kvh, page_size, lane, 32);
        }
        cp_async_commit();
    };
    const int my_slices = (n_slices - warp + DEC_WARPS - 1) / DEC_WARPS;
    issue(0);
    for (int i = 0; i < my_slices; ++i) {
        issue(i + 1);
        cp_async_wait<1>();
        __syncwarp();
        const bf16* kt = my + (size_t)(i % DEC_STAGES) * 2 * TILE;
        const int kb = k_begin + (warp + i * DEC_WARPS) * KEYS16;
        slice16<D>(qf, kt, kt + TILE, 0, kb, lo, pos, lo, pos, scale_log2, m, l, o, lane);
        __syncwarp();
    }
    cp_async_wait<0>();
    // ---- merge the four warps ----------------------------------------------------------------------
    float l0 = l[0], l1 = l[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();                                   // every warp is done with its tiles
    float* red_o = reinterpret_cast<float*>(smem_raw);               // [4 warps][16 rows][D]
    float* red_ml = red_o + DEC_WARPS * 16 * D;                       // [4 warps][16 rows][2]
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int d = nt * 8 + c * 2;
        float* r0 = red_o + ((size_t)warp * 16 + g) * D + d;
        float* r1 = red_o + ((size_t)warp * 16 + g + 8) * D + d;
        r0[0] = o[nt][0]; r0[1] = o[nt][1];
        r1[0] = o[nt][2]; r1[1] = o[nt][3];
    }
    if (c == 0) {
        red_ml[((size_t)warp * 16 + g) * 2] = m[0];
        red_ml[((size_t)warp * 16 + g) * 2 + 1] = l0;
        red_ml[((size_t)warp * 16 + g + 8) * 2] = m[1];
        red_ml[((size_t)warp * 16 + g + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < valid * D; idx += DEC_THREADS) {
        const int r = idx / D, d = idx - r * D;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_ml[((size_t)w * 16 + r) * 2]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = red_ml[((size_t)w * 16 + r) * 2];
            const float f = mw == -CUDART_INF_F ? 0.f : exp2f(mw - mm);
            acc += red_o[((size_t)w * 16 + r) * D + d] * f;
            ll += red_ml[((size_t)w * 16 + r) * 2 + 1] * f;
        }
        po[(size_t)r * n_splits * D + d] = acc;
        if (d == 0) {
            pml[(size_t)r * n_splits * 2] = mm;
            pml[(size_t)r * n_splits * 2 + 1] = ll;
        }
    }
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M = max_s m_s; splits in
// ascending order.  One warp per (token, head).
__global__ void attn_combine_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                    bf16* __restrict__ out, int out_stride, int tok_first, int n_tok, int n_heads,
                                    int n_splits, int head_dim) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tok * n_heads) return;
    const int ti = warp / n_heads, h = warp % n_heads;
    const float* ml = partial_ml + (size_t)warp * n_splits * 2;
    const float* po = partial_o + (size_t)warp * n_splits * head_dim;
    float M = -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[s * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = ml[s * 2];
        if (ms != -CUDART_INF_F) L += ml[s * 2 + 1] * exp2f(ms - M);
    }
    const float inv = 1.0f / L;
    bf16* orow = out + (size_t)(tok_first + ti) * out_stride + (size_t)h * head_dim;
    for (int d = lane; d < head_dim; d += 32) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = ml[s * 2];
            if (ms != -CUDART_INF_F) acc += po[(size_t)s * head_dim + d] * exp2f(ms - M);
        }
        orow[d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int D>
int launch_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_cache, const void* v_cache,
                   const int* block_table, int max_blocks, const int* entry_q_start, const int* entry_q_len,
                   const int* entry_pos0, int n_entries, int first_entry, int n_tiles, int n_heads, int n_kv,
                   int page_size, int window, float scale_log2, cudaStream_t stream) {
    auto kern = attn_prefill_kernel<D>;
    const int smem = 2 * 2 * tile_elems<D>(PF_KEYS) * 2;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        configured = true;
    }
    dim3 grid(n_tiles, n_heads);
    launch_pdl(kern, grid, dim3(PF_THREADS), smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride,
               (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, entry_q_start, entry_q_len,
               entry_pos0, n_entries, first_entry, n_heads, n_kv, page_size, window, scale_log2);
    return infero_check_launch("attn_prefill");
}

template <int D>
int launch_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                  int max_blocks, const int* tok_entry, const int* positions, int tok_first, int n_tok, int n_heads,
                  int n_kv, int page_size, int window, float scale_log2, int chunk, int n_splits, float* partial_o,
                  float* partial_ml, cudaStream_t stream) {
    auto kern = attn_decode_kernel<D>;
    const int tiles_bytes = DEC_WARPS * DEC_STAGES * 2 * tile_elems<D>(KEYS16) * 2;
    const int red_bytes = DEC_WARPS * 16 * (D + 2) * 4;
    const int smem = tiles_bytes > red_bytes ? tiles_bytes : red_bytes;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        configured = true;
    }
    const int group = n_heads / n_kv;
    dim3 grid(n_splits, n_kv * ((group + 15) / 16), n_tok);
    kern<<<grid, DEC_THREADS, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)k_cache, (const bf16*)v_cache,
                                              block_table, max_blocks, tok_entry, positions, tok_first, n_heads, n_kv,
                                              page_size, window, scale_log2, chunk, n_splits, partial_o, partial_ml);
    return infero_check_launch("attn_decode");
}

}  // namespace

extern "C" {

int infero_attn_mma_supported(int head_dim, int page_size) {
    return head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0 && page_size % 16 == 0;
}

#define DISPATCH_D(D_, CALL)                                                                 \
    switch (D_) {                                                                            \
        case 16: return CALL(16);                                                            \
        case 32: return CALL(32);                                                            \
        case 48: return CALL(48);                                                            \
        case 64: return CALL(64);                                                            \
        case 80: return CALL(80);                                                            \
        case 96: return CALL(96);                                                            \
        case 112: return CALL(112);                                                          \
        case 128: return CALL(128);                                                          \
    }

// Attention for requests first_entry .. n_entries - 1 of a step (bf16), each with any number
// of new tokens.  n_tiles = sum over those requests of ceil(q_len / 64).  q / out rows are indexed by the
// step's token index.
int infero_attn_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                        const void* v_cache, const int* block_table, int max_blocks, const int* entry_q_start,
                        const int* entry_q_len, const int* entry_pos0, int n_entries, int first_entry, int n_tiles,
                        int n_heads, int n_kv, int head_dim, int page_size, int window, float scale,
                        cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    INFERO_REQUIRE(infero_attn_mma_supported(head_dim, page_size), "attn_prefill: head_dim %d / page_size %d not supported", head_dim, page_size);
    INFERO_REQUIRE(n_kv > 0 && n_heads % n_kv == 0 && n_heads <= 65535, "attn_prefill: bad head counts %d / %d", n_heads, n_kv);
    INFERO_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0, "attn_prefill: odd row strides");
    const float sl2 = scale * 1.4426950408889634f;
#define CALL(D_) launch_prefill<D_>(q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_blocks, entry_q_start, entry_q_len, entry_pos0, n_entries, first_entry, n_tiles, n_heads, n_kv, page_size, window, sl2, stream)
    DISPATCH_D(head_dim, CALL)
#undef CALL
    infero_set_error("attn_prefill: head_dim %d has no instance", head_dim);
    return 1;
}

// Bytes of 32-bit scratch a decode call needs (partial outputs and their statistics).
long long infero_attn_decode_scratch(int n_tok, int n_heads, int head_dim, int n_splits) {
    return (long long)n_tok * n_heads * n_splits * (head_dim + 2) * 4;
}

// Attention for n_tok single-token requests: tokens tok_first .. tok_first + n_tok - 1 of the
// step.  chunk (keys per split, a multiple of 16) times n_splits must cover the longest
// visible context.  scratch: infero_attn_decode_scratch bytes.
int infero_attn_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                       const void* v_cache, const int* block_table, int max_blocks, const int* tok_entry,
                       const int* positions, int tok_first, int n_tok, int n_heads, int n_kv, int head_dim,
                       int page_size, int window, float scale, int chunk, int n_splits, void* scratch,
                       cudaStream_t stream) {
    if (n_tok == 0) return 0;
    INFERO_REQUIRE(infero_attn_mma_supported(head_dim, page_size), "attn_decode: head_dim %d / page_size %d not supported", head_dim, page_size);
    INFERO_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attn_decode: bad head counts %d / %d", n_heads, n_kv);
    INFERO_REQUIRE(chunk > 0 && chunk % 16 == 0 && n_splits >= 1 && n_splits <= 65535, "attn_decode: bad split plan chunk=%d splits=%d", chunk, n_splits);
    INFERO_REQUIRE(n_tok <= 65535, "attn_decode: %d tokens in one call", n_tok);
    INFERO_REQUIRE(q_stride % 2 == 0, "attn_decode: odd row stride");
    const float sl2 = scale * 1.4426950408889634f;
    float* po = (float*)scratch;
    float* pml = po + (size_t)n_tok * n_heads * n_splits * head_dim;
#define CALL(D_) launch_decode<D_>(q, q_stride, k_cache, v_cache, block_table, max_blocks, tok_entry, positions, tok_first, n_tok, n_heads, n_kv, page_size, window, sl2, chunk, n_splits, po, pml, stream)
    int rc = 1;
    switch (head_dim) {
        case 16: rc = CALL(16); break;
        case 32: rc = CALL(32); break;
        case 48: rc = CALL(48); break;
        case 64: rc = CALL(64); break;
        case 80: rc = CALL(80); break;
        case 96: rc = CALL(96); break;
        case 112: rc = CALL(112); break;
        case 128: rc = CALL(128); break;
        default: infero_set_error("attn_decode: head_dim %d has no instance", head_dim);
    }
#undef CALL
    if (rc) return rc;
    const int warps = n_tok * n_heads;
    const int blocks = (warps + 3) / 4;
    attn_combine_kernel<<<blocks, 128, 0, stream>>>(po, pml, (bf16*)out, out_stride, tok_first, n_tok, n_heads,
                                                    n_splits, head_dim);
    return infero_check_launch("attn_combine");
}

}  // extern "C"
