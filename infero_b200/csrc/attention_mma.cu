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
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int KEYS16 = 16;

__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// A tile row holds D bf16 = D/8 chunks of 16 bytes, followed by one chunk of padding.  The
// row stride is then an odd number of chunks (D is a multiple of 16), so the eight rows an
// ldmatrix reads at one column fall into eight different 16-byte bank groups.
template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
    return row * (D / 8 + 1) + chunk;
}
template <int D>
constexpr int tile_elems(int rows) { return rows * (D + 8); }

// Gather rows [r0, r0 + n) (absolute key positions pos0 + r) of one kv head from the paged
// cache into a tile.  Rows whose page is not held (or that lie beyond `limit`) become zeros.
// All `nthreads` threads of the group take part; tid is the index inside the group.
template <int D>
__device__ __forceinline__ void gather_rows(bf16* tile, const bf16* __restrict__ cache, const int* __restrict__ table,
                                            int key0, int n_rows, int limit, int n_kv, int kvh, int page_size,
                                            int tid, int nthreads) {
    constexpr int CH = D / 8;
    for (int i = tid; i < n_rows * CH; i += nthreads) {
        const int r = i / CH, c = i - r * CH;
        const int j = key0 + r;
        bf16* dst = tile + (size_t)swz<D>(r, c) * 8;
        int page = -1;
        if (j < limit) page = table[j / page_size];
        if (page >= 0) {
            const bf16* src = cache + ((((size_t)page * n_kv + kvh) * page_size + (j % page_size)) * D + c * 8);
            cp_async16(smem_addr(dst), src);
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
}

// Q fragments of a warp's 16 rows straight from global memory (once per CTA).
// Row r lives at base + r * row_stride; rows >= valid_rows read as zero.
template <int D>
__device__ __forceinline__ void load_q(uint32_t (*qf)[4], const bf16* base, size_t row_stride, int valid_rows, int lane) {
    const int g = lane >> 2, c = lane & 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int d0 = ks * 16 + c * 2;
        const bf16* r0 = base + (size_t)g * row_stride;
        const bf16* r1 = base + (size_t)(g + 8) * row_stride;
        qf[ks][0] = g < valid_rows ? *reinterpret_cast<const uint32_t*>(r0 + d0) : 0u;
        qf[ks][1] = g + 8 < valid_rows ? *reinterpret_cast<const uint32_t*>(r1 + d0) : 0u;
        qf[ks][2] = g < valid_rows ? *reinterpret_cast<const uint32_t*>(r0 + d0 + 8) : 0u;
        qf[ks][3] = g + 8 < valid_rows ? *reinterpret_cast<const uint32_t*>(r1 + d0 + 8) : 0u;
    }
}

// One 16-key slice: s = q k^T (scaled to base-2 logits), mask, running max / sum update,
// o += p v.  k_tile/v_tile hold the slice at rows [row0, row0 + 16).
//   key_base: absolute position of row row0;  lo/hi0/hi1: visible keys are lo0 <= j <= hi for
//   the thread's two rows (g and g + 8).
template <int D>
__device__ __forceinline__ void slice16(const uint32_t (*qf)[4], const bf16* k_tile, const bf16* v_tile, int row0,
                                        int key_base, int lo0, int hi0, int lo1, int hi1, float scale_log2,
                                        float* m, float* l, float (*o)[4], int lane) {
    const int g = lane >> 2, c = lane & 3;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    // ---- s = q k^T: two n-tiles of 8 keys, D/16 k-steps; one ldmatrix.x4 per k-step ----------
    {
        const int mi = lane >> 3;                     // matrix this lane addresses
        const int krow = row0 + (mi >> 1) * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t b[4];
            ldmatrix_x4(b, smem_addr(k_tile + (size_t)swz<D>(krow, ks * 2 + (mi & 1)) * 8));
            mma16816(s[0], qf[ks], b[0], b[1]);
            mma16816(s[1], qf[ks], b[2], b[3]);
        }
    }
    // ---- mask and statistics --------------------------------------------------------------------
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = key_base + nt * 8 + c * 2 + e;
            float a = s[nt][e] * scale_log2, b = s[nt][2 + e] * scale_log2;
            a = (j >= lo0 && j <= hi0) ? a : -CUDART_INF_F;
            b = (j >= lo1 && j <= hi1) ? b : -CUDART_INF_F;
            s[nt][e] = a;
            s[nt][2 + e] = b;
            mx0 = fmaxf(mx0, a);
            mx1 = fmaxf(mx1, b);
        }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    // a row that has seen no key yet keeps m = -inf; subtracting 0 instead avoids inf - inf
    const float sub0 = mn0 == -CUDART_INF_F ? 0.f : mn0, sub1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
    const float corr0 = exp2f(m[0] - sub0), corr1 = exp2f(m[1] - sub1);
    m[0] = mn0;
    m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pf[4];
    {
        float p[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            p[nt][0] = exp2f(s[nt][0] - sub0);
            p[nt][1] = exp2f(s[nt][1] - sub0);
            p[nt][2] = exp2f(s[nt][2] - sub1);
            p[nt][3] = exp2f(s[nt][3] - sub1);
            sum0 += p[nt][0] + p[nt][1];
            sum1 += p[nt][2] + p[nt][3];
        }
        pf[0] = pack_bf16(p[0][0], p[0][1]);
        pf[1] = pack_bf16(p[0][2], p[0][3]);
        pf[2] = pack_bf16(p[1][0], p[1][1]);
        pf[3] = pack_bf16(p[1][2], p[1][3]);
    }
    l[0] = l[0] * corr0 + sum0;        // per-thread partial sums; lanes are added up at the end
    l[1] = l[1] * corr1 + sum1;
    // ---- o = o * corr + p v: D/8 n-tiles, one k-step of 16 keys ------------------------------
    {
        const int mi = lane >> 3;
        const int vrow = row0 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, smem_addr(v_tile + (size_t)swz<D>(vrow, np * 2 + (mi >> 1)) * 8));
            float* o0 = o[np * 2];
            float* o1 = o[np * 2 + 1];
            o0[0] *= corr0; o0[1] *= corr0; o0[2] *= corr1; o0[3] *= corr1;
            o1[0] *= corr0; o1[1] *= corr0; o1[2] *= corr1; o1[3] *= corr1;
            mma16816(o0, pf, b[0], b[1]);
            mma16816(o1, pf, b[2], b[3]);
        }
    }
}

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
    kern<<<grid, PF_THREADS, smem, stream>>>((const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_cache,
                                             (const bf16*)v_cache, block_table, max_blocks, entry_q_start, entry_q_len,
                                             entry_pos0, n_entries, first_entry, n_heads, n_kv, page_size, window,
                                             scale_log2);
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
