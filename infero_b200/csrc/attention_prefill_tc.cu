// Prompt-portion attention over the paged cache on the 5th-generation tensor cores.
//
// One CTA = 128 consecutive query tokens of one request and TWO heads that share a kv head (the
// last head of an odd group works alone; when a grid of pairs would not fill the SMs, every head
// does).  Both heads see the same keys, so every key and value
// tile is fetched from L2 once for 256 query rows: with one head per CTA the kernel was bound by
// L2 bandwidth (128 flops per byte fetched; measured 665 TFLOP/s with the softmax taken out).
// The CTA walks the visible keys in tiles of 64; per head:
//   S = Q K^T     tcgen05.mma, both operands in shared memory (TMA, 128-byte swizzle), S in TMEM
//   P = 2^(S*c - m), reference point m and sum l per row; one thread owns one query row (it
//                 reads its row of S from TMEM with tcgen05.ld into registers, once), writes P
//                 back over S as bf16 and, when its reference point moved, rescales its row of O
//   O += P V      tcgen05.mma with P from TMEM and V from shared memory (N-contiguous operand)
// Warp roles: 0..3 softmax and epilogue of the first head (128 rows), 4..7 of the second, 8 loads
// the two Q blocks once and then the key tiles, 9 the value tiles (each into its own ring, page by
// page from the block table, four lanes side by side), 10 owns TMEM and issues the MMAs of both heads.  Each
// head has two S buffers and one O (256 TMEM columns), so Q K^T of the next tile runs while the
// softmax of this one does, and one head's softmax runs under the other's products.  Scores,
// maxima, sums and O are 32-bit; P is rounded to bf16 for the second product, as the keys and
// values are.
//
// Same formula as attention_generic.cu: key j is visible from the query at position p iff
// lo <= j <= p with lo = max(0, p - window + 1).  The reference's prefill attention is
// attn_prefill_mma_ws4 (crates/kernels/src/lib.rs:3717) on mma.sync; its formula is
// crates/kernels/src/cu/ops.cu:709-811.
//
// Head sizes 64 and 128; page sizes that are multiples of 16.  Every wait is bounded; a wait
// that runs out raises the error flag and the CTA leaves in order (TMEM freed).
#include "tc_common.cuh"
#include <math_constants.h>

namespace {

using namespace tc;

constexpr int QROWS = 128, KTILE = 64;
constexpr int PFT_K_WARP = 8, PFT_V_WARP = 9, PFT_MMA_WARP = 10, PFT_THREADS = 352;      // warps 0..7: softmax
constexpr float RESCALE_STEP = 8.0f;

template <int D>
struct PfPlan {
    static constexpr int DB = D / 64;                        // 64-element blocks along the head
    static constexpr int STAGES = D == 128 ? 4 : 8;          // key tiles (and value tiles) in flight
    static constexpr int QBLOCK_BYTES = QROWS * 128;         // the query rows of one block
    static constexpr int KBLOCK_BYTES = KTILE * 128;         // the key (or value) rows of one block
    static constexpr int Q_BYTES = DB * QBLOCK_BYTES;        // one head's queries
    static constexpr int KV_BYTES = DB * KBLOCK_BYTES;       // one K tile, or one V tile
    static constexpr int Q_OFF = 0;                          // two heads
    static constexpr int K_OFF = 2 * Q_BYTES;
    static constexpr int V_OFF = K_OFF + STAGES * KV_BYTES;
    static constexpr int BAR_OFFSET = V_OFF + STAGES * KV_BYTES;
    static constexpr int N_BARS = 1 + 4 * STAGES + 2 * 5;
    static constexpr int TOTAL = BAR_OFFSET + 8 * N_BARS + 64 + 1024;
    // per head: two S buffers of KTILE columns, then O; 256 columns per head, the SM's 512 for the CTA
    static constexpr uint32_t HEAD_COLS = 256, S_COL = 0, O_COL = 2 * KTILE;
    static constexpr uint32_t TMEM_COLS = 512;
    static_assert(2 * KTILE + D <= 256, "S, S and O must fit 256 TMEM columns");
    static_assert(TOTAL > 116 * 1024, "one CTA per SM: it takes all of the SM's tensor memory");
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// max of three in one instruction, and a multiply-add on a pair of 32-bit floats in one instruction
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void fma2(float& x0, float& x1, float a0, float a1, float b, float c) {
    asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %4};\n mov.b64 rc, {%5, %5};\n"
        " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(x0), "=f"(x1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(PFT_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int out_stride,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ entry_q_start,
                       const int* __restrict__ entry_q_len, const int* __restrict__ entry_pos0, int n_entries,
                       int first_entry, int n_tiles, int n_heads, int n_kv, int heads_per_cta, int page_size, int slice,
                       int window, float scale_log2, int* __restrict__ err_flag) {
    using Plan = PfPlan<D>;
    constexpr int DB = Plan::DB, ST = Plan::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFFSET);
    uint64_t* q_full = bars;                 // 1
    uint64_t* k_full = bars + 1;             // ST
    uint64_t* v_full = k_full + ST;          // ST
    uint64_t* k_empty = v_full + ST;         // ST
    uint64_t* v_empty = k_empty + ST;        // ST
    uint64_t* s_full = v_empty + ST;         // [head][2]
    uint64_t* p_full = s_full + 4;           // [head][2] (128 arrivals)
    uint64_t* o_done = p_full + 4;           // [head]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* never_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        mbar_init(q_full, 1);
        for (int i = 0; i < ST; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
        }
        mbar_init(&o_done[0], 1);
        mbar_init(&o_done[1], 1);
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == PFT_MMA_WARP) {
        tmem_alloc(tmem_slot, Plan::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                        // q, the tables and this step's keys come from earlier kernels

    // ---- which kv head and pair of heads, which request and which block of 128 query rows? ------
    const int group = n_heads / n_kv;
    const int pairs = (group + heads_per_cta - 1) / heads_per_cta;
    const int kvh = (int)blockIdx.x / pairs;
    const int head0 = kvh * group + heads_per_cta * ((int)blockIdx.x % pairs);
    const int n_q = min(heads_per_cta, (kvh + 1) * group - head0);      // heads of this CTA
    int e = -1, tile_in_e = 0;
    {
        int left = n_tiles - 1 - (int)blockIdx.y;                           // longest first
        for (int i = first_entry; i < n_entries; ++i) {
            const int nt = (entry_q_len[i] + QROWS - 1) / QROWS;
            if (left < nt) { e = i; tile_in_e = left; break; }
            left -= nt;
        }
    }
    int n_kt = 0, kt_begin = 0, q_len = 0, pos0 = 0, tok0 = 0, row_first = 0, rows_here = 0;
    if (e >= 0) {
        q_len = entry_q_len[e]; pos0 = entry_pos0[e]; tok0 = entry_q_start[e];
        row_first = tile_in_e * QROWS;
        rows_here = min(QROWS, q_len - row_first);
        const int first_pos = pos0 + row_first, last_pos = first_pos + rows_here - 1;
        const int key_lo = window > 0 ? max(0, first_pos - window + 1) : 0;
        kt_begin = key_lo / KTILE;
        n_kt = last_pos / KTILE - kt_begin + 1;
    }
    const int* table = block_table + (size_t)(e < 0 ? 0 : e) * max_blocks;
    const int first_pos = pos0 + row_first;

    if (warp == PFT_K_WARP || warp == PFT_V_WARP) {
        // ---- loaders: one warp for the keys (and Q), one for the values ------------------------------
        // A tile is fetched in slices of `slice` rows (64, 32 or 16: what lies in one page), one TMA box per
        // slice and 64-element block.  Lane s fetches slice s of every tile, so the look-ups in the block
        // table and the TMA instructions of a tile run side by side instead of one after the other in
        // a single thread.  Boxes of 16 rows (2 KB) are slow: about one per 130 cycles per SM.
        const bool is_k = warp == PFT_K_WARP;
        if (n_kt > 0 && lane < KTILE / slice) {
            const CUtensorMap* map = is_k ? &map_k : &map_v;
            uint64_t* full = is_k ? k_full : v_full;
            uint64_t* empty = is_k ? k_empty : v_empty;
            uint8_t* ring = smem + (is_k ? Plan::K_OFF : Plan::V_OFF);
            if (is_k && lane == 0) {
                mbar_expect_tx(q_full, n_q * Plan::Q_BYTES);
                for (int t = 0; t < n_q; ++t)
#pragma unroll
                    for (int b = 0; b < DB; ++b)
                        tma_load_2d(smem + Plan::Q_OFF + t * Plan::Q_BYTES + b * Plan::QBLOCK_BYTES, &map_q,
                                    (head0 + t) * D + b * 64, tok0 + row_first, q_full);
            }
            // pages of up to 64 rows are fetched whole (slice == page_size): no division in the loop
            const bool whole_pages = slice == page_size;
            const int per_tile = KTILE / slice;
            auto row_of = [&](int j) {
                int blk, in_page;
                if (whole_pages) {
                    blk = (kt_begin + j) * per_tile + lane;
                    in_page = 0;
                } else {
                    const int key0 = (kt_begin + j) * KTILE + lane * slice;
                    blk = key0 / page_size;
                    in_page = key0 - blk * page_size;
                }
                const int page = blk < max_blocks ? table[blk] : -1;
                // a page that is not held (beyond the request's end) is never visible; any finite rows do
                return (page < 0 ? 0 : (page * n_kv + kvh) * page_size) + in_page;
            };
            bool ok = true;
            int issued = 0;
            int row = row_of(0);
            for (int i = 0; i < n_kt; ++i) {
                const int s = i % ST;
                const int next_row = i + 1 < n_kt ? row_of(i + 1) : 0;      // looked up while waiting
                if (!mbar_wait(&empty[s], ((uint32_t)(i / ST) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                if (lane == 0) mbar_expect_tx(&full[s], Plan::KV_BYTES);
                uint8_t* dst = ring + s * Plan::KV_BYTES + lane * (slice * 128);
#pragma unroll
                for (int b = 0; b < DB; ++b) tma_load_2d(dst + b * Plan::KBLOCK_BYTES, map, b * 64, row, &full[s]);
                issued = i + 1;
                row = next_row;
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 5);
            }
            if (*abort_flag) {
                // let copies that are still in flight land before the block goes away
                if (is_k && lane == 0) mbar_wait(q_full, 0, never_flag);
                for (int i = max(0, issued - ST); i < issued; ++i) mbar_wait(&full[i % ST], (uint32_t)(i / ST) & 1u, never_flag);
            }
        }
    } else if (warp == PFT_MMA_WARP) {
        // ---- MMA issue, both heads ------------------------------------------------------------------
        if (n_kt > 0 && elect_one()) {
            constexpr uint32_t idesc_qk = idesc_bf16_f32(QROWS, KTILE);
            constexpr uint32_t idesc_pv = idesc_bf16_f32_b_mn(QROWS, D);
            bool ok = true;
            // S = Q K^T of key tile j for every head of the CTA; the key stage is free after the last
            auto issue_qk = [&](int j) {
                const uint32_t k_addr = smem_u32(smem + Plan::K_OFF + (j % ST) * Plan::KV_BYTES);
                for (int t = 0; t < n_q; ++t) {
                    const uint32_t q_addr = smem_u32(smem + Plan::Q_OFF + t * Plan::Q_BYTES);
                    const uint32_t s_tmem = tmem_base + (uint32_t)t * Plan::HEAD_COLS + Plan::S_COL + (uint32_t)(j & 1) * KTILE;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        const uint32_t in_block = (uint32_t)(ks & 3) * 32u;
                        umma_bf16(s_tmem, smem_desc_k_sw128(q_addr + (uint32_t)(ks >> 2) * Plan::QBLOCK_BYTES + in_block),
                                  smem_desc_k_sw128(k_addr + (uint32_t)(ks >> 2) * Plan::KBLOCK_BYTES + in_block), idesc_qk,
                                  ks > 0 ? 1u : 0u);
                    }
                    umma_commit(&s_full[t * 2 + (j & 1)]);
                }
                umma_commit(&k_empty[j % ST]);
            };
            if (!mbar_wait(q_full, 0, abort_flag) || !mbar_wait(&k_full[0], 0, abort_flag)) ok = false;
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0);
            }
            for (int j = 0; j < n_kt && ok; ++j) {
                if (j + 1 < n_kt) {
                    if (!mbar_wait(&k_full[(j + 1) % ST], (uint32_t)((j + 1) / ST) & 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    issue_qk(j + 1);
                }
                if (!mbar_wait(&v_full[j % ST], (uint32_t)(j / ST) & 1u, abort_flag)) { ok = false; break; }
                const uint32_t v_addr = smem_u32(smem + Plan::V_OFF + (j % ST) * Plan::KV_BYTES);
                for (int t = 0; t < n_q && ok; ++t) {
                    if (!mbar_wait(&p_full[t * 2 + (j & 1)], (uint32_t)(j >> 1) & 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t head_tmem = tmem_base + (uint32_t)t * Plan::HEAD_COLS;
                    const uint32_t p_tmem = head_tmem + Plan::S_COL + (uint32_t)(j & 1) * KTILE;
#pragma unroll
                    for (int ks = 0; ks < KTILE / 16; ++ks) {
                        // 16 keys: 8 columns of P (two bf16 each), 16 rows of V (2048 bytes)
                        const uint64_t vd = smem_desc_mn_sw128(v_addr + (uint32_t)ks * 2048u, Plan::KBLOCK_BYTES, 1024u);
                        umma_bf16_ts(head_tmem + Plan::O_COL, p_tmem + (uint32_t)ks * 8u, vd, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(&o_done[t]);
                }
                if (ok) umma_commit(&v_empty[j % ST]);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 6);
            }
        }
    } else if (n_kt > 0 && (warp >> 2) < n_q) {
        // ---- softmax, correction of O, epilogue: one query row of one head per thread -----------------
        const int t = warp >> 2;                             // which head of the CTA
        const int h = head0 + t;
        const int r = (warp & 3) * 32 + lane;
        const bool valid = r < rows_here;
        const int pos_r = first_pos + r;
        const int hi_r = valid ? pos_r : -1;
        const int lo_r = window > 0 ? max(0, pos_r - window + 1) : 0;
        const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t head_tmem = tmem_base + (uint32_t)t * Plan::HEAD_COLS + lane_sel;
        uint64_t* my_s_full = s_full + t * 2;
        uint64_t* my_p_full = p_full + t * 2;
        uint64_t* my_o_done = o_done + t;
        float m = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kt; ++j) {
            const int b = j & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&my_s_full[b], (uint32_t)(j >> 1) & 1u, abort_flag))) { ok = false; break; }   // warp-uniform
            tc_fence_after_sync();
            const uint32_t s_addr = head_tmem + Plan::S_COL + (uint32_t)b * KTILE;
            const int kb = (kt_begin + j) * KTILE;
            // every key of the tile visible from every row of the block?  (rows past the portion's
            // end then compute on, unmasked; nothing of theirs is stored)
            const bool open_tile = (kb + KTILE - 1 <= first_pos) &&
                                   (window <= 0 || kb >= first_pos + rows_here - 1 - window + 1);
            // the row's KTILE scores, once: all loads in flight, then one wait
            uint32_t sv[KTILE];
#pragma unroll
            for (int c = 0; c < KTILE / 32; ++c) tmem_ld32_nowait(s_addr + (uint32_t)c * 32u, sv + c * 32);
            tmem_wait_ld();
            // four running maxima (and sums below): a chain of 16 dependent operations instead of 64
            float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (open_tile) {
#pragma unroll
                for (int i = 0; i < KTILE; i += 2)
                    mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
            } else {
#pragma unroll
                for (int i = 0; i < KTILE; ++i) {
                    const int key = kb + i;
                    if (!(key >= lo_r && key <= hi_r)) sv[i] = 0xff800000u;      // -inf: contributes 2^-inf = 0
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // The reference point m of the exponentials follows the row's maximum lazily: it moves only
            // when the maximum has grown by more than RESCALE_STEP (in powers of two) since it was set,
            // so that O is seldom rescaled; meanwhile P stays below 2^RESCALE_STEP, which bf16 holds with
            // the same relative precision, and l and O refer to the same m, so the quotient is unchanged.
            const float m_seen = fmaxf(m, mx * scale_log2);
            const float m_new = (m_seen - m > RESCALE_STEP) ? m_seen : m;       // m = -inf: inf > step, moves
            const float sub = m_new == -CUDART_INF_F ? 0.f : m_new;     // a row with no key yet: avoid inf - inf
            const float corr = ex2(m - sub);
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[KTILE / 2];
#pragma unroll
            for (int i = 0; i < KTILE; i += 2) {
                float x0, x1;
                fma2(x0, x1, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]), scale_log2, -sub);
                const float p0 = ex2(x0), p1 = ex2(x1);
                sum4[(i >> 1) & 3] += p0 + p1;
                pk[i >> 1] = pack2(p0, p1);
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // P over S (every score is in registers by now)
#pragma unroll
            for (int c = 0; c < KTILE / 32; ++c) tmem_st16(s_addr + (uint32_t)c * 16u, pk + c * 16);
            l = l * corr + sum;
            m = m_new;
            if (j > 0) {
                // The product before this one.  It is waited for at every tile, needed or not (by now it
                // has nearly always finished): a parity wait can only tell the running phase from the one
                // before it, so the waiter must never fall two phases behind the barrier.
                if (!__all_sync(0xffffffffu, mbar_wait(my_o_done, (uint32_t)(j - 1) & 1u, abort_flag))) { ok = false; break; }
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
                    // a row's reference point moved: its O so far is scaled down
                    tc_fence_after_sync();
                    const uint32_t o_addr = head_tmem + Plan::O_COL;
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32_nowait(o_addr + (uint32_t)c * 32u, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                        tmem_st32(o_addr + (uint32_t)c * 32u, v);
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&my_p_full[b]);
        }
        // the last product (the one before it was waited for inside the loop)
        if (ok && !__all_sync(0xffffffffu, mbar_wait(my_o_done, (uint32_t)(n_kt - 1) & 1u, abort_flag))) ok = false;
        tc_fence_after_sync();
        if (ok) {
            // every lane takes part in the TMEM loads (they are warp-wide); only lanes that own a
            // row of the portion store
            const float inv = 1.0f / l;
            const uint32_t o_addr = head_tmem + Plan::O_COL;
            bf16* orow = out + (size_t)(tok0 + row_first + (valid ? r : 0)) * out_stride + (size_t)h * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld32_nowait(o_addr + (uint32_t)c * 32u, v);
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                        w.y = pack2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                        w.z = pack2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                        w.w = pack2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
                    }
                }
                __syncwarp();
            }
        } else if (lane == 0) {
            *abort_flag = 1;
            atomicExch(err_flag, 7);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == PFT_MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Plan::TMEM_COLS);
    }
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, int out_stride,
           const int* block_table, int max_blocks, const int* entry_q_start, const int* entry_q_len,
           const int* entry_pos0, int n_entries, int first_entry, int n_tiles, int n_heads, int n_kv, int page_size,
           int slice, int window, float scale_log2, int* err, cudaStream_t stream) {
    using Plan = PfPlan<D>;
    // Two heads per CTA halve the key and value traffic, but a grid that does not fill the SMs that way
    // runs faster with one head per CTA: measured at 7B sizes 25 against 35 us at 1,024 tokens (128
    // CTAs in pairs) and 45 against 37 us at 1,536 (192 CTAs in pairs); the same at 0.5B sizes.
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int group = n_heads / n_kv;
    const int hpc = (long long)n_kv * ((group + 1) / 2) * n_tiles <= sms ? 1 : 2;
    auto kern = attn_prefill_tc_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::TOTAL);
        if (e != cudaSuccess) {
            infero_set_error("attn_prefill_tc: cannot get %d bytes of shared memory: %s", Plan::TOTAL, cudaGetErrorString(e));
            return 1;
        }
        configured = true;
    }
    launch_pdl(kern, dim3(n_kv * ((group + hpc - 1) / hpc), n_tiles), dim3(PFT_THREADS), Plan::TOTAL, stream, mq, mk, mv, (bf16*)out, out_stride,
               block_table, max_blocks, entry_q_start, entry_q_len, entry_pos0, n_entries, first_entry, n_tiles, n_heads,
               n_kv, hpc, page_size, slice, window, scale_log2, err);
    return infero_check_launch("attn_prefill_tc");
}

}  // namespace

extern "C" {

int infero_attn_prefill_tc_supported(int head_dim, int page_size, int q_stride, int out_stride) {
    return (head_dim == 64 || head_dim == 128) && page_size % 16 == 0 && q_stride % 8 == 0 && out_stride % 8 == 0;
}

// The same contract as infero_attn_prefill (attention_mma.cu) with 128 query rows per block:
// n_tiles = sum over the requests first_entry .. n_entries - 1 of ceil(q_len / 128).  q is
// [n_tokens, >= n_heads * head_dim] bf16 with row stride q_stride; the caches are
// [num_pages, n_kv, page_size, head_dim] bf16, contiguous; all 16-byte aligned.
int infero_attn_prefill_tc(const void* q, int q_stride, int n_tokens, void* out, int out_stride, const void* k_cache,
                           const void* v_cache, int num_pages, const int* block_table, int max_blocks,
                           const int* entry_q_start, const int* entry_q_len, const int* entry_pos0, int n_entries,
                           int first_entry, int n_tiles, int n_heads, int n_kv, int head_dim, int page_size,
                           int window, float scale, cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    INFERO_REQUIRE(infero_attn_prefill_tc_supported(head_dim, page_size, q_stride, out_stride),
                   "attn_prefill_tc: head_dim %d / page_size %d / strides %d, %d not supported", head_dim, page_size,
                   q_stride, out_stride);
    INFERO_REQUIRE(n_kv > 0 && n_heads % n_kv == 0 && n_tiles <= 65535, "attn_prefill_tc: bad sizes heads %d / %d, %d tiles",
                   n_heads, n_kv, n_tiles);
    INFERO_REQUIRE((long long)num_pages * n_kv * page_size < (1ll << 31), "attn_prefill_tc: cache of %d pages too large", num_pages);
    INFERO_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0,
                   "attn_prefill_tc: q and out must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    const int rows = num_pages * n_kv * page_size;
    if (infero_tensor_map_bf16(q, n_tokens, n_heads * head_dim, q_stride, QROWS, &mq)) return 1;
    // one TMA box = the rows of a tile that lie in one page: 64, 32 or 16 of them
    const int slice = page_size % 64 == 0 ? 64 : page_size % 32 == 0 ? 32 : 16;
    if (infero_tensor_map_bf16(k_cache, rows, head_dim, head_dim, slice, &mk)) return 1;
    if (infero_tensor_map_bf16(v_cache, rows, head_dim, head_dim, slice, &mv)) return 1;
    int* err;
    if (infero_tc_err_flag(&err)) return 1;
    const float sl2 = scale * 1.4426950408889634f;
    if (head_dim == 128)
        return launch<128>(mq, mk, mv, out, out_stride, block_table, max_blocks, entry_q_start, entry_q_len, entry_pos0,
                           n_entries, first_entry, n_tiles, n_heads, n_kv, page_size, slice, window, sl2, err, stream);
    return launch<64>(mq, mk, mv, out, out_stride, block_table, max_blocks, entry_q_start, entry_q_len, entry_pos0,
                      n_entries, first_entry, n_tiles, n_heads, n_kv, page_size, slice, window, sl2, err, stream);
}

}  // extern "C"
