// One layer of the built-in kind (pre-norm block: RMSNorm, grouped-query attention with rotary
// positions over the paged cache, RMSNorm, SwiGLU) launched from native code.  In steps with a prompt
// portion: the same kernels with the same arguments, in the same order, as the Python parts launch
// them one by one, so the results are the same bit for bit and only the host's time per layer
// differs (one call instead of a dozen Python wrappers).  In steps of single tokens, where a launch
// costs more than its work, the layer is five launches instead of eight: decode attention finishes
// the q/k/v product itself, and the two norms are folded into the products around them (see
// infero_block_forward).  bf16 steps on the tensor-core path only; everything else stays with the parts.
//
// The reference runs its whole layer loop natively (crates/model/src/lib.rs:3423-4243); this is
// the corresponding piece for the one layout of block this engine builds itself.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>

extern "C" {
// elementwise.cu, rope_cache.cu, gemm_tc.cu, attention_*.cu, runtime.cu
int infero_embed_gather(const void* table, int table_dtype, const int* ids, const int* device_tokens, float* x,
                        int n_tokens, int d, int vocab, float scale, cudaStream_t stream);
int infero_add_rmsnorm(float* x, const void* delta, int delta_dtype, int delta_splits, long long split_stride,
                       const void* dbias, int dbias_dtype, const void* w, int w_dtype, float eps, void* out,
                       int out_dtype, const int* rows, int n_rows, int d, cudaStream_t stream);
int infero_swiglu(const void* gate_up, int splits, long long split_stride, void* out, int dtype, int out_bf16,
                  int n_tokens, int ff, cudaStream_t stream);
int infero_rope_cache(void* qkv, int dtype, int row_stride, const int* positions, const int* tok_entry,
                      const int* block_table, int max_blocks, const float* inv_freq, int rotary_dim, void* k_cache,
                      void* v_cache, int page_size, int n_tokens, int n_heads, int n_kv, int head_dim,
                      int write_cache, cudaStream_t stream);
int infero_rope_cache_partials(const float* partial, int splits, long long split_stride, const void* bias,
                               int bias_dtype, void* q_out, int q_stride, int dtype, const int* positions,
                               const int* tok_entry, const int* block_table, int max_blocks, const float* inv_freq,
                               int rotary_dim, void* k_cache, void* v_cache, int page_size, int n_tokens,
                               int n_heads, int n_kv, int head_dim, int write_cache, cudaStream_t stream);
int infero_gemm_tc_supported(const void* x, const void* w, int M, int N, int K, int ldx);
int infero_gemm_tc_plan(int M, int N, int K, int sm_count, int* splits, int* ktiles_per_split, long long* ws_bytes);
int infero_gemm_tc_partials(const void* x, const void* w, float* partial, int M, int N, int K, int ldx, int splits,
                            int ktiles_per_split, cudaStream_t stream);
int infero_gemm_tc_summed(const void* x, const void* w, float* out, int M, int N, int K, int ldx, int splits,
                          int ktiles_per_split, cudaStream_t stream);
int infero_gemm_cluster_enabled();
int infero_gemm_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype, int M,
                   int N, int K, int ldx, int ldc, void* workspace, long long workspace_bytes, int sm_count,
                   int tile_n, cudaStream_t stream);
int infero_gemm_tc_swiglu(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldc,
                          int sm_count, cudaStream_t stream);
long long infero_attn_decode_scratch(int n_tok, int n_heads, int head_dim, int n_splits);
int infero_sm_count();
void infero_attn_plan_decode(int n_tok, int n_kv, int group, int max_visible, int sm_count, int* chunk, int* splits);
int infero_attn_decode_tma_supported(int head_dim, int page_size);
int infero_attn_decode_tma(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                           const void* v_cache, int num_pages, const int* block_table, int max_blocks,
                           const int* tok_entry, const int* positions, int tok_first, int n_tok, int n_heads,
                           int n_kv, int head_dim, int page_size, int window, float scale, int chunk, int n_splits,
                           void* scratch, int* counters, int n_counters, cudaStream_t stream);
int infero_attn_decode_fused_supported(const float* partial, long long split_stride, int n_heads, int n_kv,
                                       int head_dim, int page_size, int rotary_dim, const void* k_cache,
                                       const void* v_cache);
int infero_attn_decode_tma_fused(const float* partial, int splits, long long split_stride, const void* bias,
                                 int bias_dtype, const float* inv_freq, int rotary_dim, int write_cache, void* out,
                                 int out_stride, void* k_cache, void* v_cache, int num_pages, const int* block_table,
                                 int max_blocks, const int* tok_entry, const int* positions, int tok_first, int n_tok,
                                 int n_heads, int n_kv, int head_dim, int page_size, int window, float scale, int chunk,
                                 int n_splits, void* scratch, int* counters, int n_counters, const float* sumsq,
                                 int sumsq_tiles, float inv_d, float eps, cudaStream_t stream);
int infero_gemm_tc_plan_cluster(int M, int N, int K, int sm_count, int* splits, int* ktiles_per_split);
int infero_gemm_tc_residual_norm(const void* x, const void* w, int M, int N, int K, int ldx, int splits,
                                 int ktiles_per_split, float* resid, const void* bias, int bias_dtype,
                                 const void* norm_w, int norm_w_dtype, void* h, float* sumsq, cudaStream_t stream);
int infero_gemm_tc_swiglu_scaled(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldc,
                                 const float* sumsq, int n_tiles, float inv_d, float eps, int sm_count,
                                 cudaStream_t stream);
int infero_attn_prefill_tc_supported(int head_dim, int page_size, int q_stride, int out_stride);
int infero_attn_prefill_tc(const void* q, int q_stride, int n_tokens, void* out, int out_stride, const void* k_cache,
                           const void* v_cache, int num_pages, const int* block_table, int max_blocks,
                           const int* entry_q_start, const int* entry_q_len, const int* entry_pos0, int n_entries,
                           int first_entry, int n_tiles, int n_heads, int n_kv, int head_dim, int page_size,
                           int window, float scale, cudaStream_t stream);
}
void infero_set_error(const char* fmt, ...);

extern "C" {

enum : int { F32 = 0, BF16 = 1, PRENORMED = 2 };

// What is fixed for one execution of a block (a schedule entry): sizes, weights, its cache.
struct InferoBlock {
    int hidden, n_heads, n_kv, head_dim, intermediate, rotary_dim, window, write_cache;
    float eps_mixer, eps_ffn, scale;
    int norm_dtype, qkv_bias_dtype, o_bias_dtype;
    const void* w_norm_mixer;
    const void* w_norm_ffn;
    const void* w_qkv;
    const void* b_qkv;          // or null
    const void* w_o;
    const void* b_o;            // or null
    const void* w_gate_up;      // rows alternate gate_j, up_j
    const void* w_down;
    const float* inv_freq;      // rotary_dim / 2 floats (rotary_dim 0: none)
    void* k_cache;
    void* v_cache;
    int num_pages, page_size;
};

// What is fixed for one step: the batch and where things live.  The same for every layer.
struct InferoStep {
    int n_tokens, n_entries, n_decode;          // single-token requests come first
    int decode_visible;                         // keys the decode kernel is planned for
    int prefill_tiles;                          // blocks of 128 query rows of the other requests
    int sm_count;
    const int* positions;
    const int* tok_entry;
    const int* entry_q_start;
    const int* entry_q_len;
    const int* entry_pos0;
    float* x;                                   // residual stream [n_tokens, hidden]
    uint8_t* arena;                             // scratch of infero_block_arena_bytes
    long long arena_bytes;
    int* counters;                              // zeroed ints for the decode kernel
    int n_counters;
    cudaStream_t stream;
};

// A layer's pending output: the next norm adds it to x.
struct InferoDelta {
    const void* data;           // null: nothing pending
    int dtype;                  // F32 (partial sums) or BF16 (a finished product)
    int splits;
    long long split_stride;
    const void* bias;           // added with the sum (partial sums only), or null
    int bias_dtype;
    // PRENORMED: nothing is pending any more.  x already holds the sum, data is bf16(x * w) with w the
    // weight of the next layer's first norm, and sumsq holds, per 128-feature tile and token (256 floats
    // per tile), the sums of x^2 from which that norm's scalar follows.
    const float* sumsq;
    int sumsq_tiles;
};

static long long align_up(long long v) { return (v + 255) / 256 * 256; }

struct ArenaPlan {
    long long sumsq[2], delta[2], h, qkv, q, attn, scratch, o_delta, act, gate_up, total;
};

// Room for the product of T rows with a [N, K] matrix, which comes as partial sums (few rows) or finished
// (bf16, or 32-bit when it is an update of the residual stream).
static long long product_bytes(int T, int N, int K, int sm_count, bool residual = false) {
    if (T > 256) return align_up((long long)T * N * (residual ? 4 : 2));
    int splits = 1, per = 1;
    long long ws = 0;
    infero_gemm_tc_plan(T, N, K, sm_count, &splits, &per, &ws);
    return align_up((long long)std::max(1, splits) * T * N * 4);
}

static ArenaPlan plan_arena(const InferoBlock& b, int T, int sm_count) {
    ArenaPlan p;
    const int da = b.n_heads * b.head_dim, nqkv = (b.n_heads + 2 * b.n_kv) * b.head_dim;
    long long off = 0;
    auto take = [&](long long bytes) { long long at = off; off += align_up(bytes); return at; };
    // The two output areas lie at places that depend on the step and the residual width only, not on the
    // block (up to 16 splits of up to 256 rows, or a finished product): the layer that reads one as its
    // input may be built to other sizes and must not have its own areas overlap it.
    const long long delta_bytes = std::max(16LL * std::min(T, 256) * b.hidden * 4, (long long)T * b.hidden * 4);
    // sums of squares of the residual stream, per 128-feature tile and token: [0] inside a layer (for its
    // second norm), [1] between layers (for the next layer's first)
    p.sumsq[0] = take((long long)((b.hidden + 127) / 128) * 256 * 4);
    p.sumsq[1] = take((long long)((b.hidden + 127) / 128) * 256 * 4);
    p.delta[0] = take(delta_bytes);
    p.delta[1] = take(delta_bytes);
    p.h = take((long long)T * b.hidden * 2);
    p.qkv = take(product_bytes(T, nqkv, b.hidden, sm_count));
    p.q = take((long long)T * da * 2);
    p.attn = take((long long)T * da * 2);
    // the decode kernel's splits: tokens x splits stays below about two CTAs per SM (or one split each)
    p.scratch = take(infero_attn_decode_scratch(std::max(T, 2 * (sm_count > 0 ? sm_count : infero_sm_count())), b.n_heads,
                                                b.head_dim, 1));
    p.o_delta = take(product_bytes(T, b.hidden, da, sm_count, true));
    p.act = take((long long)T * b.intermediate * 2);
    p.gate_up = take(T <= 256 ? product_bytes(T, 2 * b.intermediate, b.hidden, sm_count) : 0);
    p.total = off;
    return p;
}

// The most any step of up to max_tokens tokens needs (the need does not grow evenly with the tokens:
// few rows come as partial sums).
long long infero_block_arena_bytes(const InferoBlock* b, int max_tokens, int sm_count) {
    long long most = 0;
    const int probes[] = {1, 16, 32, 64, 128, 256, 257, max_tokens};
    for (int t : probes)
        if (t <= max_tokens || t == 1) most = std::max(most, plan_arena(*b, std::min(t, std::max(1, max_tokens)), sm_count).total);
    return most;
}

// Can this block run here at all?  (Shapes the tensor-core kernels take, head sizes the TMA-fed
// attention kernels take.)
int infero_block_supported(const InferoBlock* b) {
    const int da = b->n_heads * b->head_dim;
    auto ok_k = [](int K) { return K >= 8 && K % 8 == 0; };
    return (b->head_dim == 64 || b->head_dim == 128) && b->page_size % 16 == 0 && b->n_kv > 0 &&
           b->n_heads % b->n_kv == 0 && ok_k(b->hidden) && ok_k(da) && ok_k(b->intermediate) &&
           b->rotary_dim % 2 == 0 && b->rotary_dim <= b->head_dim;
}

// out = a[T, K] * w[N, K]^T for the caller's next kernel: partial sums for few rows, a finished
// product (bias added) for many: bf16, or 32-bit when it updates the residual stream (a token's residual
// then receives 32-bit sums however many rows its step has).
static int product(const InferoStep& s, const void* a, int K, const void* w, int N, const void* bias, int bias_dtype,
                   void* dst, InferoDelta* out, bool residual = false) {
    const int T = s.n_tokens;
    if (T <= 256) {
        int splits = 1, per = 1;
        long long ws = 0;
        infero_gemm_tc_plan(T, N, K, s.sm_count, &splits, &per, &ws);
        int rc;
        if (splits >= 2 && splits <= 8 && infero_gemm_cluster_enabled()) {
            rc = infero_gemm_tc_summed(a, w, (float*)dst, T, N, K, K, splits, per, s.stream);
            splits = 1;
        } else {
            rc = infero_gemm_tc_partials(a, w, (float*)dst, T, N, K, K, splits, per, s.stream);
        }
        if (rc) return rc;
        *out = InferoDelta{dst, F32, splits, (long long)T * N, bias, bias_dtype, nullptr, 0};
        return 0;
    }
    const int out_dtype = residual ? F32 : BF16;
    if (int rc = infero_gemm_tc(a, w, bias, bias_dtype, dst, out_dtype, T, N, K, K, N, nullptr, 0, s.sm_count, 0, s.stream))
        return rc;
    *out = InferoDelta{dst, out_dtype, 1, 0, nullptr, F32, nullptr, 0};
    return 0;
}

// Can decode attention finish this block's q/k/v product itself in this step?  (A step of single tokens
// whose product comes as partial sums; INFERO_FUSED_DECODE=0 keeps the two kernels apart.)
static int g_fused_decode = -1, g_fused_norm = -1;       // -1: ask the environment at first use
static bool env_on(const char* name) {
    const char* e = getenv(name);
    return !(e && e[0] == '0');
}
static bool fused_decode(const InferoBlock& b, const InferoStep& s, const ArenaPlan& p) {
    if (g_fused_decode < 0) g_fused_decode = env_on("INFERO_FUSED_DECODE") ? 1 : 0;
    const bool wanted = g_fused_decode != 0;
    const int T = s.n_tokens, nqkv = (b.n_heads + 2 * b.n_kv) * b.head_dim;
    return wanted && T <= 256 && s.n_decode == s.n_entries && s.n_decode == T &&
           infero_attn_decode_fused_supported((const float*)(s.arena + p.qkv), (long long)T * nqkv, b.n_heads, b.n_kv,
                                              b.head_dim, b.page_size, b.rotary_dim, b.k_cache, b.v_cache);
}

// May the residual-add-and-norm kernels of such a step be folded into the products around them?
// (INFERO_FUSED_NORM=0 keeps them as kernels.)
static bool fused_norm_wanted() {
    if (g_fused_norm < 0) g_fused_norm = env_on("INFERO_FUSED_NORM") ? 1 : 0;
    return g_fused_norm != 0;
}
// A product whose splits add up inside a cluster has at most 8 of them.  Where the plan without that limit
// would cut K into many more (small matrices, whose products are bound by latency, not by bandwidth), the
// cluster's blocks each stream twice as long and the norm kernel saved does not make up for it (measured at
// hidden 896: 0.82 against 0.77 ms per step): the norm is then left as a kernel.
static bool cluster_plan_ok(int T, int N, int K, int sm_count, int* splits, int* per) {
    int ps = 1, pp = 1;
    long long ws = 0;
    infero_gemm_tc_plan(T, N, K, sm_count, &ps, &pp, &ws);
    infero_gemm_tc_plan_cluster(T, N, K, sm_count, splits, per);
    return *splits * 4 >= ps * 3;
}

// The two switches at run time (tests compare the folded launches with the separate ones).
void infero_block_set_fusion(int fused_decode_on, int fused_norm_on) {
    g_fused_decode = fused_decode_on ? 1 : 0;
    g_fused_norm = fused_norm_on ? 1 : 0;
}

// x += pending; the block; leaves its own feed-forward output pending in *delta.  layer_parity picks
// which of the arena's two output areas this layer writes (the other one still holds its input).
// next: the block that runs after this one on the same residual stream, or null (then, and whenever
// that block could not take it, the output is left pending as partial sums or a finished product).
int infero_block_forward(const InferoBlock* b, const InferoStep* s, const int* block_table, int max_blocks,
                         int layer_parity, InferoDelta* delta, const InferoBlock* next) {
    const int T = s->n_tokens;
    if (T == 0) return 0;
    const ArenaPlan p = plan_arena(*b, T, s->sm_count);
    if (p.total > s->arena_bytes) {
        infero_set_error("block_forward: %lld bytes of scratch needed for %d tokens, %lld given", p.total, T, s->arena_bytes);
        return 1;
    }
    uint8_t* A = s->arena;
    const int H = b->n_heads, Hkv = b->n_kv, D = b->head_dim, d = b->hidden, ff = b->intermediate;
    const int da = H * D, nqkv = (H + 2 * Hkv) * D;
    const int tiles = (d + 127) / 128;
    const float inv_d = 1.0f / (float)d;
    const bool fused = fused_decode(*b, *s, p);
    const bool fold_norms = fused && fused_norm_wanted();
    void* h = A + p.h;
    // ---- mixer ------------------------------------------------------------------------------------
    const float* ss_mixer = nullptr;                   // the first norm's scalar is still to be applied
    if (delta->data && delta->dtype == PRENORMED && fused) {
        h = const_cast<void*>(delta->data);
        ss_mixer = delta->sumsq;
    } else {
        const bool pending = delta->data && delta->dtype != PRENORMED;
        if (int rc = infero_add_rmsnorm(s->x, pending ? delta->data : nullptr, pending ? delta->dtype : F32,
                                        pending ? delta->splits : 1, pending ? delta->split_stride : 0,
                                        pending ? delta->bias : nullptr, delta->bias_dtype, b->w_norm_mixer, b->norm_dtype,
                                        b->eps_mixer, h, BF16, nullptr, T, d, s->stream))
            return rc;
    }
    InferoDelta qkv;
    if (int rc = product(*s, h, d, b->w_qkv, nqkv, b->b_qkv, b->qkv_bias_dtype, A + p.qkv, &qkv)) return rc;
    h = A + p.h;
    const void* q = nullptr;
    int q_stride = 0;
    // A step of single tokens whose q/k/v product came as partial sums: decode attention finishes the
    // product itself (bias, rotary positions, cache append), one launch instead of two.
    if (fused && qkv.dtype == F32) {
    } else if (qkv.dtype == F32) {
        q = A + p.q;
        q_stride = da;
        if (int rc = infero_rope_cache_partials((const float*)qkv.data, qkv.splits, qkv.split_stride, qkv.bias, qkv.bias_dtype,
                                                A + p.q, da, BF16, s->positions, s->tok_entry, block_table, max_blocks,
                                                b->inv_freq, b->rotary_dim, b->k_cache, b->v_cache, b->page_size, T, H, Hkv,
                                                D, b->write_cache, s->stream))
            return rc;
    } else {
        q = qkv.data;
        q_stride = nqkv;
        if (int rc = infero_rope_cache(A + p.qkv, BF16, nqkv, s->positions, s->tok_entry, block_table, max_blocks,
                                       b->inv_freq, b->rotary_dim, b->k_cache, b->v_cache, b->page_size, T, H, Hkv, D,
                                       b->write_cache, s->stream))
            return rc;
    }
    void* attn = A + p.attn;
    if (s->n_decode > 0) {
        int vis = s->decode_visible;
        if (b->window > 0) vis = std::min(vis, b->window + 15);
        int chunk, splits;
        infero_attn_plan_decode(s->n_decode, Hkv, H / Hkv, vis, s->sm_count, &chunk, &splits);
        if (infero_attn_decode_scratch(s->n_decode, H, D, splits) > p.o_delta - p.scratch) {
            infero_set_error("block_forward: %d decode tokens in %d splits need more scratch than was set aside", s->n_decode, splits);
            return 1;
        }
        int rc;
        if (fused && qkv.dtype == F32)
            rc = infero_attn_decode_tma_fused((const float*)qkv.data, qkv.splits, qkv.split_stride, qkv.bias, qkv.bias_dtype,
                                              b->inv_freq, b->rotary_dim, b->write_cache, attn, da, b->k_cache, b->v_cache,
                                              b->num_pages, block_table, max_blocks, s->tok_entry, s->positions, 0,
                                              s->n_decode, H, Hkv, D, b->page_size, b->window, b->scale, chunk, splits,
                                              A + p.scratch, s->counters, s->n_counters, ss_mixer, tiles, inv_d,
                                              b->eps_mixer, s->stream);
        else
            rc = infero_attn_decode_tma(q, q_stride, attn, da, b->k_cache, b->v_cache, b->num_pages, block_table,
                                        max_blocks, s->tok_entry, s->positions, 0, s->n_decode, H, Hkv, D,
                                        b->page_size, b->window, b->scale, chunk, splits, A + p.scratch, s->counters,
                                        s->n_counters, s->stream);
        if (rc) return rc;
    }
    if (s->n_decode < s->n_entries) {
        if (int rc = infero_attn_prefill_tc(q, q_stride, T, attn, da, b->k_cache, b->v_cache, b->num_pages, block_table,
                                            max_blocks, s->entry_q_start, s->entry_q_len, s->entry_pos0, s->n_entries,
                                            s->n_decode, s->prefill_tiles, H, Hkv, D, b->page_size, b->window, b->scale,
                                            s->stream))
            return rc;
    }
    // ---- output projection, second norm, feed-forward ----------------------------------------------
    void* act = A + p.act;
    int gu_splits = 1, gu_per = 1;
    long long gu_ws = 0;
    infero_gemm_tc_plan(T, 2 * ff, d, s->sm_count, &gu_splits, &gu_per, &gu_ws);
    int rc;
    int o_splits = 1, o_per = 1;
    if (fold_norms && gu_splits == 1 && cluster_plan_ok(T, d, da, s->sm_count, &o_splits, &o_per)) {
        // the output projection adds itself to x and leaves x * w and the sums of squares; the gate/up
        // product applies the norm's scalar to its own result before the activation
        float* ss_ffn = (float*)(A + p.sumsq[0]);
        if (int rc2 = infero_gemm_tc_residual_norm(attn, b->w_o, T, d, da, da, o_splits, o_per, s->x, b->b_o, b->o_bias_dtype,
                                                   b->w_norm_ffn, b->norm_dtype, h, ss_ffn, s->stream))
            return rc2;
        rc = infero_gemm_tc_swiglu_scaled(h, b->w_gate_up, act, T, 2 * ff, d, d, ff, ss_ffn, tiles, inv_d, b->eps_ffn,
                                          s->sm_count, s->stream);
    } else {
        InferoDelta o;
        if (int rc2 = product(*s, attn, da, b->w_o, d, b->b_o, b->o_bias_dtype, A + p.o_delta, &o, true)) return rc2;
        if (int rc2 = infero_add_rmsnorm(s->x, o.data, o.dtype, o.splits, o.split_stride, o.bias, o.bias_dtype, b->w_norm_ffn,
                                         b->norm_dtype, b->eps_ffn, h, BF16, nullptr, T, d, s->stream))
            return rc2;
        rc = infero_gemm_tc_swiglu(h, b->w_gate_up, act, T, 2 * ff, d, d, ff, s->sm_count, s->stream);
        if (rc == 2) {
            // few rows and K cut into splits: the activation is not linear, so the product comes as
            // partial sums and the SwiGLU kernel adds them up
            InferoDelta gu;
            if (int rc2 = product(*s, h, d, b->w_gate_up, 2 * ff, nullptr, F32, A + p.gate_up, &gu)) return rc2;
            rc = infero_swiglu(gu.data, gu.splits, gu.split_stride, act, F32, 1, T, ff, s->stream);
        }
    }
    if (rc) return rc;
    // ---- down projection -----------------------------------------------------------------------------
    int dn_splits = 1, dn_per = 1;
    if (fold_norms && next && next->hidden == d && next->norm_dtype == b->norm_dtype &&
        fused_decode(*next, *s, plan_arena(*next, T, s->sm_count)) &&
        cluster_plan_ok(T, d, ff, s->sm_count, &dn_splits, &dn_per)) {
        // the next layer is of the same kind and takes its input without its first norm's scalar
        float* ss_next = (float*)(A + p.sumsq[1]);
        if (int rc2 = infero_gemm_tc_residual_norm(act, b->w_down, T, d, ff, ff, dn_splits, dn_per, s->x, nullptr, F32,
                                                   next->w_norm_mixer, next->norm_dtype, h, ss_next, s->stream))
            return rc2;
        *delta = InferoDelta{h, PRENORMED, 1, 0, nullptr, F32, ss_next, tiles};
        return 0;
    }
    return product(*s, act, ff, b->w_down, d, nullptr, F32, A + p.delta[layer_parity & 1], delta, true);
}

// The whole model in one call: embedding, the schedule of built-in blocks, the final norm on the rows whose
// logits are wanted, the output product.  What ``DecoderModel.forward`` does when every entry of its
// schedule is a built-in block that goes the native way, launch for launch (the same functions with the
// same arguments), so the logits are the same bit for bit; the host's share of a step that is not replayed
// from a CUDA graph drops from a Python call per layer to this one call.  The reference runs its layer
// loop natively too (crates/model/src/lib.rs:3423-4243).
struct InferoDecoder {
    int n_entries;                  // executions of blocks, in the order they run
    const InferoBlock* blocks;      // one descriptor per execution (bound to its cache slot)
    const int* entry_group;         // which block table each execution reads
    const void* embed;              // [vocab, hidden]
    int embed_dtype, vocab, hidden;
    float embed_scale;
    const void* final_norm_w;
    int final_norm_dtype;
    float final_eps;
    const void* head_w;             // [vocab, hidden] bf16 (the embedding itself when tied)
    const void* head_bias;          // or null
    int head_bias_dtype;
};

// tables: one block table per layer group [n_entries of the step, max_blocks].  rows (n_rows of them, may be
// none): the step's rows whose logits are wanted; h_rows: bf16 [n_rows, hidden] scratch; logits: float
// [n_rows, vocab]; head_ws: what infero_gemm_tc_plan asks for the output product (may be null when nothing).
int infero_decoder_forward(const InferoDecoder* m, const InferoStep* s, const int* token_ids, const int* device_tokens,
                           const int* const* tables, int max_blocks, const int* rows, int n_rows, void* h_rows,
                           float* logits, void* head_ws, long long head_ws_bytes) {
    const int T = s->n_tokens;
    if (T == 0) return 0;
    if (int rc = infero_embed_gather(m->embed, m->embed_dtype, token_ids, device_tokens, s->x, T, m->hidden, m->vocab,
                                     m->embed_scale, s->stream))
        return rc;
    InferoDelta delta = {};
    for (int i = 0; i < m->n_entries; ++i) {
        const InferoBlock* next = i + 1 < m->n_entries ? &m->blocks[i + 1] : nullptr;
        if (int rc = infero_block_forward(&m->blocks[i], s, tables[m->entry_group[i]], max_blocks, i & 1, &delta, next))
            return rc;
    }
    if (n_rows == 0) return 0;
    const bool pending = delta.data && delta.dtype != PRENORMED;
    if (int rc = infero_add_rmsnorm(s->x, pending ? delta.data : nullptr, pending ? delta.dtype : F32,
                                    pending ? delta.splits : 1, pending ? delta.split_stride : 0,
                                    pending ? delta.bias : nullptr, delta.bias_dtype, m->final_norm_w, m->final_norm_dtype,
                                    m->final_eps, h_rows, BF16, rows, n_rows, m->hidden, s->stream))
        return rc;
    return infero_gemm_tc(h_rows, m->head_w, m->head_bias, m->head_bias_dtype, logits, F32, n_rows, m->vocab, m->hidden,
                          m->hidden, m->vocab, head_ws, head_ws_bytes, s->sm_count, 0, s->stream);
}

}  // extern "C"
