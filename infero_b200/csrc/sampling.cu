// Turning rows of logits into tokens on the device.
//
// The distribution is the reference's (crates/model/src/sampling.rs:169-235):
//   repetition penalty (divide a positive logit, multiply a negative one)
//   -> keep the top_k largest -> sort descending -> w = exp((z - max) / max(T, 1e-5))
//   -> top_p: shortest prefix whose mass reaches top_p * total (top_p clamped to [1e-4, 1])
//   -> r = u * total; the first candidate at which the running remainder is <= 0.
// Greedy is a strict '>' scan, so ties keep the lowest index (sampling.rs:302-310;
// crates/kernels/src/cu/sample.cu:42-47).  The uniform draw u comes from the host, one per
// row, as in the reference (crates/server/src/scheduler.rs:1279-1299), so a host sampler
// fed the same u picks the same token.
//
// The selection is a 4-pass radix select over order-preserving 32-bit keys with integer
// histograms, ties at the threshold taken in ascending index, so the result is a deterministic
// function of the row.  At most SAMPLE_MAX_K candidates survive the top-k stage; a larger (or
// disabled) top_k is clamped to that.  Small vocabularies: one block per row.  Large ones (a
// block alone takes hundreds of microseconds over 150,000 logits): blocks over chunks of 8,192
// logits each keep their chunk's k largest, then one block per row selects among those.
#include "common.cuh"
#include <math_constants.h>

extern "C" int infero_sm_count();     // runtime.cu
int infero_tc_err_flag(int** out);      // tc_host.cu: the flag that kernels with bounded waits raise

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_MAX_K = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
    // larger float -> larger unsigned key; NaN sorts lowest
    if (v != v) return 0u;
    uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

// (token, exponent) pairs: logits[row, token] is divided (if positive) or multiplied by
// penalty^exponent.  Pairs with token < 0 are padding.
__global__ void apply_penalty_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ pen_tokens,
                                     const int* __restrict__ pen_counts, int pen_stride,
                                     const float* __restrict__ penalty) {
    const int row = blockIdx.x;
    const float p = penalty[row];
    if (p == 1.0f) return;
    for (int i = threadIdx.x; i < pen_stride; i += blockDim.x) {
        const int tok = pen_tokens[(size_t)row * pen_stride + i];
        if (tok < 0 || tok >= vocab) continue;
        const int c = pen_counts[(size_t)row * pen_stride + i];
        float* z = logits + (size_t)row * vocab + tok;
        float v = *z;
        for (int k = 0; k < c; ++k) v = v > 0.f ? v / p : v * p;
        *z = v;
    }
}

// The same penalty from a history kept on the device: ring[slot][0 .. ring_width) holds a request's
// generated tokens (position n % ring_width for the n-th), ring_len[slot] how many there have been.
// The last min(len, window) of them count: a token seen c times is penalised c times in a sampled
// row and once in a greedy one (crates/model/src/sampling.rs:240-310).  One block per row; entry i of
// the window is thread i's; the first occurrence of a token does the work for all of them.
constexpr int PENALTY_RING_THREADS = 256;

__global__ void __launch_bounds__(PENALTY_RING_THREADS)
apply_penalty_ring_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ slot,
                          const float* __restrict__ penalty, const int* __restrict__ window,
                          const int* __restrict__ use_sample, const int* __restrict__ ring,
                          const int* __restrict__ ring_len, int ring_width) {
    extern __shared__ int recent[];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const float p = penalty[row];
    const int s = slot[row];
    if (p == 1.0f || s < 0) return;
    const int len = ring_len[s];
    int n = min(len, min(window[row], ring_width));
    if (n <= 0) return;
    const int* r = ring + (size_t)s * ring_width;
    for (int i = threadIdx.x; i < n; i += blockDim.x) recent[i] = r[(len - n + i) % ring_width];
    __syncthreads();
    const bool every = use_sample[row] != 0;             // sampled rows: once per occurrence
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int tok = recent[i];
        if (tok < 0 || tok >= vocab) continue;
        int count = 0;
        bool first = true;
        for (int j = 0; j < n; ++j) {
            if (recent[j] == tok) {
                if (j < i) { first = false; break; }
                ++count;
            }
        }
        if (!first) continue;
        float* z = logits + (size_t)row * vocab + tok;
        float v = *z;
        const int times = every ? count : 1;
        for (int k = 0; k < times; ++k) v = v > 0.f ? v / p : v * p;
        *z = v;
    }
}

// Greedy pick in two passes: every block scans one chunk of one row for its best (value, index),
// then one warp per row merges the chunks.  "Best" is the larger value, and among equal values
// the lower index, at every stage, so the result is the row's first maximum.
constexpr int ARGMAX_CHUNK = 4096, ARGMAX_THREADS = 256;

__device__ __forceinline__ void argmax_merge(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
}

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_partial_kernel(const float* __restrict__ logits, int vocab, int n_chunks, float* __restrict__ pv,
                      int* __restrict__ pi) {
    __shared__ float bv[ARGMAX_THREADS / 32];
    __shared__ int bi[ARGMAX_THREADS / 32];
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* z = logits + (size_t)row * vocab;
    const int lo = chunk * ARGMAX_CHUNK, hi = min(vocab, lo + ARGMAX_CHUNK);
    float best = -CUDART_INF_F;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) {
        const float v = z[i];
        if (v > best) { best = v; idx = i; }       // ascending i per thread: lowest index wins ties
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_merge(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < ARGMAX_THREADS / 32 ? bv[lane] : -CUDART_INF_F;
        idx = lane < ARGMAX_THREADS / 32 ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            argmax_merge(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
        if (lane == 0) { pv[(size_t)row * n_chunks + chunk] = best; pi[(size_t)row * n_chunks + chunk] = idx; }
    }
    TL_END(TL_ARGMAX);
}

__global__ void __launch_bounds__(128)
argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int n_rows, int n_chunks,
                    int* __restrict__ out) {
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    float best = -CUDART_INF_F;
    int idx = 0x7fffffff;
    for (int c = lane; c < n_chunks; c += 32) argmax_merge(best, idx, pv[(size_t)row * n_chunks + c], pi[(size_t)row * n_chunks + c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_merge(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) out[row] = (idx == 0x7fffffff) ? 0 : idx;   // all -inf / NaN: token 0
    TL_END(TL_ARGMAX_FINAL);
}

// final[r] = use_sample[r] ? sampled[r] : greedy[r];  device_tokens[slot[r]] = final[r]: the
// sampler's picks, left on the device for a step that is launched before the host reads them.
// With a ring (see apply_penalty_ring_kernel) the pick is also appended to its request's history.
// With fault_flag, final_tok[n_rows] receives the flag the kernels with bounded waits raise when a wait
// ran out, so that the host learns of it in the same copy that brings the picks.
__global__ void keep_tokens_kernel(const int* __restrict__ greedy, const int* __restrict__ sampled,
                                   const int* __restrict__ use_sample, const int* __restrict__ slot,
                                   int* __restrict__ final_tok, int* __restrict__ device_tokens, int n_rows,
                                   int* __restrict__ ring, int* __restrict__ ring_len, int ring_width,
                                   const int* __restrict__ fault_flag) {
    TL_BEGIN();
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r == 0 && fault_flag) final_tok[n_rows] = *(const volatile int*)fault_flag;
    if (r >= n_rows) return;
    const int tok = (sampled && use_sample[r]) ? sampled[r] : greedy[r];
    final_tok[r] = tok;
    const int s = slot[r];
    if (s < 0) return;
    device_tokens[s] = tok;
    if (ring) {
        const int len = ring_len[s];
        ring[(size_t)s * ring_width + len % ring_width] = tok;
        ring_len[s] = len + 1;
    }
    TL_END(TL_KEEP);
}

// Exclusive prefix sum of one int per thread over the block; returns the total too.
__device__ __forceinline__ int block_exclusive_scan(int v, int* total, int* warp_sums) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (int)((blockDim.x + 31) >> 5) ? warp_sums[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_sums[lane] = winc - w;
        if (lane == 31) warp_sums[32] = winc;
    }
    __syncthreads();
    *total = warp_sums[32];
    return warp_sums[warp] + inc - v;
}

// Where a selection reads its (key, token) pairs: a stretch of a row of logits, or the survivors
// that the chunks of a row left in scratch (SAMPLE_MAX_K slots per chunk, each chunk's in token order).
struct FromLogits {
    const float* z;
    int first;                                           // token of element 0
    __device__ __forceinline__ uint32_t key(int i) const { return order_key(z[i]); }
    __device__ __forceinline__ uint32_t token(int i) const { return (uint32_t)(first + i); }
};
struct FromChunks {
    const unsigned long long* list;                      // [chunks][SAMPLE_MAX_K]: (key << 32) | ~token
    int per_chunk;                                       // survivors of every chunk but perhaps the last
    __device__ __forceinline__ unsigned long long at(int i) const {
        return list[(size_t)(i / per_chunk) * SAMPLE_MAX_K + (i % per_chunk)];
    }
    __device__ __forceinline__ uint32_t key(int i) const { return (uint32_t)(at(i) >> 32); }
    __device__ __forceinline__ uint32_t token(int i) const { return ~(uint32_t)(at(i) & 0xffffffffull); }
};

constexpr int HIST_COPIES = 8;                           // warps spread over copies: fewer colliding atomics

// The k largest of src's n elements (ties at the threshold: lowest tokens first), written to cand[]
// in the order of the source (ascending token) as (key << 32) | ~token.  Returns how many (k, or n).
// A 4-pass radix select over order-preserving 32-bit keys with integer histograms: a deterministic
// function of the elements.  Every thread of the block calls it.
template <class Src>
__device__ int select_largest(const Src& src, int n, int k, unsigned long long* cand, int (*hist)[256], int* scan_ws,
                              uint32_t* s_prefix, int* s_need) {
    if (k > n) k = n;
    if (threadIdx.x == 0) { *s_prefix = 0u; *s_need = k; }
    __syncthreads();
    int* my_hist = hist[(threadIdx.x >> 5) % HIST_COPIES];
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = threadIdx.x; i < HIST_COPIES * 256; i += blockDim.x) hist[0][i] = 0;
        __syncthreads();
        const uint32_t prefix = *s_prefix;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const uint32_t key = src.key(i);
            if ((key & mask) == prefix) atomicAdd(&my_hist[(key >> shift) & 255], 1);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            int t = 0;
#pragma unroll
            for (int c = 0; c < HIST_COPIES; ++c) t += hist[c][i];
            hist[0][i] = t;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int need = *s_need, b = 255;
            for (; b > 0; --b) {
                if (hist[0][b] >= need) break;
                need -= hist[0][b];
            }
            *s_prefix = prefix | ((uint32_t)b << shift);
            *s_need = need;
        }
        __syncthreads();
    }
    const uint32_t thr = *s_prefix;    // key of the k-th largest
    const int need_eq = *s_need;       // how many elements equal to thr are taken (lowest tokens)

    // survivors in source order (a contiguous range per thread)
    const int per = (n + blockDim.x - 1) / blockDim.x;
    const int lo = min(n, (int)threadIdx.x * per), hi = min(n, lo + per);
    int n_gt = 0, n_eq = 0;
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = src.key(i);
        n_gt += key > thr;
        n_eq += key == thr;
    }
    int tot_gt, tot_eq;
    int off_gt = block_exclusive_scan(n_gt, &tot_gt, scan_ws);
    int off_eq = block_exclusive_scan(n_eq, &tot_eq, scan_ws);
    for (int i = threadIdx.x; i < SAMPLE_MAX_K; i += blockDim.x) cand[i] = 0ull;   // sorts last
    __syncthreads();
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = src.key(i);
        const unsigned long long e = ((unsigned long long)key << 32) | (uint32_t)(~src.token(i));
        if (key > thr) {
            cand[off_gt++] = e;
        } else if (key == thr) {
            if (off_eq < need_eq) cand[tot_gt + off_eq] = e;
            ++off_eq;
        }
    }
    __syncthreads();
    return tot_gt + min(need_eq, tot_eq);                // == k
}

__device__ __forceinline__ int effective_k(int k, int vocab) {
    if (k <= 0 || k > SAMPLE_MAX_K) k = SAMPLE_MAX_K;
    return k > vocab ? vocab : k;
}

// Stage 1 for large vocabularies: block (chunk, row) leaves the k largest of its chunk in scratch.
// The k largest of the row are among them, and the chunks' survivors, chunk after chunk, are in
// token order, so stage 2 selects from them exactly what it would select from the whole row.
constexpr int SAMPLE_CHUNK = 8192;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_chunk_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ top_k,
                    unsigned long long* __restrict__ scratch) {
    __shared__ int hist[HIST_COPIES][256];
    __shared__ int scan_ws[33];
    __shared__ unsigned long long cand[SAMPLE_MAX_K];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, chunk = blockIdx.x;
    const int lo = chunk * SAMPLE_CHUNK, n = min(SAMPLE_CHUNK, vocab - lo);
    const int k = effective_k(top_k[row], vocab);
    const FromLogits src{logits + (size_t)row * vocab + lo, lo};
    const int n_cand = select_largest(src, n, k, cand, hist, scan_ws, &s_prefix, &s_need);
    unsigned long long* dst = scratch + ((size_t)row * gridDim.x + chunk) * SAMPLE_MAX_K;
    for (int i = threadIdx.x; i < n_cand; i += blockDim.x) dst[i] = cand[i];
}

// The pick.  chunks == 0: the candidates are selected from the row of logits itself (small
// vocabularies); else from what sample_chunk_kernel left in scratch.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const double* __restrict__ draw, int* __restrict__ out, const unsigned long long* __restrict__ scratch,
              int chunks) {
    __shared__ int hist[HIST_COPIES][256];
    __shared__ int scan_ws[33];
    __shared__ unsigned long long cand[SAMPLE_MAX_K];   // (key << 32) | ~token : descending sort = value desc, token asc
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const int k = effective_k(top_k[row], vocab);
    int n_cand;
    if (chunks == 0) {
        const FromLogits src{logits + (size_t)row * vocab, 0};
        n_cand = select_largest(src, vocab, k, cand, hist, scan_ws, &s_prefix, &s_need);
    } else {
        const int last = vocab - (chunks - 1) * SAMPLE_CHUNK;
        const int per_chunk = min(k, SAMPLE_CHUNK);
        const FromChunks src{scratch + (size_t)row * chunks * SAMPLE_MAX_K, per_chunk};
        n_cand = select_largest(src, (chunks - 1) * per_chunk + min(k, last), k, cand, hist, scan_ws, &s_prefix, &s_need);
    }

    // ---- bitonic sort, descending, over the smallest power of two of slots that holds the candidates
    // (the slots past them hold 0, which sorts last) ---------------------------------------------------
    int sort_n = 2;
    while (sort_n < n_cand) sort_n <<= 1;
    for (int size = 2; size <= sort_n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = threadIdx.x;
            const int j = i ^ stride;
            if (i < sort_n && j > i) {
                const bool desc = (i & size) == 0;
                const unsigned long long a = cand[i], b = cand[j];
                if ((a < b) == desc) { cand[i] = b; cand[j] = a; }
            }
            __syncthreads();
        }
    }

    // ---- weights in parallel, then nucleus and pick in the reference's sequential order -------
    __shared__ double wd[SAMPLE_MAX_K];
    {
        const float t = fmaxf(temperature[row], 1e-5f);
        const float inv_t = 1.0f / t;
        const float zmax = key_value((uint32_t)(cand[0] >> 32));
        for (int i = threadIdx.x; i < n_cand; i += blockDim.x) {
            const float zi = key_value((uint32_t)(cand[i] >> 32));
            wd[i] = exp((double)((zi - zmax) * inv_t));
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the total is summed from the double weights; afterwards each weight is its float rounding
        double total = 0.0;
        for (int i = 0; i < n_cand; ++i) total += wd[i];
        int keep = n_cand;
        float tp = top_p[row];
        if (tp < 1.0f) {
            tp = fminf(fmaxf(tp, 1e-4f), 1.0f);
            const double target = total * (double)tp;
            double acc = 0.0;
            keep = 0;
            for (int i = 0; i < n_cand; ++i) {
                acc += (double)(float)wd[i];
                ++keep;
                if (acc >= target) break;
            }
            if (keep < 1) keep = 1;
            total = 0.0;
            for (int i = 0; i < keep; ++i) total += (double)(float)wd[i];
        }
        double r = draw[row] * total;
        int pick = keep - 1;
        for (int i = 0; i < keep; ++i) {
            r -= (double)(float)wd[i];
            if (r <= 0.0) { pick = i; break; }
        }
        out[row] = (int)(~(uint32_t)(cand[pick] & 0xffffffffull));
    }
}

}  // namespace

extern "C" {

int infero_apply_penalty(float* logits, int n_rows, int vocab, const int* pen_tokens, const int* pen_counts,
                         int pen_stride, const float* penalty, cudaStream_t stream) {
    if (n_rows == 0 || pen_stride == 0) return 0;
    apply_penalty_kernel<<<n_rows, 128, 0, stream>>>(logits, vocab, pen_tokens, pen_counts, pen_stride, penalty);
    return infero_check_launch("apply_penalty");
}

// Bytes of scratch infero_argmax needs for n_rows rows of vocab logits.
long long infero_argmax_scratch(int n_rows, int vocab) {
    const int n_chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    return (long long)n_rows * n_chunks * 8;
}

int infero_argmax(const float* logits, int n_rows, int vocab, int* out, void* scratch, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    INFERO_REQUIRE(vocab > 0 && n_rows <= 65535, "argmax: bad sizes rows=%d vocab=%d", n_rows, vocab);
    const int n_chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    float* pv = (float*)scratch;
    int* pi = (int*)(pv + (size_t)n_rows * n_chunks);
    launch_pdl(argmax_partial_kernel, dim3(n_chunks, n_rows), dim3(ARGMAX_THREADS), 0, stream, logits, vocab, n_chunks, pv, pi);
    if (infero_check_launch("argmax_partial")) return 1;
    launch_pdl(argmax_final_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, stream, (const float*)pv, (const int*)pi,
               n_rows, n_chunks, out);
    return infero_check_launch("argmax_final");
}

// Bytes of scratch infero_sample needs (0 for vocabularies small enough for one block per row).
static int sample_chunks(int vocab) { return vocab > 2 * SAMPLE_CHUNK ? (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK : 0; }
long long infero_sample_scratch(int n_rows, int vocab) {
    return (long long)n_rows * sample_chunks(vocab) * SAMPLE_MAX_K * 8;
}

int infero_sample(const float* logits, int n_rows, int vocab, const float* temperature, const int* top_k,
                  const float* top_p, const double* draw, int* out, void* scratch, long long scratch_bytes,
                  cudaStream_t stream) {
    if (n_rows == 0) return 0;
    INFERO_REQUIRE(vocab > 0 && n_rows <= 65535, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
    const int chunks = sample_chunks(vocab);
    if (chunks) {
        INFERO_REQUIRE(scratch && scratch_bytes >= infero_sample_scratch(n_rows, vocab),
                       "sample: %lld bytes of scratch needed, %lld given", infero_sample_scratch(n_rows, vocab), scratch_bytes);
        // few blocks: large ones finish sooner; many: small ones, eight to an SM, finish in one round
        const int chunk_threads = (long long)chunks * n_rows <= 2 * infero_sm_count() ? SAMPLE_THREADS : 256;
        launch_pdl(sample_chunk_kernel, dim3(chunks, n_rows), dim3(chunk_threads), 0, stream, logits, vocab, top_k,
                   (unsigned long long*)scratch);
        if (infero_check_launch("sample_chunk")) return 1;
    }
    launch_pdl(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab, temperature, top_k, top_p, draw,
               out, (const unsigned long long*)scratch, chunks);
    return infero_check_launch("sample");
}

// rows_info: [n_rows] slot per row, then [n_rows] use_sample flags.  final_tok [n_rows].
// ring [slots, ring_width] and ring_len [slots], or both null: the requests' generated tokens on the device.
// with_fault: final_tok has n_rows + 1 ints, the last one receives the device's fault flag (0: all waits were met).
int infero_keep_tokens(const int* greedy, const int* sampled, const int* rows_info, int* final_tok,
                       int* device_tokens, int n_rows, int* ring, int* ring_len, int ring_width, int with_fault,
                       cudaStream_t stream) {
    if (n_rows == 0) return 0;
    int* fault = nullptr;
    if (with_fault && infero_tc_err_flag(&fault)) return 1;
    launch_pdl(keep_tokens_kernel, dim3((n_rows + 127) / 128), dim3(128), 0, stream, greedy, sampled,
               rows_info + n_rows, rows_info, final_tok, device_tokens, n_rows, ring, ring_len, ring_width,
               (const int*)fault);
    return infero_check_launch("keep_tokens");
}

// rows_info as for infero_keep_tokens (slot per row, then the use-the-sample flag per row).
int infero_apply_penalty_ring(float* logits, int n_rows, int vocab, const int* rows_info, const float* penalty,
                              const int* window, const int* ring, const int* ring_len, int ring_width,
                              cudaStream_t stream) {
    if (n_rows == 0) return 0;
    INFERO_REQUIRE(ring_width > 0 && ring_width <= 8192, "apply_penalty_ring: ring of %d tokens", ring_width);
    launch_pdl(apply_penalty_ring_kernel, dim3(n_rows), dim3(PENALTY_RING_THREADS), (size_t)ring_width * sizeof(int), stream,
               logits, vocab, rows_info, penalty, window, rows_info + n_rows, ring, ring_len, ring_width);
    return infero_check_launch("apply_penalty_ring");
}

int infero_sample_max_k() { return SAMPLE_MAX_K; }

}  // extern "C"

INFERO_TL_UNIT(sampling)
