// bf16 matrix product on the 5th-generation tensor cores: out[M,N] = X[M,K] * W[N,K]^T (+ bias).
//
// One CTA computes one 128 x BN tile of D = A * B^T over a range of K, where A and B are both
// K-major row-major matrices (activations [M,K] and weights [N,K] are stored exactly so):
//   * TMA (cp.async.bulk.tensor, 128-byte swizzle) brings 128x64 and BNx64 bf16 tiles into a
//     ring of shared-memory stages, signalled through mbarriers;
//   * one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times per stage; the
//     accumulator lives in tensor memory (128 lanes x BN 32-bit columns);
//   * tcgen05.commit hands finished stages back to the loader and the finished accumulator
//     to four epilogue warps, which read it with tcgen05.ld and write the result.
// Warp roles: 0 loads, 1 owns TMEM and issues MMAs, 2..5 run the epilogue.
//
// Which matrix is "A" is the launcher's choice:
//   many tokens (M > 256): A = activations, B = weights; an epilogue thread owns one token
//     row and writes BN consecutive features (ROW mode).
//   few tokens (decode, small chunks): A = weights, B = activations, so that the 128-wide
//     side of the MMA is always full and the token side is as narrow as 16.  The CTAs then
//     number N/128 x splits of K, enough to keep every SM streaming weights; with more than
//     one split each CTA writes a 32-bit partial result [split, M, N] that the consumer
//     (reduce_partials here, or a fused norm / activation kernel) sums in a fixed order
//     (PARTIAL mode); with one split it writes the result itself (COL mode).
// The reference takes cuBLAS for the same products above a row threshold and its own
// mat-vec below (crates/model/src/lib.rs:8462-8505).
//
// Sizes: any M and N; K a multiple of 8 (rows must start on 16-byte boundaries for TMA);
// edges are zero-filled by TMA on the way in and masked on the way out.
#include "tc_common.cuh"
#include <atomic>
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>
#include <cstring>
#include <cstdlib>

namespace {

using namespace tc;

constexpr int TILE_A = 128;
constexpr int TILE_K = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int A_STAGE_BYTES = TILE_A * TILE_K * 2;

// The SWIGLU epilogues take a weight matrix whose rows alternate gate_j, up_j and write
// silu(gate_j) * up_j to column j of a bf16 result half as wide.
// EPI_CLUSTER: the CTAs that share a tile and differ in their split of K form a cluster; each leaves its
// 32-bit tile in its own shared memory and the cluster adds the tiles up through distributed shared
// memory, in ascending order of the splits, each CTA a share of the token columns: out[token, feature].
enum : int { EPI_ROW = 0, EPI_COL = 1, EPI_PARTIAL = 2, EPI_ROW_SWIGLU = 3, EPI_COL_SWIGLU = 4, EPI_CLUSTER = 5 };

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

template <int BN, int STAGES>
struct SmemPlan {
    static constexpr int B_STAGE_BYTES = BN * TILE_K * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int SCALE_OFFSET = BAR_OFFSET + 256;      // one float per token column (GemmFuse::sumsq_in)
    static constexpr int TOTAL = SCALE_OFFSET + BN * 4 + 1024; // barriers + scales + slack for 1024-byte alignment
};

// A layer's residual-add-and-norm kernels folded into the few-token products around them (steps of
// single tokens, where every launch costs more than its work).  RMSNorm is x * rsqrt(mean(x^2) + eps) * w
// and the product that follows is linear in its input, so the scalar rsqrt(...) of a token can be
// applied after the product; what is left of the norm is the residual sum, the weight and a sum of
// squares, which the product in front can do on its own output once its splits are added up:
//   producer (EPI_CLUSTER, x given): the summed tile is a residual update.  x[t, f] += sum (+ bias[f]);
//     h[t, f] = bf16(x[t, f] * norm_w[f]); sumsq_out[tile][t] = sum of x[t, f]^2 over the tile's features.
//   consumer (sumsq_in given): token t's column is scaled by rsqrt(sum_tiles sumsq_in[tile][t] * inv_d + eps)
//     (SwiGLU epilogue here; the fused decode attention does the same to the q/k/v partial sums).
constexpr int SUMSQ_STRIDE = 256;                              // floats between the tiles' rows of sums
struct GemmFuse {
    float* x;
    const void* bias;
    const void* norm_w;
    bf16* h;
    float* sumsq_out;
    const float* sumsq_in;
    int bias_dtype, norm_w_dtype, in_tiles;
    float inv_d, eps;
};

template <typename OutT>
__device__ __forceinline__ void store16(OutT* dst, const float* v, bool vec_ok);
template <>
__device__ __forceinline__ void store16<float>(float* dst, const float* v, bool vec_ok) {
    if (vec_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = v[i];
    }
}
template <>
__device__ __forceinline__ void store16<bf16>(bf16* dst, const float* v, bool vec_ok) {
    if (vec_ok) {
        uint32_t p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            p[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(p[4], p[5], p[6], p[7]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = __float2bfloat16_rn(v[i]);
    }
}

template <int BN, int STAGES, int EPI, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               OutT* __restrict__ out, const void* __restrict__ bias, int bias_dtype,
               int RA, int RB, int K, int ktiles_per_split, long long ldc, int a_evict_first,
               int* __restrict__ err_flag, const GemmFuse fuse) {
    using Plan = SmemPlan<BN, STAGES>;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFFSET);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* never_flag = abort_flag + 1;           // stays 0: for waits that must not be cut short

    TL_BEGIN();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * TILE_A, b0 = blockIdx.y * BN;
    const int total_kt = (K + TILE_K - 1) / TILE_K;
    const int kt_begin = blockIdx.z * ktiles_per_split;
    const int kt_end = min(total_kt, kt_begin + ktiles_per_split);
    const int n_kt = kt_end - kt_begin;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- loader --------------------------------------------------------------------------
        if (elect_one()) {
            // few-token path: A is the weight matrix, read once (evict first); B the activations,
            // read by every CTA (evict last)
            const uint64_t pol_a = policy_evict_first();
            const uint64_t pol_b = policy_evict_last();
            int issued = 0;
            bool ok = true;
            // The weights do not depend on the kernel before this one: their first tiles are on
            // their way before that kernel has finished (programmatic dependent launch); the
            // activations follow once it has.  The ring is empty, so these stages need no wait.
            const int pre = n_kt < STAGES ? n_kt : STAGES;
            for (int i = 0; i < pre; ++i) {
                uint8_t* sa = smem + i * Plan::STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], Plan::STAGE_BYTES);
                const int kx = (kt_begin + i) * TILE_K;
                if (a_evict_first) tma_load_2d_hint(sa, &map_a, kx, a0, &full_bar[i], pol_a);
                else tma_load_2d(sa + A_STAGE_BYTES, &map_b, kx, b0, &full_bar[i]);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                uint8_t* sa = smem + i * Plan::STAGE_BYTES;
                const int kx = (kt_begin + i) * TILE_K;
                if (a_evict_first) tma_load_2d_hint(sa + A_STAGE_BYTES, &map_b, kx, b0, &full_bar[i], pol_b);
                else tma_load_2d(sa, &map_a, kx, a0, &full_bar[i]);
                issued = i + 1;
            }
            for (int i = pre; i < n_kt; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                uint8_t* sa = smem + s * Plan::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], Plan::STAGE_BYTES);
                const int kx = (kt_begin + i) * TILE_K;
                if (a_evict_first) {
                    tma_load_2d_hint(sa, &map_a, kx, a0, &full_bar[s], pol_a);
                    tma_load_2d_hint(sa + A_STAGE_BYTES, &map_b, kx, b0, &full_bar[s], pol_b);
                } else {
                    tma_load_2d(sa, &map_a, kx, a0, &full_bar[s]);
                    tma_load_2d(sa + A_STAGE_BYTES, &map_b, kx, b0, &full_bar[s]);
                }
                issued = i + 1;
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 1);
            }
            if (*abort_flag) {
                // someone gave up: let the copies that are still in flight land before the
                // block (and its shared memory) goes away
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    mbar_wait(&full_bar[i % STAGES], (uint32_t)(i / STAGES) & 1u, never_flag);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue -----------------------------------------------------------------------
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_bf16_f32(TILE_A, BN);
            bool ok = true;
            for (int i = 0; i < n_kt; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(smem + s * Plan::STAGE_BYTES);
                const uint64_t da = smem_desc_k_sw128(sa);
                const uint64_t db = smem_desc_k_sw128(sa + A_STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                    // 16 elements along K = 32 bytes = 2 units of the descriptor's address field
                    umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                              (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);
            }
            if (ok) {
                umma_commit(accum_bar);
            } else {
                *abort_flag = 1;
                atomicExch(err_flag, 2);
            }
        }
    } else {
        // ---- epilogue ------------------------------------------------------------------------
        const int q = warp & 3;                              // the TMEM lane quarter this warp may read
        const int ra = a0 + q * 32 + lane;
        float* col_scale = reinterpret_cast<float*>(smem + Plan::SCALE_OFFSET);
        if (EPI == EPI_COL_SWIGLU && fuse.sumsq_in) {
            // the tokens' scales, while the product runs: the sums of squares come from the kernel in front
            pdl_wait();
            for (int c = (warp - 2) * 32 + lane; c < BN; c += 128) {
                float ss = 0.f;
                if (b0 + c < RB)
                    for (int tl = 0; tl < fuse.in_tiles; ++tl) ss += __ldcg(fuse.sumsq_in + (size_t)tl * SUMSQ_STRIDE + b0 + c);
                col_scale[c] = 1.0f / sqrtf(ss * fuse.inv_d + fuse.eps);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const bool ok = mbar_wait(accum_bar, 0, abort_flag);
        tc_fence_after_sync();
        if (ok) {
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (b0 + c0 >= RB) break;                    // uniform over the block
                __syncwarp();
                float v[16];
                tmem_ld16(lane_addr + (uint32_t)c0, v);
                const int rb = b0 + c0;
                if (EPI == EPI_CLUSTER) {
                    // the ring is free (every load was consumed and every MMA has finished): the tile goes
                    // there, token-major, so that the threads of a warp touch consecutive words
                    float* stage = reinterpret_cast<float*>(smem);
#pragma unroll
                    for (int i = 0; i < 16; ++i) stage[(c0 + i) * TILE_A + q * 32 + lane] = v[i];
                    continue;
                }
                if (EPI == EPI_COL_SWIGLU) {
                    // lanes 2j, 2j+1 hold gate_j and up_j of the same tokens: out[rb + i, ra / 2]
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if (fuse.sumsq_in) v[i] *= col_scale[c0 + i];
                        const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);
                        if (!(lane & 1) && ra + 1 < RA && rb + i < RB)
                            out[(size_t)(rb + i) * ldc + (ra >> 1)] = from_f32<OutT>(silu_mul(v[i], other));
                    }
                    continue;
                }
                if (ra >= RA) continue;
                if (EPI == EPI_ROW_SWIGLU) {
                    // columns 2j, 2j+1 of this token's row are gate_j and up_j: out[ra, rb / 2 ..]
                    OutT* dst = out + (size_t)ra * ldc + (rb >> 1);
                    float h[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) h[i] = silu_mul(v[2 * i], v[2 * i + 1]);
                    if (rb + 16 <= RB && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && sizeof(OutT) == 2) {
                        uint32_t pk[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
                            pk[i] = *reinterpret_cast<uint32_t*>(&t2);
                        }
                        *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (rb + 2 * i + 1 < RB) dst[i] = from_f32<OutT>(h[i]);
                    }
                } else if (EPI == EPI_ROW) {
                    // out[ra, rb .. rb+15] (+ bias[rb ..])
                    OutT* dst = out + (size_t)ra * ldc + rb;
                    const bool full = rb + 16 <= RB;
                    if (bias) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (rb + i < RB) v[i] += load_any(bias, bias_dtype, rb + i);
                    }
                    if (full) {
                        const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
                        store16<OutT>(dst, v, vec_ok);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (rb + i < RB) dst[i] = from_f32<OutT>(v[i]);
                    }
                } else if (EPI == EPI_COL) {
                    // out[rb + i, ra] (+ bias[ra]): lanes walk consecutive features
                    const float bv = bias ? load_any(bias, bias_dtype, ra) : 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (rb + i < RB) out[(size_t)(rb + i) * ldc + ra] = from_f32<OutT>(v[i] + bv);
                } else {
                    // partial[split, rb + i, ra], 32-bit
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (rb + i < RB)
                            out[((size_t)blockIdx.z * RB + (rb + i)) * (size_t)RA + ra] = from_f32<OutT>(v[i]);
                }
            }
        } else if (lane == 0) {
            *abort_flag = 1;
            atomicExch(err_flag, 3);
        }
    }
    if (EPI == EPI_CLUSTER) {
        // every thread of every CTA of the cluster comes here, also after a wait that ran out
        __syncwarp();
        cluster_sync_all();                                  // all tiles are in shared memory
        if (warp >= 2 && !*abort_flag) {
            const int S = (int)gridDim.z;                    // = the cluster's size: one CTA per split
            const int rank = (int)cluster_ctarank();
            const int n_cols = min(BN, RB - b0);
            const int per_rank = (n_cols + S - 1) / S;
            const int c_lo = rank * per_rank, c_hi = min(n_cols, c_lo + per_rank);
            const int row = (warp & 3) * 32 + lane, ra = a0 + row;
            uint32_t remote[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) remote[sp] = cluster_addr_of(smem, (uint32_t)(sp < S ? sp : 0));
            // (behind the tile this CTA staged for the cluster: one float per epilogue warp and token)
            float* warp_sq = reinterpret_cast<float*>(smem) + BN * TILE_A;
            float bias_v = 0.f, norm_w_v = 0.f;
            if (fuse.x && ra < RA) {
                if (fuse.bias) bias_v = load_any(fuse.bias, fuse.bias_dtype, ra);
                norm_w_v = load_any(fuse.norm_w, fuse.norm_w_dtype, ra);
            }
            // four tokens at a time: the loads of all of them (the splits' tiles through distributed shared
            // memory, the residual stream from global memory) are on their way before the first sum
            for (int cb = c_lo; cb < c_hi; cb += 4) {
                float v[4][8], xin[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = cb + u;
                    if (c < c_hi) {
                        const uint32_t off = (uint32_t)(c * TILE_A + row) * 4u;
#pragma unroll
                        for (int sp = 0; sp < 8; ++sp)
                            if (sp < S) v[u][sp] = ld_cluster_f32(remote[sp] + off);
                        if (fuse.x && ra < RA) xin[u] = __ldcg(fuse.x + (size_t)(b0 + c) * (size_t)RA + ra);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = cb + u;
                    if (c >= c_hi) break;
                    float acc = v[u][0];
#pragma unroll
                    for (int sp = 1; sp < 8; ++sp)
                        if (sp < S) acc += v[u][sp];
                    if (fuse.x) {
                        float sq = 0.f;
                        if (ra < RA) {
                            const size_t at = (size_t)(b0 + c) * (size_t)RA + ra;
                            const float xv = xin[u] + (acc + bias_v);
                            fuse.x[at] = xv;
                            fuse.h[at] = __float2bfloat16_rn(xv * norm_w_v);
                            sq = xv * xv;
                        }
                        sq = warp_sum(sq);
                        if (lane == 0) warp_sq[(warp & 3) * BN + (c - c_lo)] = sq;
                    } else if (ra < RA) {
                        out[(size_t)(b0 + c) * (size_t)RA + ra] = from_f32<OutT>(acc);
                    }
                }
            }
            if (fuse.x) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                // the four warps' sums in the order of their rows: warps 2, 3 hold rows 64..127, warps 4, 5 rows 0..63
                for (int j = (warp - 2) * 32 + lane; j < c_hi - c_lo; j += 128)
                    fuse.sumsq_out[(size_t)blockIdx.x * SUMSQ_STRIDE + b0 + c_lo + j] =
                        (warp_sq[0 * BN + j] + warp_sq[1 * BN + j]) + (warp_sq[2 * BN + j] + warp_sq[3 * BN + j]);
            }
        }
        cluster_sync_all();                                  // nobody leaves while its tile is still being read
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    TL_END(TL_GEMM);
}

// One epilogue warp's share of a finished accumulator: its 32 rows (TMEM lanes at lane_addr, result
// row ra for this thread) by BN columns starting at feature b0, written as the epilogue EPI says.
template <int EPI, typename OutT>
__device__ __forceinline__ void drain_accumulator(uint32_t lane_addr, int ra, int b0, int BN, int RA, int RB,
                                                  OutT* __restrict__ out, const void* __restrict__ bias,
                                                  int bias_dtype, long long ldc) {
    const int col_end = min(RB, b0 + BN);                // what this tile owns
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        if (b0 + c0 >= col_end) break;               // uniform over the block
        uint32_t u[32];
        tmem_ld32_nowait(lane_addr + (uint32_t)c0, u);
        tmem_wait_ld();
        if (ra < RA) {
#pragma unroll
            for (int hseg = 0; hseg < 2; ++hseg) {
                const int rb = b0 + c0 + hseg * 16;
                if (rb >= col_end) break;
                float v[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(u[hseg * 16 + e]);
                if (EPI == EPI_ROW_SWIGLU) {
                    OutT* dst = out + (size_t)ra * ldc + (rb >> 1);
                    float h[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) h[e] = silu_mul(v[2 * e], v[2 * e + 1]);
                    if (rb + 16 <= RB && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && sizeof(OutT) == 2) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(h[2 * e], h[2 * e + 1]);
                            pk[e] = *reinterpret_cast<uint32_t*>(&t2);
                        }
                        *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (rb + 2 * e + 1 < RB) dst[e] = from_f32<OutT>(h[e]);
                    }
                } else {
                    OutT* dst = out + (size_t)ra * ldc + rb;
                    if (bias) {
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if (rb + e < RB) v[e] += load_any(bias, bias_dtype, rb + e);
                    }
                    if (rb + 16 <= RB) {
                        store16<OutT>(dst, v, (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if (rb + e < RB) dst[e] = from_f32<OutT>(v[e]);
                    }
                }
            }
        }
        __syncwarp();
    }
}

// ---- many tokens: persistent, two accumulators --------------------------------------------------
// One CTA per SM walks over 128 x 256 tiles of the result (tile t = blockIdx.x, + gridDim.x, ...).
// Tile numbers run over the token blocks of one block of 256 features first, so that at any
// moment the CTAs together work on a few feature blocks and all token blocks, which L2 holds.  The shared-memory ring runs on across tiles; tensor memory
// holds two accumulators of 256 columns, so the four epilogue warps drain tile i while the MMAs
// of tile i + 1 run.  A = activations [RA, K], B = weights [RB, K].
// The tile width bn (a multiple of 16 up to 256) is chosen per problem so that the tiles fill
// whole rounds of the CTAs (3584 features in tiles of 256 are 224 tiles with 16 token blocks:
// two rounds on 148 SMs, the second half empty; in tiles of 208 they are 288 and nearly fill two).
constexpr int PERS_MAX_BN = 256, PERS_STAGES = 4;

template <int EPI, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          OutT* __restrict__ out, const void* __restrict__ bias, int bias_dtype,
                          int RA, int RB, int K, long long ldc, int BN, int* __restrict__ err_flag) {
    constexpr int STAGES = PERS_STAGES;
    using Plan = SmemPlan<PERS_MAX_BN, STAGES>;             // where the barriers sit; stages are packed by BN
    const int stage_bytes = A_STAGE_BYTES + BN * TILE_K * 2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFFSET);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;             // 2
    uint64_t* acc_empty = acc_full + 2;                  // 2 (four arrivals: one per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* never_flag = abort_flag + 1;

    TL_BEGIN();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_a = (RA + TILE_A - 1) / TILE_A, tiles_b = (RB + BN - 1) / BN;
    const int n_tiles = tiles_a * tiles_b;
    const int n_kt = (K + TILE_K - 1) / TILE_K;
    const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);
        }
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * PERS_MAX_BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- loader: the ring index runs over (tile, k-tile) pairs ---------------------------------
        if (elect_one()) {
            const long long total = (long long)my_tiles * n_kt;
            long long issued = 0;
            bool ok = true;
            // (tile, k-tile) of the next load, kept as running counters
            int tile = (int)blockIdx.x, kt = 0;
            int a0 = (tile % tiles_a) * TILE_A, b0 = (tile / tiles_a) * BN;
            auto advance = [&]() {
                if (++kt == n_kt) {
                    kt = 0;
                    tile += (int)gridDim.x;
                    a0 = (tile % tiles_a) * TILE_A;
                    b0 = (tile / tiles_a) * BN;
                }
            };
            // weights of the first stages before the kernel in front has finished, activations after
            const int pre = (int)(total < STAGES ? total : STAGES);
            int pa0[STAGES], pkx[STAGES];
            for (int it = 0; it < pre; ++it) {
                mbar_expect_tx(&full_bar[it], stage_bytes);
                tma_load_2d(smem + it * stage_bytes + A_STAGE_BYTES, &map_b, kt * TILE_K, b0, &full_bar[it]);
                pa0[it] = a0;
                pkx[it] = kt * TILE_K;
                advance();
            }
            pdl_wait();
            for (int it = 0; it < pre; ++it) {
                tma_load_2d(smem + it * stage_bytes, &map_a, pkx[it], pa0[it], &full_bar[it]);
                issued = it + 1;
            }
            int s = pre % STAGES;
            uint32_t ph = (uint32_t)(pre / STAGES) & 1u;
            for (long long it = pre; it < total; ++it) {
                if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                uint8_t* sa = smem + s * stage_bytes;
                mbar_expect_tx(&full_bar[s], stage_bytes);
                tma_load_2d(sa, &map_a, kt * TILE_K, a0, &full_bar[s]);
                tma_load_2d(sa + A_STAGE_BYTES, &map_b, kt * TILE_K, b0, &full_bar[s]);
                issued = it + 1;
                advance();
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 1);
            }
            if (*abort_flag) {
                for (long long it = issued > STAGES ? issued - STAGES : 0; it < issued; ++it)
                    mbar_wait(&full_bar[it % STAGES], (uint32_t)(it / STAGES) & 1u, never_flag);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ---------------------------------------------------------------------------
        if (elect_one()) {
            const uint32_t idesc = idesc_bf16_f32(TILE_A, BN);
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int a = i & 1;
                // the epilogue has drained this accumulator's previous tile
                if (!mbar_wait(&acc_empty[a], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)a * PERS_MAX_BN;
                for (int kt = 0; kt < n_kt; ++kt) {
                    if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * stage_bytes);
                    const uint64_t da = smem_desc_k_sw128(sa);
                    const uint64_t db = smem_desc_k_sw128(sa + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        umma_bf16(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[a]);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 2);
            }
        }
    } else {
        // ---- epilogue: tile i while the MMAs of tile i + 1 run ------------------------------------
        const int q = warp & 3;
        bool ok = true;
        for (int i = 0; i < my_tiles; ++i) {
            const int a = i & 1;
            const int t = (int)blockIdx.x + i * (int)gridDim.x;
            const int a0 = (t % tiles_a) * TILE_A, b0 = (t / tiles_a) * BN;
            const int ra = a0 + q * 32 + lane;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[a], (uint32_t)(i >> 1) & 1u, abort_flag))) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t lane_addr = tmem_base + (uint32_t)a * PERS_MAX_BN + ((uint32_t)(q * 32) << 16);
            drain_accumulator<EPI, OutT>(lane_addr, ra, b0, BN, RA, RB, out, bias, bias_dtype, ldc);
            // this warp has read its quarter of the accumulator: hand it back
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[a]);
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicExch(err_flag, 3);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * PERS_MAX_BN);
    }
    TL_END(TL_GEMM);
}

// ---- many tokens: a pair of CTAs per tile (cta_group::2) ---------------------------------------------
// A cluster of two CTAs works on tiles of 256 token rows x BN features.  Each CTA loads its own 128
// rows of the activations and its own half of the tile's weight rows, so every byte enters the
// pair's shared memory once and an SM's shared memory takes 128 + BN/2 rows per step of K instead
// of 128 + BN; the CTA of rank 0 issues the MMAs for both, each CTA's tensor memory holds the
// accumulator rows of its own tokens, and each CTA's four epilogue warps write those rows.  All
// loads of a stage report to rank 0's barrier; the commits that free a stage or publish an
// accumulator reach both CTAs; the epilogue warps of both hand an accumulator back on rank 0's
// barrier.  The pairs walk the tiles as the single CTAs above do.
constexpr int PAIR_STAGES = 6, PAIR_ROWS = 2 * TILE_A;

template <int EPI, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OutT* __restrict__ out, const void* __restrict__ bias, int bias_dtype,
                    int RA, int RB, int K, long long ldc, int BN, int* __restrict__ err_flag) {
    constexpr int STAGES = PAIR_STAGES;
    constexpr int BAR_OFFSET = STAGES * (A_STAGE_BYTES + (PERS_MAX_BN / 2) * TILE_K * 2);
    const int half_bn = BN >> 1;
    const int stage_bytes = A_STAGE_BYTES + half_bn * TILE_K * 2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + BAR_OFFSET);    // used in rank 0
    uint64_t* empty_bar = full_bar + STAGES;                                 // in both
    uint64_t* acc_full = empty_bar + STAGES;                                 // 2, in both
    uint64_t* acc_empty = acc_full + 2;                                      // 2, used in rank 0 (eight arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* never_flag = abort_flag + 1;

    TL_BEGIN();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
    const int tiles_a = (RA + PAIR_ROWS - 1) / PAIR_ROWS, tiles_b = (RB + BN - 1) / BN;
    const int n_tiles = tiles_a * tiles_b;
    const int n_kt = (K + TILE_K - 1) / TILE_K;
    const int my_tiles = pair < n_tiles ? (n_tiles - 1 - pair) / n_pairs + 1 : 0;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 8);
        }
        *abort_flag = 0;
        *never_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * PERS_MAX_BN);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();                                   // both CTAs' barriers exist before either is used
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- loader (one thread in each CTA) ---------------------------------------------------------
        if (elect_one()) {
            const long long total = (long long)my_tiles * n_kt;
            long long issued = 0;
            bool ok = true;
            int tile = pair, kt = 0;
            int a0 = (tile % tiles_a) * PAIR_ROWS + (int)rank * TILE_A;
            int b0 = (tile / tiles_a) * BN + (int)rank * half_bn;
            auto advance = [&]() {
                if (++kt == n_kt) {
                    kt = 0;
                    tile += n_pairs;
                    a0 = (tile % tiles_a) * PAIR_ROWS + (int)rank * TILE_A;
                    b0 = (tile / tiles_a) * BN + (int)rank * half_bn;
                }
            };
            uint32_t lead_full[STAGES];
            for (int s = 0; s < STAGES; ++s) lead_full[s] = cluster_addr_of(&full_bar[s], 0);
            // weights of the first stages before the kernel in front has finished, activations after
            const int pre = (int)(total < STAGES ? total : STAGES);
            int pa0[STAGES], pkx[STAGES];
            for (int it = 0; it < pre; ++it) {
                if (rank == 0) mbar_expect_tx(&full_bar[it], 2 * stage_bytes);
                tma_load_2d_pair(smem + it * stage_bytes + A_STAGE_BYTES, &map_b, kt * TILE_K, b0, lead_full[it]);
                pa0[it] = a0;
                pkx[it] = kt * TILE_K;
                advance();
            }
            pdl_wait();
            for (int it = 0; it < pre; ++it) {
                tma_load_2d_pair(smem + it * stage_bytes, &map_a, pkx[it], pa0[it], lead_full[it]);
                issued = it + 1;
            }
            int s = pre % STAGES;
            uint32_t ph = (uint32_t)(pre / STAGES) & 1u;
            for (long long it = pre; it < total; ++it) {
                if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                uint8_t* sa = smem + s * stage_bytes;
                if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * stage_bytes);
                tma_load_2d_pair(sa, &map_a, kt * TILE_K, a0, lead_full[s]);
                tma_load_2d_pair(sa + A_STAGE_BYTES, &map_b, kt * TILE_K, b0, lead_full[s]);
                issued = it + 1;
                advance();
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 1);
            }
            if (*abort_flag && rank == 0) {
                // what is still in flight into rank 0's own stages reports to these barriers
                for (long long it = issued > STAGES ? issued - STAGES : 0; it < issued; ++it)
                    mbar_wait(&full_bar[it % STAGES], (uint32_t)(it / STAGES) & 1u, never_flag);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue: rank 0 for the pair -----------------------------------------------------------
        if (rank == 0 && elect_one()) {
            const uint32_t idesc = idesc_bf16_f32(PAIR_ROWS, BN);
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int a = i & 1;
                if (!mbar_wait(&acc_empty[a], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)a * PERS_MAX_BN;
                for (int kt = 0; kt < n_kt; ++kt) {
                    if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * stage_bytes);
                    const uint64_t da = smem_desc_k_sw128(sa);
                    const uint64_t db = smem_desc_k_sw128(sa + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        umma_bf16_pair(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty_bar[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit_pair(&acc_full[a]);
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err_flag, 2);
            }
        }
    } else {
        // ---- epilogue: each CTA its own 128 rows ------------------------------------------------------
        const int q = warp & 3;
        bool ok = true;
        uint32_t lead_empty[2];
        for (int a = 0; a < 2; ++a) lead_empty[a] = cluster_addr_of(&acc_empty[a], 0);
        for (int i = 0; i < my_tiles; ++i) {
            const int a = i & 1;
            const int t = pair + i * n_pairs;
            const int a0 = (t % tiles_a) * PAIR_ROWS + (int)rank * TILE_A, b0 = (t / tiles_a) * BN;
            const int ra = a0 + q * 32 + lane;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[a], (uint32_t)(i >> 1) & 1u, abort_flag))) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t lane_addr = tmem_base + (uint32_t)a * PERS_MAX_BN + ((uint32_t)(q * 32) << 16);
            drain_accumulator<EPI, OutT>(lane_addr, ra, b0, BN, RA, RB, out, bias, bias_dtype, ldc);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_empty[a]);
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicExch(err_flag, 3);
        }
    }
    // neither CTA may leave while the other can still read its shared memory or signal its barriers
    __syncwarp();
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 2 * PERS_MAX_BN);
    }
    TL_END(TL_GEMM);
}

// out[t, n] = sum_s partial[s, t, n] (+ bias[n]); the sum runs over s in ascending order.
template <typename OutT>
__global__ void reduce_partials_kernel(const float* __restrict__ partial, int splits, const void* __restrict__ bias,
                                       int bias_dtype, OutT* __restrict__ out, int M, int N, long long ldc) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / N), n = (int)(i - (size_t)t * N);
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) acc += partial[(size_t)s * total + i];
        if (bias) acc += load_any(bias, bias_dtype, n);
        out[(size_t)t * ldc + n] = from_f32<OutT>(acc);
    }
}

// ---- host ------------------------------------------------------------------------------------
int get_map(const void* ptr, int rows, int cols, int ld, int box_rows, CUtensorMap* out) {
    return infero_tensor_map_bf16(ptr, rows, cols, ld, box_rows, out);
}

int err_flag_ptr(int** out) { return infero_tc_err_flag(out); }

template <int BN, int STAGES, int EPI, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* out, const void* bias, int bias_dtype, int RA,
           int RB, int K, int ktiles_per_split, int splits, long long ldc, int a_evict_first, int* err,
           cudaStream_t stream, const GemmFuse& fuse = GemmFuse{}) {
    using Plan = SmemPlan<BN, STAGES>;
    auto kern = gemm_tc_kernel<BN, STAGES, EPI, OutT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::TOTAL);
        if (e != cudaSuccess) {
            infero_set_error("gemm_tc: cannot get %d bytes of shared memory: %s", Plan::TOTAL, cudaGetErrorString(e));
            return 1;
        }
        configured = true;
    }
    dim3 grid((RA + TILE_A - 1) / TILE_A, (RB + BN - 1) / BN, splits);
    launch_pdl(kern, grid, dim3(GEMM_THREADS), Plan::TOTAL, stream, ma, mb, (OutT*)out, bias, bias_dtype, RA, RB, K,
               ktiles_per_split, ldc, a_evict_first, err, fuse);
    return infero_check_launch("gemm_tc");
}

// The few-token kernel with the splits of a tile as one cluster (at most 8 CTAs).
template <int BN, int STAGES>
int launch_cluster(const CUtensorMap& ma, const CUtensorMap& mb, float* out, int RA, int RB, int K,
                   int ktiles_per_split, int splits, int* err, cudaStream_t stream, const GemmFuse& fuse = GemmFuse{}) {
    using Plan = SmemPlan<BN, STAGES>;
    auto kern = gemm_tc_kernel<BN, STAGES, EPI_CLUSTER, float>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::TOTAL);
        if (e != cudaSuccess) {
            infero_set_error("gemm_tc: cannot get %d bytes of shared memory: %s", Plan::TOTAL, cudaGetErrorString(e));
            return 1;
        }
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((RA + TILE_A - 1) / TILE_A, (RB + BN - 1) / BN, splits);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Plan::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = infero_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, ma, mb, out, (const void*)nullptr, 0, RA, RB, K, ktiles_per_split, (long long)0, 1, err, fuse);
    return infero_check_launch("gemm_tc_cluster");
}

// Splits of a tile add up inside a cluster when INFERO_GEMM_CLUSTER=1 (or infero_gemm_set_cluster(1)).
// Off by default: measured on whole decode steps it gains nothing at batch 1 and 64 and loses 1.6 % at
// batch 8 (a cluster starts only when all of its CTAs find room at once, which costs more of the early
// weight prefetch than the partial sums' trip through L2 did).
constexpr int MAX_CLUSTER = 8;
std::atomic<int> g_cluster{-1};
bool cluster_sum() {
    int v = g_cluster.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("INFERO_GEMM_CLUSTER");
        v = (e && e[0] == '1') ? 1 : 0;
        g_cluster.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

// Tile width for the persistent kernel: the multiple of 16 (64..256) with the shortest schedule.
// A tile's time does not shrink in proportion to its width (the token operand is read from
// shared memory for every MMA whatever the width): measured at K = 18944 a tile of width bn
// costs about bn + 200 columns' worth.
int pick_tile_n(int M, int N, int ctas, int multiple) {
    if (const char* e = getenv("INFERO_GEMM_TILE_N")) {       // tuning knob: force a width
        const int v = atoi(e);
        if (v >= 16 && v <= PERS_MAX_BN && v % multiple == 0) return v;
    }
    const int tiles_a = (M + TILE_A - 1) / TILE_A;
    long long best_cost = -1;
    int best = PERS_MAX_BN;
    for (int bn = PERS_MAX_BN; bn >= 64; bn -= 16) {
        if (bn % multiple) continue;
        const long long tiles = (long long)tiles_a * ((N + bn - 1) / bn);
        const long long rounds = (tiles + ctas - 1) / ctas;
        const long long cost = rounds * (bn + 200);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

template <int EPI, typename OutT>
int launch_persistent(const void* x, const void* w, void* out, const void* bias, int bias_dtype,
                      int RA, int RB, int K, int ldx, long long ldc, int sm_count, int* err, cudaStream_t stream) {
    using Plan = SmemPlan<PERS_MAX_BN, PERS_STAGES>;
    auto kern = gemm_tc_persistent_kernel<EPI, OutT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::TOTAL);
        if (e != cudaSuccess) {
            infero_set_error("gemm_tc: cannot get %d bytes of shared memory: %s", Plan::TOTAL, cudaGetErrorString(e));
            return 1;
        }
        configured = true;
    }
    const int sms = sm_count > 0 ? sm_count : 148;
    const int bn = pick_tile_n(RA, RB, sms, EPI == EPI_ROW_SWIGLU ? 32 : 16);
    CUtensorMap ma, mb;
    if (get_map(x, RA, K, ldx, TILE_A, &ma)) return 1;
    if (get_map(w, RB, K, K, bn, &mb)) return 1;
    const int n_tiles = ((RA + TILE_A - 1) / TILE_A) * ((RB + bn - 1) / bn);
    const int ctas = n_tiles < sms ? n_tiles : sms;
    launch_pdl(kern, dim3(ctas), dim3(GEMM_THREADS), Plan::TOTAL, stream, ma, mb, (OutT*)out, bias, bias_dtype, RA, RB,
               K, ldc, bn, err);
    return infero_check_launch("gemm_tc_persistent");
}

// Tile width for pairs of CTAs (256 token rows per tile).
int pick_pair_tile_n(int M, int N, int pairs, int multiple) {
    if (const char* e = getenv("INFERO_GEMM_TILE_N")) {
        const int v = atoi(e);
        if (v >= 32 && v <= PERS_MAX_BN && v % multiple == 0) return v;
    }
    const int tiles_a = (M + PAIR_ROWS - 1) / PAIR_ROWS;
    long long best_cost = -1;
    int best = PERS_MAX_BN;
    for (int bn = PERS_MAX_BN; bn >= 64; bn -= 32) {
        if (bn % multiple) continue;
        const long long tiles = (long long)tiles_a * ((N + bn - 1) / bn);
        const long long rounds = (tiles + pairs - 1) / pairs;
        const long long cost = rounds * (bn + 100);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

// 0: pairs not tried yet; > 0: clusters of two that fit on the device at once; < 0: unusable
template <int EPI, typename OutT>
int launch_pair(const void* x, const void* w, void* out, const void* bias, int bias_dtype,
                int RA, int RB, int K, int ldx, long long ldc, int* err, cudaStream_t stream) {
    constexpr int SMEM = PAIR_STAGES * (A_STAGE_BYTES + (PERS_MAX_BN / 2) * TILE_K * 2) + 256 + 1024;
    auto kern = gemm_tc_pair_kernel<EPI, OutT>;
    static int max_pairs = 0;
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2);
            cfg.blockDim = dim3(GEMM_THREADS);
            cfg.dynamicSmemBytes = SMEM;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
            max_pairs = (e == cudaSuccess && n > 0) ? n : -1;
        } else {
            max_pairs = -1;
        }
        if (max_pairs < 0) cudaGetLastError();
    }
    if (max_pairs < 0) return -1;
    const int bn = pick_pair_tile_n(RA, RB, max_pairs, 32);
    CUtensorMap ma, mb;
    if (get_map(x, RA, K, ldx, TILE_A, &ma)) return 1;
    if (get_map(w, RB, K, K, bn / 2, &mb)) return 1;
    const int n_tiles = ((RA + PAIR_ROWS - 1) / PAIR_ROWS) * ((RB + bn - 1) / bn);
    const int pairs = n_tiles < max_pairs ? n_tiles : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = infero_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, ma, mb, (OutT*)out, bias, bias_dtype, RA, RB, K, ldc, bn, err);
    return infero_check_launch("gemm_tc_pair");
}

// Pairs of CTAs are used unless INFERO_GEMM_PAIR=0 (or infero_gemm_set_pairs(0)), for token counts
// that fill tiles of 256 rows nearly as well as tiles of 128.
std::atomic<int> g_pairs{-1};
bool pairs_wanted(int M) {
    int v = g_pairs.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("INFERO_GEMM_PAIR");
        v = (e && e[0] == '0') ? 0 : 1;
        g_pairs.store(v, std::memory_order_relaxed);
    }
    if (!v) return false;
    const long long pad256 = (long long)((M + PAIR_ROWS - 1) / PAIR_ROWS) * PAIR_ROWS;
    const long long pad128 = (long long)((M + TILE_A - 1) / TILE_A) * TILE_A;
    return pad256 * 100 <= pad128 * 107;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" {

void infero_gemm_set_pairs(int on) { g_pairs.store(on ? 1 : 0, std::memory_order_relaxed); }

// Can the tensor-core kernel take this product?  (bf16 operands are the caller's business.)
int infero_gemm_tc_supported(const void* x, const void* w, int M, int N, int K, int ldx) {
    return M > 0 && N > 0 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldx >= K && aligned16(x) && aligned16(w);
}

// How the few-token path would cut the work: the number of splits of K and the bytes of
// 32-bit partials it needs (0 when one split writes the result directly).
int infero_gemm_tc_plan(int M, int N, int K, int sm_count, int* splits, int* ktiles_per_split,
                        long long* workspace_bytes) {
    const int total_kt = (K + TILE_K - 1) / TILE_K;
    int s = 1, per = total_kt;
    if (M <= 256) {
        const int tiles = (N + TILE_A - 1) / TILE_A;
        const int target = 2 * (sm_count > 0 ? sm_count : 148);
        s = target / tiles;
        if (s < 1) s = 1;
        if (s > 16) s = 16;
        if (cluster_sum() && s > MAX_CLUSTER) s = MAX_CLUSTER;     // the splits of a tile form one cluster
        const int min_kt = 4;                              // a split shorter than this is all start-up
        if (s > total_kt / min_kt) s = total_kt / min_kt > 0 ? total_kt / min_kt : 1;
        per = (total_kt + s - 1) / s;
        s = (total_kt + per - 1) / per;
    }
    *splits = s;
    *ktiles_per_split = per;
    *workspace_bytes = s > 1 ? (long long)s * M * N * 4 : 0;
    return 0;
}

// 32-bit partial products of the few-token path: partial[s, t, n] for s < splits.
// x [M, K] (row stride ldx) and w [N, K] are bf16; M <= 256.
int infero_gemm_tc_partials(const void* x, const void* w, float* partial, int M, int N, int K, int ldx,
                            int splits, int ktiles_per_split, cudaStream_t stream) {
    INFERO_REQUIRE(infero_gemm_tc_supported(x, w, M, N, K, ldx), "gemm_tc: shape M=%d N=%d K=%d ldx=%d not supported", M, N, K, ldx);
    INFERO_REQUIRE(M <= 256, "gemm_tc_partials: M=%d above 256", M);
    INFERO_REQUIRE(splits >= 1 && ktiles_per_split >= 1 && (long long)(splits - 1) * ktiles_per_split * TILE_K < K,
                   "gemm_tc_partials: %d splits of %d k-tiles do not fit K=%d", splits, ktiles_per_split, K);
    int* err;
    if (err_flag_ptr(&err)) return 1;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mw, mx;
    if (get_map(w, N, K, K, TILE_A, &mw)) return 1;
    if (get_map(x, M, K, ldx, bn, &mx)) return 1;
#define GO(BN_, ST_) return launch<BN_, ST_, EPI_PARTIAL, float>(mw, mx, partial, nullptr, 0, N, M, K, ktiles_per_split, splits, 0, 1, err, stream)
    switch (bn) {
        case 16: GO(16, 6);
        case 32: GO(32, 5);
        case 64: GO(64, 4);
        case 128: GO(128, 3);
        default: GO(256, 4);
    }
#undef GO
}

// The same product added up over the splits inside the kernel (a cluster per tile, at most 8 splits):
// out[t, n], 32-bit, no bias.
int infero_gemm_tc_summed(const void* x, const void* w, float* out, int M, int N, int K, int ldx, int splits,
                          int ktiles_per_split, cudaStream_t stream) {
    INFERO_REQUIRE(infero_gemm_tc_supported(x, w, M, N, K, ldx), "gemm_tc: shape M=%d N=%d K=%d ldx=%d not supported", M, N, K, ldx);
    INFERO_REQUIRE(M <= 256, "gemm_tc_summed: M=%d above 256", M);
    INFERO_REQUIRE(splits >= 2 && splits <= MAX_CLUSTER && ktiles_per_split >= 1 &&
                       (long long)(splits - 1) * ktiles_per_split * TILE_K < K,
                   "gemm_tc_summed: %d splits of %d k-tiles do not fit K=%d (2..%d splits)", splits, ktiles_per_split, K, MAX_CLUSTER);
    int* err;
    if (err_flag_ptr(&err)) return 1;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mw, mx;
    if (get_map(w, N, K, K, TILE_A, &mw)) return 1;
    if (get_map(x, M, K, ldx, bn, &mx)) return 1;
#define GO(BN_, ST_) return launch_cluster<BN_, ST_>(mw, mx, out, N, M, K, ktiles_per_split, splits, err, stream)
    switch (bn) {
        case 16: GO(16, 6);
        case 32: GO(32, 5);
        case 64: GO(64, 4);
        case 128: GO(128, 3);
        default: GO(256, 4);
    }
#undef GO
}

// How the kernels below cut K: as infero_gemm_tc_plan, but the splits of a tile are one cluster, so there
// are at most 8, and no more than leave about a fifth of the multiprocessors' block slots free: a cluster
// starts only when all of its blocks find room in one group of multiprocessors at once, and a grid that
// fills the slots to the brim starts late, behind the blocks of the kernel in front as they drain
// (measured at hidden 5120, 40 tiles: 7 splits = 280 blocks 6.58 ms per step, 6 splits = 240 blocks
// 6.04 ms; at hidden 3584, 28 tiles, 8 splits = 224 blocks are the best).
int infero_gemm_tc_plan_cluster(int M, int N, int K, int sm_count, int* splits, int* ktiles_per_split) {
    long long ws = 0;
    infero_gemm_tc_plan(M, N, K, sm_count, splits, ktiles_per_split, &ws);
    const int total_kt = (K + TILE_K - 1) / TILE_K;
    const int tiles = (N + TILE_A - 1) / TILE_A;
    const int slots = 2 * (sm_count > 0 ? sm_count : 148);
    int cap = (int)(0.82 * slots) / tiles;
    if (cap > MAX_CLUSTER) cap = MAX_CLUSTER;
    if (cap < 1) cap = 1;
    if (const char* e = getenv("INFERO_CLUSTER_SPLITS")) {        // tuning knob
        const int want = atoi(e);
        if (want >= 1 && want <= MAX_CLUSTER) cap = want;
    }
    if (*splits > cap) {
        *ktiles_per_split = (total_kt + cap - 1) / cap;
        *splits = (total_kt + *ktiles_per_split - 1) / *ktiles_per_split;
    }
    return 0;
}

// A product whose result is a residual update, with what the RMSNorm behind it needs (see GemmFuse):
//   resid[t, n] += sum_k x[t, k] w[n, k] (+ bias[n]);  h[t, n] = bf16(resid[t, n] * norm_w[n]);
//   sumsq[tile * 256 + t] = sum over the 128 features n of tile of resid[t, n]^2.
// x [M, K] bf16 (row stride ldx), w [N, K] bf16, resid [M, N] float and h [M, N] bf16 contiguous; M <= 256;
// 1..8 splits of K as infero_gemm_tc_plan_cluster says; sumsq holds ceil(N / 128) * 256 floats.
int infero_gemm_tc_residual_norm(const void* x, const void* w, int M, int N, int K, int ldx, int splits,
                                 int ktiles_per_split, float* resid, const void* bias, int bias_dtype,
                                 const void* norm_w, int norm_w_dtype, void* h, float* sumsq, cudaStream_t stream) {
    INFERO_REQUIRE(infero_gemm_tc_supported(x, w, M, N, K, ldx), "gemm_tc: shape M=%d N=%d K=%d ldx=%d not supported", M, N, K, ldx);
    INFERO_REQUIRE(M <= 256, "gemm_tc_residual_norm: M=%d above 256", M);
    INFERO_REQUIRE(splits >= 1 && splits <= MAX_CLUSTER && ktiles_per_split >= 1 &&
                       (long long)(splits - 1) * ktiles_per_split * TILE_K < K,
                   "gemm_tc_residual_norm: %d splits of %d k-tiles do not fit K=%d (1..%d splits)", splits, ktiles_per_split, K, MAX_CLUSTER);
    INFERO_REQUIRE(resid && norm_w && h && sumsq, "gemm_tc_residual_norm: a null output");
    int* err;
    if (err_flag_ptr(&err)) return 1;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mw, mx;
    if (get_map(w, N, K, K, TILE_A, &mw)) return 1;
    if (get_map(x, M, K, ldx, bn, &mx)) return 1;
    GemmFuse f = {};
    f.x = resid, f.bias = bias, f.bias_dtype = bias_dtype, f.norm_w = norm_w, f.norm_w_dtype = norm_w_dtype;
    f.h = (bf16*)h, f.sumsq_out = sumsq;
#define GO(BN_, ST_) return launch_cluster<BN_, ST_>(mw, mx, nullptr, N, M, K, ktiles_per_split, splits, err, stream, f)
    switch (bn) {
        case 16: GO(16, 6);
        case 32: GO(32, 5);
        case 64: GO(64, 4);
        case 128: GO(128, 3);
        default: GO(256, 4);
    }
#undef GO
}

int infero_gemm_cluster_enabled() { return cluster_sum() ? 1 : 0; }
void infero_gemm_set_cluster(int on) { g_cluster.store(on ? 1 : 0, std::memory_order_relaxed); }

int infero_reduce_partials(const float* partial, int splits, const void* bias, int bias_dtype, void* out,
                           int out_dtype, int M, int N, int ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    const size_t total = (size_t)M * N;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
    if (out_dtype == INFERO_F32)
        launch_pdl(reduce_partials_kernel<float>, dim3(blocks), dim3(256), 0, stream, partial, splits, bias, bias_dtype, (float*)out, M, N, ldc);
    else
        launch_pdl(reduce_partials_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, partial, splits, bias, bias_dtype, (bf16*)out, M, N, ldc);
    return infero_check_launch("reduce_partials");
}

// out[M, N] (bf16 or float, row stride ldc) = x[M, K] * w[N, K]^T (+ bias), bf16 operands.
// workspace: what infero_gemm_tc_plan asked for (may be null when it asked for nothing).
// tile_n: 0 = default, else 128 or 256 for the many-token path.
int infero_gemm_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                   int M, int N, int K, int ldx, int ldc, void* workspace, long long workspace_bytes,
                   int sm_count, int tile_n, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    INFERO_REQUIRE(infero_gemm_tc_supported(x, w, M, N, K, ldx), "gemm_tc: shape M=%d N=%d K=%d ldx=%d not supported", M, N, K, ldx);
    INFERO_REQUIRE(ldc >= N, "gemm_tc: ldc=%d below N=%d", ldc, N);
    int* err;
    if (err_flag_ptr(&err)) return 1;
    if (M <= 256) {
        int splits, per;
        long long need;
        infero_gemm_tc_plan(M, N, K, sm_count, &splits, &per, &need);
        if (splits > 1) {
            INFERO_REQUIRE(workspace && workspace_bytes >= need, "gemm_tc: workspace of %lld bytes needed, %lld given", need, workspace_bytes);
            if (cluster_sum() && splits <= MAX_CLUSTER) {
                if (infero_gemm_tc_summed(x, w, (float*)workspace, M, N, K, ldx, splits, per, stream)) return 1;
                return infero_reduce_partials((const float*)workspace, 1, bias, bias_dtype, out, out_dtype, M, N, ldc, stream);
            }
            if (infero_gemm_tc_partials(x, w, (float*)workspace, M, N, K, ldx, splits, per, stream)) return 1;
            return infero_reduce_partials((const float*)workspace, splits, bias, bias_dtype, out, out_dtype, M, N, ldc, stream);
        }
        const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        CUtensorMap mw, mx;
        if (get_map(w, N, K, K, TILE_A, &mw)) return 1;
        if (get_map(x, M, K, ldx, bn, &mx)) return 1;
#define GO(BN_, ST_)                                                                                              \
    do {                                                                                                          \
        if (out_dtype == INFERO_F32)                                                                              \
            return launch<BN_, ST_, EPI_COL, float>(mw, mx, out, bias, bias_dtype, N, M, K, per, 1, ldc, 1, err, stream); \
        return launch<BN_, ST_, EPI_COL, bf16>(mw, mx, out, bias, bias_dtype, N, M, K, per, 1, ldc, 1, err, stream);      \
    } while (0)
        switch (bn) {
            case 16: GO(16, 6);
            case 32: GO(32, 5);
            case 64: GO(64, 4);
            case 128: GO(128, 3);
            default: GO(256, 4);
        }
#undef GO
    }
    const int total_kt = (K + TILE_K - 1) / TILE_K;
    const int bn = tile_n == 128 ? 128 : 256;
    CUtensorMap mx, mw;
    if (get_map(x, M, K, ldx, TILE_A, &mx)) return 1;
    if (get_map(w, N, K, K, bn, &mw)) return 1;
    if (bn == 128) {
        if (out_dtype == INFERO_F32)
            return launch<128, 3, EPI_ROW, float>(mx, mw, out, bias, bias_dtype, M, N, K, total_kt, 1, ldc, 0, err, stream);
        return launch<128, 3, EPI_ROW, bf16>(mx, mw, out, bias, bias_dtype, M, N, K, total_kt, 1, ldc, 0, err, stream);
    }
    if (tile_n == 256) {                                   // the one-tile-per-CTA kernel, kept for comparison
        if (out_dtype == INFERO_F32)
            return launch<256, 4, EPI_ROW, float>(mx, mw, out, bias, bias_dtype, M, N, K, total_kt, 1, ldc, 0, err, stream);
        return launch<256, 4, EPI_ROW, bf16>(mx, mw, out, bias, bias_dtype, M, N, K, total_kt, 1, ldc, 0, err, stream);
    }
    if (pairs_wanted(M)) {
        const int r = out_dtype == INFERO_F32
                          ? launch_pair<EPI_ROW, float>(x, w, out, bias, bias_dtype, M, N, K, ldx, ldc, err, stream)
                          : launch_pair<EPI_ROW, bf16>(x, w, out, bias, bias_dtype, M, N, K, ldx, ldc, err, stream);
        if (r >= 0) return r;
    }
    if (out_dtype == INFERO_F32)
        return launch_persistent<EPI_ROW, float>(x, w, out, bias, bias_dtype, M, N, K, ldx, ldc, sm_count, err, stream);
    return launch_persistent<EPI_ROW, bf16>(x, w, out, bias, bias_dtype, M, N, K, ldx, ldc, sm_count, err, stream);
}

// out[M, N/2] (bf16, row stride ldc) = silu(g) * u with [g_0 u_0 g_1 u_1 ...] = x[M, K] * w[N, K]^T:
// w's rows alternate gate and up.  With few rows this needs the one-split plan (the activation
// is not linear, so partial sums cannot be combined afterwards): returns 2 when the plan has
// more than one split, and nothing is launched.
int infero_gemm_tc_swiglu(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldc,
                          int sm_count, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    INFERO_REQUIRE(infero_gemm_tc_supported(x, w, M, N, K, ldx), "gemm_tc_swiglu: shape M=%d N=%d K=%d ldx=%d not supported", M, N, K, ldx);
    INFERO_REQUIRE(N % 2 == 0 && ldc >= N / 2, "gemm_tc_swiglu: N=%d must be even and ldc=%d at least N/2", N, ldc);
    int* err;
    if (err_flag_ptr(&err)) return 1;
    if (M <= 256) {
        int splits, per;
        long long need;
        infero_gemm_tc_plan(M, N, K, sm_count, &splits, &per, &need);
        if (splits > 1) return 2;
        const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        CUtensorMap mw, mx;
        if (get_map(w, N, K, K, TILE_A, &mw)) return 1;
        if (get_map(x, M, K, ldx, bn, &mx)) return 1;
#define GO(BN_, ST_) return launch<BN_, ST_, EPI_COL_SWIGLU, bf16>(mw, mx, out, nullptr, 0, N, M, K, per, 1, ldc, 1, err, stream)
        switch (bn) {
            case 16: GO(16, 6);
            case 32: GO(32, 5);
            case 64: GO(64, 4);
            case 128: GO(128, 3);
            default: GO(256, 4);
        }
#undef GO
    }
    CUtensorMap mx, mw;
    if (get_map(x, M, K, ldx, TILE_A, &mx)) return 1;
    if (get_map(w, N, K, K, 256, &mw)) return 1;
    if (pairs_wanted(M)) {
        const int r = launch_pair<EPI_ROW_SWIGLU, bf16>(x, w, out, nullptr, 0, M, N, K, ldx, ldc, err, stream);
        if (r >= 0) return r;
    }
    return launch_persistent<EPI_ROW_SWIGLU, bf16>(x, w, out, nullptr, 0, M, N, K, ldx, ldc, sm_count, err, stream);
}

// The few-token, one-split case of infero_gemm_tc_swiglu on an input that still lacks its norm's scalar:
// token t's products are multiplied by rsqrt(sum_{tile < n_tiles} sumsq[tile * 256 + t] * inv_d + eps) before
// the activation.  Returns 2, with nothing launched, when the plan has more than one split or M > 256.
int infero_gemm_tc_swiglu_scaled(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldc,
                                 const float* sumsq, int n_tiles, float inv_d, float eps, int sm_count,
                                 cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    INFERO_REQUIRE(infero_gemm_tc_supported(x, w, M, N, K, ldx), "gemm_tc_swiglu: shape M=%d N=%d K=%d ldx=%d not supported", M, N, K, ldx);
    INFERO_REQUIRE(N % 2 == 0 && ldc >= N / 2, "gemm_tc_swiglu: N=%d must be even and ldc=%d at least N/2", N, ldc);
    INFERO_REQUIRE(sumsq && n_tiles >= 1, "gemm_tc_swiglu_scaled: no sums of squares");
    if (M > 256) return 2;
    int splits, per;
    long long need;
    infero_gemm_tc_plan(M, N, K, sm_count, &splits, &per, &need);
    if (splits > 1) return 2;
    int* err;
    if (err_flag_ptr(&err)) return 1;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mw, mx;
    if (get_map(w, N, K, K, TILE_A, &mw)) return 1;
    if (get_map(x, M, K, ldx, bn, &mx)) return 1;
    GemmFuse f = {};
    f.sumsq_in = sumsq, f.in_tiles = n_tiles, f.inv_d = inv_d, f.eps = eps;
#define GO(BN_, ST_) return launch<BN_, ST_, EPI_COL_SWIGLU, bf16>(mw, mx, out, nullptr, 0, N, M, K, per, 1, ldc, 1, err, stream, f)
    switch (bn) {
        case 16: GO(16, 6);
        case 32: GO(32, 5);
        case 64: GO(64, 4);
        case 128: GO(128, 3);
        default: GO(256, 4);
    }
#undef GO
}

// Reads (and clears) the flag a tensor-core kernel raises when one of its waits ran out.
// Synchronises the device.  0 = no error.
int infero_tc_error_flag() {
    int* err;
    if (err_flag_ptr(&err)) return -1;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, err, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        infero_set_error("tc_error_flag: %s", cudaGetErrorString(e));
        return -1;
    }
    if (v) cudaMemset(err, 0, sizeof(int));
    return v;
}

// Writes the flag from the host (0 clears it).  For tests of what the host does when a wait has run
// out: no kernel has to miss a wait for that.  Synchronises the device.
int infero_tc_set_error_flag(int value) {
    int* err;
    if (err_flag_ptr(&err)) return -1;
    cudaError_t e = cudaMemcpy(err, &value, sizeof(int), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        infero_set_error("tc_set_error_flag: %s", cudaGetErrorString(e));
        return -1;
    }
    return 0;
}

}  // extern "C"

INFERO_TL_UNIT(gemm_tc)
