// Matrix products on the ordinary cores: out[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
//
//  * gemm_tiled: any shape, any mix of float / bf16 operands, 32-bit accumulation with one
//    fused multiply-add per k in ascending k.  The value of out[m,n] therefore does not
//    depend on M, on the tile it falls in or on its batch-mates: this is the product of the
//    true 32-bit path (no reduced-precision matrix mode anywhere).
//  * gemm_skinny: up to 4 rows of A (decode at tiny batch): one warp per pair of output
//    features streams the weight rows with 16-byte loads.  The reference switches to its
//    own mat-vec at the same point (crates/model/src/lib.rs:1574, cu/quant.cu:266-286).
//
// W is [N,K] row-major, as checkpoints store it (crates/model/src/weights.rs:2276-2277).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const void* __restrict__ bias,
                  int bias_dtype, TC* __restrict__ C, int M, int N, int K, int lda, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64x16 elements per operand, 4 per thread; k fastest so global reads are contiguous
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_any(bias, bias_dtype, gn);
            C[(size_t)gm * ldc + gn] = from_f32<TC>(v);
        }
    }
}

// bf16 weights and activations, M <= 4.  Each warp owns ROWS output features and walks K
// in steps of 256 (32 lanes x 8 elements).  K % 8 == 0 and 16-byte aligned rows required.
constexpr int SK_ROWS = 2;
template <int MT, typename TC>
__global__ void __launch_bounds__(256)
gemm_skinny_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, const void* __restrict__ bias,
                   int bias_dtype, TC* __restrict__ C, int M, int N, int K, int lda, int ldc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_base = (blockIdx.x * 8 + warp) * SK_ROWS;
    if (n_base >= N) return;
    float acc[SK_ROWS][MT];
#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

    for (int k = lane * 8; k < K; k += 256) {
        uint4 wv[SK_ROWS];
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) {
            const int n = n_base + r < N ? n_base + r : N - 1;
            wv[r] = __ldg(reinterpret_cast<const uint4*>(W + (size_t)n * K + k));
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const uint4 av = *reinterpret_cast<const uint4*>(A + (size_t)m * lda + k);
                const uint32_t au[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                for (int r = 0; r < SK_ROWS; ++r) {
                    const uint32_t wu[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        // a bf16 is the upper half of a float
                        const float a0 = __uint_as_float(au[q] << 16), a1 = __uint_as_float(au[q] & 0xffff0000u);
                        const float w0 = __uint_as_float(wu[q] << 16), w1 = __uint_as_float(wu[q] & 0xffff0000u);
                        acc[r][m] = fmaf(a0, w0, acc[r][m]);
                        acc[r][m] = fmaf(a1, w1, acc[r][m]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = warp_sum(acc[r][m]);
            const int n = n_base + r;
            if (lane == 0 && m < M && n < N) {
                if (bias) v += load_any(bias, bias_dtype, n);
                C[(size_t)m * ldc + n] = from_f32<TC>(v);
            }
        }
}

template <typename TA, typename TW, typename TC>
int launch_tiled(const void* A, const void* W, const void* bias, int bias_dtype, void* C, int M, int N,
                 int K, int lda, int ldc, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_tiled_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, bias, bias_dtype,
                                                             (TC*)C, M, N, K, lda, ldc);
    return infero_check_launch("gemm_tiled");
}

}  // namespace

extern "C" {

// Any of A, W, C may be float or bf16; accumulation is 32-bit in ascending k.
int infero_gemm_tiled(const void* A, int a_dtype, const void* W, int w_dtype, const void* bias,
                      int bias_dtype, void* C, int c_dtype, int M, int N, int K, int lda, int ldc,
                      cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    INFERO_REQUIRE(K > 0 && lda >= K && ldc >= N, "gemm_tiled: bad sizes M=%d N=%d K=%d lda=%d ldc=%d", M, N, K, lda, ldc);
    INFERO_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_tiled: M=%d too large", M);
    const int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (key) {
        case 0: return launch_tiled<float, float, float>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 1: return launch_tiled<float, float, bf16>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 2: return launch_tiled<float, bf16, float>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 3: return launch_tiled<float, bf16, bf16>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 4: return launch_tiled<bf16, float, float>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 5: return launch_tiled<bf16, float, bf16>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 6: return launch_tiled<bf16, bf16, float>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
        case 7: return launch_tiled<bf16, bf16, bf16>(A, W, bias, bias_dtype, C, M, N, K, lda, ldc, stream);
    }
    infero_set_error("gemm_tiled: unknown dtype tags %d %d %d", a_dtype, w_dtype, c_dtype);
    return 1;
}

// bf16 x bf16, 1 <= M <= 4, K % 8 == 0, A rows and W 16-byte aligned.
int infero_gemm_skinny(const void* A, const void* W, const void* bias, int bias_dtype, void* C,
                       int c_dtype, int M, int N, int K, int lda, int ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    INFERO_REQUIRE(M >= 1 && M <= 4, "gemm_skinny: M=%d outside 1..4", M);
    INFERO_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0, "gemm_skinny: K=%d and lda=%d must be multiples of 8", K, lda);
    INFERO_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_skinny: operands must be 16-byte aligned");
    const int blocks = (N + 8 * SK_ROWS - 1) / (8 * SK_ROWS);
#define LAUNCH(MT)                                                                                       \
    do {                                                                                                 \
        if (c_dtype == INFERO_F32)                                                                       \
            gemm_skinny_kernel<MT, float><<<blocks, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, \
                                                                      bias_dtype, (float*)C, M, N, K, lda, ldc); \
        else                                                                                             \
            gemm_skinny_kernel<MT, bf16><<<blocks, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, \
                                                                     bias_dtype, (bf16*)C, M, N, K, lda, ldc); \
    } while (0)
    if (M == 1) LAUNCH(1);
    else if (M == 2) LAUNCH(2);
    else LAUNCH(4);
#undef LAUNCH
    return infero_check_launch("gemm_skinny");
}

}  // extern "C"
