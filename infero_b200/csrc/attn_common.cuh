// Pieces shared by the bf16 attention kernels that run on the warp-level tensor cores
// (mma.sync m16n8k16): fragment loads, shared-memory tile layouts, and the 16-key step of the
// online softmax.
#pragma once
#include "common.cuh"
#include <math_constants.h>

namespace attn {

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
template <int D>
struct PaddedRows {
    __device__ static __forceinline__ int chunk(int row, int c) { return swz<D>(row, c); }
};
// What a tiled TMA load with 128-byte swizzle leaves in shared memory: the tile is cut into
// column blocks of 64 elements (128 bytes per row); inside a block, row r holds its eight
// 16-byte chunks at positions c ^ (r & 7).  ROWS = rows of one block (a multiple of 8); the
// tile base must be aligned to 1024 bytes.
template <int D, int ROWS>
struct Swizzled128 {
    __device__ static __forceinline__ int chunk(int row, int c) {
        return (c >> 3) * (ROWS * 8) + row * 8 + ((c & 7) ^ (row & 7));
    }
};

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
template <int D, typename Layout = PaddedRows<D>>
__device__ __forceinline__ void slice16(const uint32_t (*qf)[4], const bf16* k_tile, const bf16* v_tile, int row0,
                                        int key_base, int lo0, int hi0, int lo1, int hi1, float scale_log2,
                                        float* m, float* l, float (*o)[4], int lane) {
    const int c = lane & 3;
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
            ldmatrix_x4(b, smem_addr(k_tile + (size_t)Layout::chunk(krow, ks * 2 + (mi & 1)) * 8));
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
            ldmatrix_x4_trans(b, smem_addr(v_tile + (size_t)Layout::chunk(vrow, np * 2 + (mi >> 1)) * 8));
            float* o0 = o[np * 2];
            float* o1 = o[np * 2 + 1];
            o0[0] *= corr0; o0[1] *= corr0; o0[2] *= corr1; o0[3] *= corr1;
            o1[0] *= corr0; o1[1] *= corr0; o1[2] *= corr1; o1[3] *= corr1;
            mma16816(o0, pf, b[0], b[1]);
            mma16816(o1, pf, b[2], b[3]);
        }
    }
}

}  // namespace attn
