// Host-side state shared by the kernels that use TMA and tcgen05: tensor maps (TMA
// descriptors) for bf16 matrices, made once per (pointer, shape, box) and kept, and the
// device flag that reports a wait that ran out.
#include "tc_common.cuh"
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int TILE_K = 64;

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::mutex g_mutex;

struct MapKey {
    const void* ptr;
    int rows, cols, ld, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld;
        h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

int load_encoder() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
        infero_set_error("tensor map: the driver does not offer cuTensorMapEncodeTiled (%s)", cudaGetErrorString(e));
        return 1;
    }
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    return 0;
}

}  // namespace

// A [rows, cols] bf16 matrix with row stride ld (elements), tiles of box_rows x 64 elements,
// 128-byte swizzle, zero fill outside the matrix.  Returns 0, or 1 with the error recorded.
int infero_tensor_map_bf16(const void* ptr, int rows, int cols, int ld, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (load_encoder()) return 1;
    MapKey key{ptr, rows, cols, ld, box_rows};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return 0;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        infero_set_error("tensor map: cuTensorMapEncodeTiled failed (%d) for a [%d, %d] matrix, row stride %d, box %d",
                         (int)r, rows, cols, ld, box_rows);
        return 1;
    }
    if (g_maps.size() > 8192) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return 0;
}

namespace {
int* g_err_flag = nullptr;
}  // namespace

// The flag a tensor-core kernel raises when one of its bounded waits ran out (device memory,
// allocated on first use; do that before any stream capture).
int infero_tc_err_flag(int** out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_err_flag) {
        cudaError_t e = cudaMalloc(&g_err_flag, sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(g_err_flag, 0, sizeof(int));
        if (e != cudaSuccess) {
            g_err_flag = nullptr;
            infero_set_error("tc: cannot allocate the error flag: %s", cudaGetErrorString(e));
            return 1;
        }
    }
    *out = g_err_flag;
    return 0;
}

