// Host-side helpers shared by the tensor-core mLSTM kernels (mlstm_tc_fw.cu, mlstm_tc_bw.cu): TMA
// tensor-map encoding, the shape test, the layout of the chunk-state record, and the device status
// word that bounded waits report through.
#include <cuda.h>

#include "common.cuh"
#include "mlstm.cuh"

namespace xl {

__device__ int g_tc_status = 0;  // 0 ok, else the code of the first wait that ran out of budget

static constexpr int D = 128;  // dqk = dhv
static constexpr int L = 64;   // chunk length

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved at run time so the library does not link libcuda.
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// [B][T][W] bf16 row-major viewed as a 3-D tensor (W inner); box = {64 cols, 64 rows, 1}, 128-byte swizzle.
// Rows past T are out of bounds for the map, so a ragged last chunk is zero-filled.
bool tc_make_map3(CUtensorMap* m, const void* base, int B, int T, int W) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)W, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t strides[2] = {(cuuint64_t)W * 2, (cuuint64_t)W * 2 * (cuuint64_t)T};
    cuuint32_t box[3] = {64, 64, 1};
    cuuint32_t es[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows][W] bf16 row-major, box = {64 cols, box_rows}, 128-byte swizzle.
bool tc_make_map2(CUtensorMap* m, const void* base, uint64_t rows, int W, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)W, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)W * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* tc_status_ptr() {
    // resolved once per device: the lookup is a driver call, too slow for every launch
    static std::atomic<int*> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        void* q = nullptr;
        if (cudaGetSymbolAddress(&q, g_tc_status) != cudaSuccess) return nullptr;
        p = (int*)q;
        cached[dev].store(p, std::memory_order_release);
    }
    return p;
}

bool mlstm_tc_supported(int L_, int dqk, int dhv, int dtype) {
    return L_ == L && dqk >= D && dhv >= D && dqk % D == 0 && dhv % D == 0 && dqk <= 4 * D && dhv <= 4 * D && dtype == XLSTM_BF16;
}
int mlstm_tc_subheads(int dqk, int dhv) { return (dqk / D) * (dhv / D); }

size_t mlstm_tc_saved_C_bytes(int BH, int NC) { return align_up((size_t)BH * (NC + 1) * D * D * sizeof(bf16), 256); }
size_t mlstm_tc_saved_n_bytes(int BH, int NC) { return align_up((size_t)BH * (NC + 1) * D * sizeof(float), 256); }

int tc_status_read_and_clear(int* out) {
    int v = 0;
    XL_CUDA(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)));
    if (v != 0) {
        int z = 0;
        XL_CUDA(cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int)));
    }
    *out = v;
    return XLSTM_OK;
}

}  // namespace xl
