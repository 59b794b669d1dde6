// Shared device/host helpers for the xlstm_b200 kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/xlstm_b200.h"

namespace xl {

typedef __nv_bfloat16 bf16;

// ---- error plumbing --------------------------------------------------------------------
void set_error(const char* fmt, ...);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

#define XL_CHECK_ARG(cond, ...)                 \
    do {                                        \
        if (!(cond)) {                          \
            xl::set_error(__VA_ARGS__);         \
            return XLSTM_ERR_ARG;               \
        }                                       \
    } while (0)

#define XL_CUDA(expr)                                                              \
    do {                                                                           \
        cudaError_t e__ = (expr);                                                  \
        if (e__ != cudaSuccess) {                                                  \
            xl::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));        \
            return XLSTM_ERR_CUDA;                                                 \
        }                                                                          \
    } while (0)

// Checks the launch that was just issued (configuration errors only; no sync).
#define XL_LAUNCH_OK(name)                                                         \
    do {                                                                           \
        cudaError_t e__ = cudaGetLastError();                                      \
        if (e__ != cudaSuccess) {                                                  \
            xl::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__)); \
            return XLSTM_ERR_CUDA;                                                 \
        }                                                                          \
        xl::count_launch();                                                        \
    } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- typed loads / stores (storage type -> float) -----------------------------------------
__device__ __forceinline__ float ldf(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const bf16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// The reference's branch-stable forms (src/gpu/cuda/prelude.cu; src/nn2/mlstm.rs:31-47).
__device__ __forceinline__ float stable_sigmoid(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    float e = expf(x);
    return e / (1.f + e);
}
__device__ __forceinline__ float log_sigmoid(float x) {
    if (x >= 0.f) return -log1pf(expf(-x));
    return x - log1pf(expf(x));
}

// acc[c] += sum over the parts of partial[part][c], in a fixed order (no float atomics): eight lanes per column take the
// parts lane, lane + 8, ... in ascending order and the eight sums are combined pairwise. One CTA per 32 columns.
static __global__ void __launch_bounds__(256) merge_parts8(const float* __restrict__ partial, float* __restrict__ acc,
                                                           int nparts, int cols) {
    __shared__ float sh[8][32];
    const int cl = threadIdx.x & 31, pl = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cl;
    float s = 0.f;
    if (c < cols)
        for (int p = pl; p < nparts; p += 8) s += partial[(size_t)p * cols + c];
    sh[pl][cl] = s;
    __syncthreads();
    if (pl == 0 && c < cols)
        acc[c] += ((sh[0][cl] + sh[1][cl]) + (sh[2][cl] + sh[3][cl])) + ((sh[4][cl] + sh[5][cl]) + (sh[6][cl] + sh[7][cl]));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed combination order (warp tree, then warp 0 over the partials).
// `red` is shared scratch of >= 32 floats. All threads receive the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

int sm_count();

}  // namespace xl
