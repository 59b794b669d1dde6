// AdamW over many tensors in one launch per batch of descriptors.
//
// Work is cut into fixed-size chunks; a CTA finds the tensor its chunk belongs to by a
// binary search over the per-tensor chunk prefix carried in the kernel parameters, then
// streams p, g, m, v with 128-bit accesses: 28 B/parameter, plus 2 B when the bf16 copy of
// the updated parameter is written in the same pass and 4 B when the gradient is cleared.
//
// Math: src/nn2/optim.rs:49-71 (decoupled decay on the raw parameter, then the Adam step;
// bias corrections 1-beta^t computed by the caller). Kernels replaced:
// src/gpu/cuda/common.cu:312-361.
#include "common.cuh"

namespace xl {

static constexpr int kMaxDescs = 48;
static constexpr int kChunk = 4096;  // elements per CTA: 256 threads x 4 float4

struct AdamBatch {
    float* p[kMaxDescs];
    float* g[kMaxDescs];
    float* m[kMaxDescs];
    float* v[kMaxDescs];
    bf16* pb[kMaxDescs];
    unsigned long long len[kMaxDescs];
    float wd[kMaxDescs];
    unsigned start[kMaxDescs + 1];  // chunk prefix
    int n;
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, float lr, float b1, float b2,
                                         float eps, float bc1, float bc2, float wd) {
    m = b1 * m + (1.f - b1) * g;
    v = b2 * v + (1.f - b2) * g * g;
    float mh = m / bc1, vh = v / bc2;
    p -= lr * wd * p;
    p -= lr * mh / (sqrtf(vh) + eps);
}

__global__ void __launch_bounds__(256) adamw_multi_kernel(const __grid_constant__ AdamBatch bt, float lr, float b1,
                                                          float b2, float eps, float bc1, float bc2, int zero_grad) {
    // owner of this chunk
    int lo = 0, hi = bt.n;
    const unsigned cid = blockIdx.x;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (bt.start[mid] <= cid) lo = mid; else hi = mid;
    }
    const int ti = lo;
    const unsigned long long base = (unsigned long long)(cid - bt.start[ti]) * kChunk;
    const unsigned long long len = bt.len[ti];
    float* __restrict__ p = bt.p[ti];
    float* __restrict__ g = bt.g[ti];
    float* __restrict__ m = bt.m[ti];
    float* __restrict__ v = bt.v[ti];
    bf16* __restrict__ pb = bt.pb[ti];
    const float wd = bt.wd[ti];
    const bool al = ((((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0) && (((uintptr_t)pb & 7) == 0);
    if (al && base + kChunk <= len) {
        float4 P[4], G[4], M[4], V[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unsigned long long e = base + (unsigned long long)(i * 256 + threadIdx.x) * 4;
            P[i] = *reinterpret_cast<const float4*>(p + e);
            G[i] = *reinterpret_cast<const float4*>(g + e);
            M[i] = *reinterpret_cast<const float4*>(m + e);
            V[i] = *reinterpret_cast<const float4*>(v + e);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unsigned long long e = base + (unsigned long long)(i * 256 + threadIdx.x) * 4;
            adam_one(P[i].x, G[i].x, M[i].x, V[i].x, lr, b1, b2, eps, bc1, bc2, wd);
            adam_one(P[i].y, G[i].y, M[i].y, V[i].y, lr, b1, b2, eps, bc1, bc2, wd);
            adam_one(P[i].z, G[i].z, M[i].z, V[i].z, lr, b1, b2, eps, bc1, bc2, wd);
            adam_one(P[i].w, G[i].w, M[i].w, V[i].w, lr, b1, b2, eps, bc1, bc2, wd);
            *reinterpret_cast<float4*>(p + e) = P[i];
            *reinterpret_cast<float4*>(m + e) = M[i];
            *reinterpret_cast<float4*>(v + e) = V[i];
            if (zero_grad) *reinterpret_cast<float4*>(g + e) = make_float4(0.f, 0.f, 0.f, 0.f);
            if (pb) {
                __nv_bfloat162 lo2 = __floats2bfloat162_rn(P[i].x, P[i].y);
                __nv_bfloat162 hi2 = __floats2bfloat162_rn(P[i].z, P[i].w);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo2);
                pk.y = *reinterpret_cast<unsigned*>(&hi2);
                *reinterpret_cast<uint2*>(pb + e) = pk;
            }
        }
    } else {
        unsigned long long end = base + kChunk < len ? base + kChunk : len;
        for (unsigned long long e = base + threadIdx.x; e < end; e += 256) {
            float pp = p[e], mm = m[e], vv = v[e];
            adam_one(pp, g[e], mm, vv, lr, b1, b2, eps, bc1, bc2, wd);
            p[e] = pp; m[e] = mm; v[e] = vv;
            if (zero_grad) g[e] = 0.f;
            if (pb) pb[e] = __float2bfloat16_rn(pp);
        }
    }
}

}  // namespace xl

using namespace xl;

extern "C" int xlstm_adamw_multi(void* stream, const xlstm_adamw_desc* descs, int n, float lr, float beta1,
                                 float beta2, float eps, float bc1, float bc2, int zero_grad) {
    XL_CHECK_ARG(n >= 0 && (n == 0 || descs), "adamw_multi: null descriptor array");
    XL_CHECK_ARG(bc1 > 0.f && bc2 > 0.f, "adamw_multi: bias corrections must be positive (step count t >= 1)");
    cudaStream_t st = (cudaStream_t)stream;
    int i = 0;
    while (i < n) {
        AdamBatch bt;
        bt.n = 0;
        unsigned chunks = 0;
        while (i < n && bt.n < kMaxDescs) {
            const xlstm_adamw_desc& d = descs[i++];
            if (d.len == 0) continue;
            XL_CHECK_ARG(d.p && d.g && d.m && d.v, "adamw_multi: tensor %d has a null pointer", i - 1);
            unsigned long long c = (d.len + kChunk - 1) / kChunk;
            if ((unsigned long long)chunks + c > 0x7fffffffull) { --i; break; }
            int k = bt.n++;
            bt.p[k] = d.p; bt.g[k] = d.g; bt.m[k] = d.m; bt.v[k] = d.v; bt.pb[k] = (bf16*)d.p_bf16;
            bt.len[k] = d.len; bt.wd[k] = d.wd; bt.start[k] = chunks;
            chunks += (unsigned)c;
        }
        if (bt.n == 0) {
            if (i < n && chunks == 0) { set_error("adamw_multi: tensor %d is too large for one launch", i); return XLSTM_ERR_ARG; }
            continue;
        }
        bt.start[bt.n] = chunks;
        for (int k = bt.n + 1; k <= kMaxDescs; ++k) bt.start[k] = chunks;
        adamw_multi_kernel<<<chunks, 256, 0, st>>>(bt, lr, beta1, beta2, eps, bc1, bc2, zero_grad);
        XL_LAUNCH_OK("adamw_multi_kernel");
    }
    return XLSTM_OK;
}
