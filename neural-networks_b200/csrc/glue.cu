// Element-wise glue between the GEMMs and the recurrent cores, one HBM pass each, with the narrowing
// to bf16 folded into the producer (the reference's most frequent launches are stand-alone casts,
// src/gpu/cuda/bf16_cast.cu:22-60):
//   SwiGLU forward/backward        src/gpu/cuda/block.cu:6-29 (swiglu_forward / swiglu_backward)
//   output gate forward/backward   src/gpu/cuda/mlstm_ops.cu:147-153, 400-407 (ogate_fwd / ogate_bwd)
// All tensors are flat arrays of n elements; 128-bit accesses when n and the pointers allow, scalar
// otherwise. Outputs that feed a GEMM may be asked for in bf16 (RNE), everything else is fp32.
#include "common.cuh"

#include <cuda_bf16.h>

namespace xl {

typedef __nv_bfloat16 bf16;
static constexpr int kUnrollFw = 4;  // SwiGLU forward: eight pieces per thread measured slower (0.57 against 0.65 of the copy peak)
static constexpr int kUnroll = 4;  // 16-byte pieces per thread in the vector paths (loads in flight before first use)

__device__ __forceinline__ void st4(float* p, size_t i4, float4 v) { __stcs(reinterpret_cast<float4*>(p) + i4, v); }
__device__ __forceinline__ void st4(bf16* p, size_t i4, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    __stcs(reinterpret_cast<uint2*>(p) + i4, pk);
}
__device__ __forceinline__ void st1(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st1(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float4 ld4(const float* p, size_t i4) { return __ldcs(reinterpret_cast<const float4*>(p) + i4); }
__device__ __forceinline__ float4 ld4(const bf16* p, size_t i4) {
    const uint2 r = __ldcs(reinterpret_cast<const uint2*>(p) + i4);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float ld1(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ld1(const bf16* p, size_t i) { return __bfloat162float(p[i]); }

// The sigmoid of a kernel whose results leave as bf16: one ex2 and one rcp on the special-function unit instead of the
// library exponential and an IEEE division (relative error below 1e-6, a five-hundredth of the bf16 rounding that
// follows), branch-free. The fp32-output kernels keep the reference's branch-stable form (stable_sigmoid).
__device__ __forceinline__ float fast_sigmoid(float x) {
    const float e = __expf(-fabsf(x));
    const float r = __fdividef(1.f, 1.f + e);
    return x >= 0.f ? r : e * r;
}
template <typename OT>
__device__ __forceinline__ float sigmoid_for(float x) {
    if constexpr (sizeof(OT) == 2) return fast_sigmoid(x);
    else return stable_sigmoid(x);
}

template <typename OT>
__device__ __forceinline__ float silu_f(float x, float* sig) {
    const float s = sigmoid_for<OT>(x);
    *sig = s;
    return x * s;
}

// Optional per-column biases of the two projections, folded in here so that the GEMMs' outputs need no
// bias pass of their own: element i belongs to column i % cols.
__device__ __forceinline__ float4 bias4(const float* b, unsigned col) {
    if (!b) return make_float4(0.f, 0.f, 0.f, 0.f);
    return __ldg(reinterpret_cast<const float4*>(b + col));
}
// column of 16-byte piece j0 + 256*k given the column of piece j0 (one 64-bit remainder per thread, then 32-bit)
__device__ __forceinline__ unsigned col_of(unsigned col0, int k, int cols) { return (col0 + 1024u * (unsigned)k) % (unsigned)cols; }
__device__ __forceinline__ float bias1(const float* b, size_t i, int cols) { return b ? __ldg(b + i % (size_t)cols) : 0.f; }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// out = SiLU(gate + bg) * (value + bv)
template <typename IT, typename OT>
__global__ void __launch_bounds__(256) swiglu_fw_k(const IT* __restrict__ gate, const IT* __restrict__ value,
                                                   const float* __restrict__ bg, const float* __restrict__ bv, int cols,
                                                   OT* __restrict__ out, size_t n, int vec) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    float s;
    if (vec) {
        // kUnrollFw 16-byte pieces per thread, all loads issued before the first use
        const size_t n4 = n / 4, i0 = (size_t)blockIdx.x * (256 * kUnrollFw) + threadIdx.x;
        float4 g[kUnrollFw], v[kUnrollFw];
        const unsigned col0 = (unsigned)((4 * i0) % (size_t)cols);
#pragma unroll
        for (int k = 0; k < kUnrollFw; ++k) {
            const size_t j = i0 + 256 * k;
            if (j < n4) { g[k] = ld4(gate, j); v[k] = ld4(value, j); }
        }
#pragma unroll
        for (int k = 0; k < kUnrollFw; ++k) {
            const size_t j = i0 + 256 * k;
            if (j >= n4) continue;
            const unsigned c = col_of(col0, k, cols);
            const float4 gg = add4(g[k], bias4(bg, c)), vv = add4(v[k], bias4(bv, c));
            st4(out, j, make_float4(silu_f<OT>(gg.x, &s) * vv.x, silu_f<OT>(gg.y, &s) * vv.y, silu_f<OT>(gg.z, &s) * vv.z, silu_f<OT>(gg.w, &s) * vv.w));
        }
    } else {
        if (i >= n) return;
        st1(out, i, silu_f<OT>(ld1(gate, i) + bias1(bg, i, cols), &s) * (ld1(value, i) + bias1(bv, i, cols)));
    }
}

// d_gate = d * value * SiLU'(gate), d_value = d * SiLU(gate);  SiLU'(x) = s (1 + x (1 - s))
template <typename DT, typename IT, typename OT>
__global__ void __launch_bounds__(256) swiglu_bw_k(const DT* __restrict__ d, const IT* __restrict__ gate,
                                                   const IT* __restrict__ value, const float* __restrict__ bg,
                                                   const float* __restrict__ bv, int cols, OT* __restrict__ d_gate,
                                                   OT* __restrict__ d_value, size_t n, int vec) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    auto one = [](float dd, float g, float v, float* dg, float* dv) {
        float s;
        const float act = silu_f<OT>(g, &s);
        *dg = dd * v * (s * (1.f + g * (1.f - s)));
        *dv = dd * act;
    };
    if (vec) {
        const size_t n4 = n / 4, i0 = (size_t)blockIdx.x * (256 * kUnroll) + threadIdx.x;
        float4 dd[kUnroll], g[kUnroll], v[kUnroll];
        const unsigned col0 = (unsigned)((4 * i0) % (size_t)cols);
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j < n4) { dd[k] = ld4(d, j); g[k] = ld4(gate, j); v[k] = ld4(value, j); }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j >= n4) continue;
            const unsigned c = col_of(col0, k, cols);
            const float4 gg = add4(g[k], bias4(bg, c)), vv = add4(v[k], bias4(bv, c));
            float4 dg, dv;
            one(dd[k].x, gg.x, vv.x, &dg.x, &dv.x); one(dd[k].y, gg.y, vv.y, &dg.y, &dv.y);
            one(dd[k].z, gg.z, vv.z, &dg.z, &dv.z); one(dd[k].w, gg.w, vv.w, &dg.w, &dv.w);
            st4(d_gate, j, dg);
            st4(d_value, j, dv);
        }
    } else {
        if (i >= n) return;
        float dg, dv;
        one(ld1(d, i), ld1(gate, i) + bias1(bg, i, cols), ld1(value, i) + bias1(bv, i, cols), &dg, &dv);
        st1(d_gate, i, dg);
        st1(d_value, i, dv);
    }
}

// o <- sigmoid(o + bias) in place (kept for the backward), hc = o * yhat
template <typename OT>
__global__ void __launch_bounds__(256) ogate_fw_k(float* __restrict__ o, const float* __restrict__ yhat,
                                                  const float* __restrict__ bias, int cols, OT* __restrict__ hc, size_t n, int vec) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (vec) {
        const size_t n4 = n / 4, i0 = (size_t)blockIdx.x * (256 * kUnroll) + threadIdx.x;
        float4 a[kUnroll], y[kUnroll];
        const unsigned col0 = (unsigned)((4 * i0) % (size_t)cols);
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j < n4) { a[k] = ld4(o, j); y[k] = ld4(yhat, j); }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j >= n4) continue;
            float4 t = add4(a[k], bias4(bias, col_of(col0, k, cols)));
            t.x = sigmoid_for<OT>(t.x); t.y = sigmoid_for<OT>(t.y); t.z = sigmoid_for<OT>(t.z); t.w = sigmoid_for<OT>(t.w);
            reinterpret_cast<float4*>(o)[j] = t;
            st4(hc, j, make_float4(t.x * y[k].x, t.y * y[k].y, t.z * y[k].z, t.w * y[k].w));
        }
    } else {
        if (i >= n) return;
        const float a = sigmoid_for<OT>(o[i] + bias1(bias, i, cols));
        o[i] = a;
        st1(hc, i, a * yhat[i]);
    }
}

// do_pre = d_hc * yhat * o (1 - o), d_yhat = d_hc * o   (o is the activated gate)
template <typename OT>
__global__ void __launch_bounds__(256) ogate_bw_k(const float* __restrict__ d_hc, const float* __restrict__ o,
                                                  const float* __restrict__ yhat, OT* __restrict__ do_pre,
                                                  float* __restrict__ d_yhat, size_t n, int vec) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (vec) {
        const size_t n4 = n / 4, i0 = (size_t)blockIdx.x * (256 * kUnroll) + threadIdx.x;
        float4 dd[kUnroll], aa[kUnroll], yy[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j < n4) { dd[k] = ld4(d_hc, j); aa[k] = ld4(o, j); yy[k] = ld4(yhat, j); }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j >= n4) continue;
            const float4 d = dd[k], a = aa[k], y = yy[k];
            st4(do_pre, j, make_float4(d.x * y.x * a.x * (1.f - a.x), d.y * y.y * a.y * (1.f - a.y), d.z * y.z * a.z * (1.f - a.z),
                                       d.w * y.w * a.w * (1.f - a.w)));
            st4(d_yhat, j, make_float4(d.x * a.x, d.y * a.y, d.z * a.z, d.w * a.w));
        }
    } else {
        if (i >= n) return;
        const float d = d_hc[i], a = o[i];
        st1(do_pre, i, d * yhat[i] * a * (1.f - a));
        d_yhat[i] = d * a;
    }
}

// First position after p whose id differs from `id` (the ids are sorted: a binary search, not a walk along a run that a
// byte vocabulary makes hundreds of positions long).
__device__ __forceinline__ int run_end(const int* __restrict__ sorted_ids, int p, int n, int id) {
    int lo = p + 1, hi = n;  // the answer is in [lo, hi]
    while (lo < hi) {
        const int mid = lo + (hi - lo) / 2;
        if (__ldg(sorted_ids + mid) == id) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// table_g[id] += sum of the rows of d that carry token id, summed in ascending position order so the result
// does not depend on scheduling (no float atomics). `sorted_ids` are the token ids sorted stably and `order`
// the positions in that order; CTA p works only when p starts a run of equal ids, and then owns that row.
__global__ void __launch_bounds__(256) embedding_scatter_add_k(const float* __restrict__ d, const int* __restrict__ sorted_ids,
                                                               const int* __restrict__ order, float* __restrict__ table_g,
                                                               int n, int dm) {
    const int p = blockIdx.x;
    const int id = sorted_ids[p];
    if (p > 0 && sorted_ids[p - 1] == id) return;
    const int end = run_end(sorted_ids, p, n, id);
    float* dst = table_g + (size_t)id * dm;
    for (int c = threadIdx.x; c < dm; c += 256) {
        float acc = dst[c];
        for (int q = p; q < end; ++q) acc += d[(size_t)order[q] * dm + c];
        dst[c] = acc;
    }
}

// The same for row widths that are a multiple of four floats and whose 16-byte pieces (at most 256) divide the CTA:
// the CTA's threads form RL row lanes x CL column lanes; row lane r sums the run's rows r, r + RL, ... in that order with
// four rows' loads in flight, and the RL partial rows are added in lane order. A fixed order again, and a long run (a byte
// vocabulary: hundreds of rows per id) no longer walks its rows one dependent load after the other.
__global__ void __launch_bounds__(256) embedding_scatter_add_v4_k(const float* __restrict__ d, const int* __restrict__ sorted_ids,
                                                                  const int* __restrict__ order, float* __restrict__ table_g,
                                                                  int n, int dm, int CL) {
    __shared__ float4 part[256];
    const int p = blockIdx.x;
    const int id = sorted_ids[p];
    if (p > 0 && sorted_ids[p - 1] == id) return;
    const int end = run_end(sorted_ids, p, n, id);
    const int RL = 256 / CL, cl = threadIdx.x % CL, rl = threadIdx.x / CL, c4n = dm / 4;
    float4* dst = reinterpret_cast<float4*>(table_g + (size_t)id * dm);
    for (int c0 = 0; c0 < c4n; c0 += CL) {  // CL divides c4n or exceeds it only when c4n < CL is impossible (CL <= c4n)
        const int c4 = c0 + cl;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = p + rl; q < end; q += 4 * RL) {
            float4 r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int qq = q + k * RL;
                r[k] = qq < end ? __ldcs(reinterpret_cast<const float4*>(d + (size_t)__ldg(order + qq) * dm) + c4)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) { acc.x += r[k].x; acc.y += r[k].y; acc.z += r[k].z; acc.w += r[k].w; }
        }
        part[threadIdx.x] = acc;
        __syncthreads();
        if (rl == 0) {
            float4 t = dst[c4];
            for (int r2 = 0; r2 < RL; ++r2) {
                const float4 v = part[r2 * CL + cl];
                t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
            }
            dst[c4] = t;
        }
        __syncthreads();
    }
}

// x = hi + mid + lo with three bf16 terms (RNE at each step: hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid)),
// the operand form of the split-bf16 fp32 product; one pass instead of five casts and two subtractions.
__global__ void __launch_bounds__(256) split3_k(const float* __restrict__ x, bf16* __restrict__ hi, bf16* __restrict__ mid,
                                                bf16* __restrict__ lo, size_t n, int vec) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    auto one = [](float v, float* h, float* m, float* l) {
        *h = __bfloat162float(__float2bfloat16_rn(v));
        const float r = v - *h;
        *m = __bfloat162float(__float2bfloat16_rn(r));
        *l = r - *m;
    };
    if (vec) {
        const size_t n4 = n / 4, i0 = (size_t)blockIdx.x * (256 * kUnroll) + threadIdx.x;
        float4 vv[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j < n4) vv[k] = ld4(x, j);
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j >= n4) continue;
            const float4 v = vv[k];
            float4 h, m, l;
            one(v.x, &h.x, &m.x, &l.x); one(v.y, &h.y, &m.y, &l.y); one(v.z, &h.z, &m.z, &l.z); one(v.w, &h.w, &m.w, &l.w);
            st4(hi, j, h); st4(mid, j, m); st4(lo, j, l);
        }
    } else {
        if (i >= n) return;
        float h, m, l;
        one(x[i], &h, &m, &l);
        st1(hi, i, h); st1(mid, i, m); st1(lo, i, l);
    }
}

// ---- column sums (bias gradients) with the narrowing of the same tensor folded in -------------------------------
// partial[part][c] = sum over the part's rows of x[r][c]; out[r][c] = bf16(scale * x[r][c]) when asked for.
// A CTA covers 128 columns (32 threads x 4) and eight row lanes; the lanes are combined in lane order and the
// parts in part order by the merge kernel: fixed summation order, no float atomics (the reference's add_col_sum is
// deterministic the same way, src/gpu/cuda/common.cu:49-124).
template <typename T>
__global__ void __launch_bounds__(256) colsum_narrow_k(const T* __restrict__ x, bf16* __restrict__ out, float* __restrict__ partial,
                                                       int rows, int cols, float scale, int rows_per_part) {
    __shared__ float4 sacc[8][32];
    const int cq = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 128 + 4 * cq;
    const int r0 = blockIdx.y * rows_per_part, r1 = min(rows, r0 + rows_per_part);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c0 < cols) {
        const size_t c4 = (size_t)c0 / 4, row4 = (size_t)cols / 4;
        int r = r0 + rl;
        for (; r + 24 < r1; r += 32) {  // four rows in flight (summed in the same order as the loops below)
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = ld4(x, (size_t)(r + 8 * k) * row4 + c4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc.x += v[k].x; acc.y += v[k].y; acc.z += v[k].z; acc.w += v[k].w;
                if (out) st4(out, (size_t)(r + 8 * k) * row4 + c4, make_float4(v[k].x * scale, v[k].y * scale, v[k].z * scale, v[k].w * scale));
            }
        }
        for (; r + 8 < r1; r += 16) {  // two rows in flight
            const float4 v0 = ld4(x, (size_t)r * row4 + c4), v1 = ld4(x, (size_t)(r + 8) * row4 + c4);
            acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
            acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
            if (out) {
                st4(out, (size_t)r * row4 + c4, make_float4(v0.x * scale, v0.y * scale, v0.z * scale, v0.w * scale));
                st4(out, (size_t)(r + 8) * row4 + c4, make_float4(v1.x * scale, v1.y * scale, v1.z * scale, v1.w * scale));
            }
        }
        for (; r < r1; r += 8) {
            const float4 v0 = ld4(x, (size_t)r * row4 + c4);
            acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
            if (out) st4(out, (size_t)r * row4 + c4, make_float4(v0.x * scale, v0.y * scale, v0.z * scale, v0.w * scale));
        }
    }
    sacc[rl][cq] = acc;
    __syncthreads();
    if (threadIdx.x < 32 && c0 < cols) {
        float4 t = sacc[0][cq];
#pragma unroll
        for (int l = 1; l < 8; ++l) { const float4 u = sacc[l][cq]; t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
        *reinterpret_cast<float4*>(partial + (size_t)blockIdx.y * cols + c0) = make_float4(t.x * scale, t.y * scale, t.z * scale, t.w * scale);
    }
}
// any width / alignment: one thread per column
template <typename T>
__global__ void __launch_bounds__(128) colsum_narrow_gen_k(const T* __restrict__ x, bf16* __restrict__ out, float* __restrict__ partial,
                                                           int rows, int cols, float scale, int rows_per_part) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= cols) return;
    const int r0 = blockIdx.y * rows_per_part, r1 = min(rows, r0 + rows_per_part);
    float acc = 0.f;
    for (int r = r0; r < r1; ++r) {
        const float v = ldf(x, (size_t)r * cols + c);
        acc += v;
        if (out) out[(size_t)r * cols + c] = __float2bfloat16_rn(v * scale);
    }
    partial[(size_t)blockIdx.y * cols + c] = acc * scale;
}
static int colsum_parts(int rows, int cols) {
    const int tiles = (cols + 127) / 128;
    int want = (sm_count() * 4 + tiles - 1) / tiles;
    const int maxp = (rows + 15) / 16;
    if (want > maxp) want = maxp;
    return want < 1 ? 1 : want;
}

// out[r][c] = (residual ? residual[r][c] : 0) + bias[c]: the seed a GEMM with beta = 1 accumulates into
// (broadcast_row / broadcast_row_resid, src/gpu/cuda/common.cu:20-48).
__global__ void __launch_bounds__(256) bias_rows_k(const float* __restrict__ residual, const float* __restrict__ bias,
                                                   float* __restrict__ out, size_t n, int cols, int vec) {
    if (vec) {
        const size_t n4 = n / 4, i0 = (size_t)blockIdx.x * (256 * kUnroll) + threadIdx.x;
        float4 r[kUnroll];
        const unsigned col0 = (unsigned)((4 * i0) % (size_t)cols);
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            r[k] = (residual && j < n4) ? ld4(residual, j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const size_t j = i0 + 256 * k;
            if (j < n4) reinterpret_cast<float4*>(out)[j] = add4(r[k], bias4(bias, col_of(col0, k, cols)));
        }
    } else {
        const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
        if (i < n) out[i] = (residual ? residual[i] : 0.f) + bias[i % (size_t)cols];
    }
}

static inline int can_vec(size_t n, std::initializer_list<const void*> ptrs) {
    if (n % 4) return 0;
    for (const void* p : ptrs)
        if ((uintptr_t)p & 15) return 0;
    return 1;
}
static inline unsigned blocks_for(size_t n, int vec) {
    return vec ? (unsigned)((n / 4 + 256 * kUnroll - 1) / (256 * kUnroll)) : (unsigned)((n + 255) / 256);
}

}  // namespace xl

using namespace xl;

#define GLUE_CHECK(who)                                                                               \
    XL_CHECK_ARG(out_dtype == XLSTM_F32 || out_dtype == XLSTM_BF16, who ": out_dtype must be XLSTM_F32 or XLSTM_BF16"); \
    if (n == 0) return XLSTM_OK;

// the biases are read as float4 in the vector path: usable when cols is a multiple of 4 and they are 16-byte aligned
static inline int bias_vec_ok(const float* bg, const float* bv, int cols) {
    if (!bg && !bv) return 1;
    return cols % 4 == 0 && !((uintptr_t)bg & 15) && !((uintptr_t)bv & 15);
}

extern "C" int xlstm_swiglu_fw(void* stream, const void* gate_pre, const void* value, int in_dtype, const float* bias_gate,
                               const float* bias_value, int cols, void* out, int out_dtype, size_t n) {
    XL_CHECK_ARG(gate_pre && value && out, "swiglu_fw: null pointer");
    XL_CHECK_ARG((!bias_gate && !bias_value) || (cols > 0 && n % (size_t)cols == 0), "swiglu_fw: biases need cols > 0 dividing n");
    XL_CHECK_ARG(in_dtype == XLSTM_F32 || in_dtype == XLSTM_BF16, "swiglu_fw: in_dtype");
    GLUE_CHECK("swiglu_fw")
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = can_vec(n, {gate_pre, value, out}) && bias_vec_ok(bias_gate, bias_value, cols);
    if (cols <= 0) cols = 1;
    const unsigned nb = vec ? (unsigned)((n / 4 + 256 * kUnrollFw - 1) / (256 * kUnrollFw)) : blocks_for(n, 0);
    const bool ib = in_dtype == XLSTM_BF16, ob = out_dtype == XLSTM_BF16;
#define XL_SWIGLU_FW(IT, OT) \
    swiglu_fw_k<IT, OT><<<nb, 256, 0, st>>>((const IT*)gate_pre, (const IT*)value, bias_gate, bias_value, cols, (OT*)out, n, vec)
    if (ib && ob) XL_SWIGLU_FW(bf16, bf16);
    else if (ib) XL_SWIGLU_FW(bf16, float);
    else if (ob) XL_SWIGLU_FW(float, bf16);
    else XL_SWIGLU_FW(float, float);
#undef XL_SWIGLU_FW
    XL_LAUNCH_OK("swiglu_fw");
    return XLSTM_OK;
}

extern "C" int xlstm_swiglu_bw(void* stream, const void* d_mixed, int d_dtype, const void* gate_pre, const void* value,
                               int in_dtype, const float* bias_gate, const float* bias_value, int cols, void* d_gate,
                               void* d_value, int out_dtype, size_t n) {
    XL_CHECK_ARG(d_mixed && gate_pre && value && d_gate && d_value, "swiglu_bw: null pointer");
    XL_CHECK_ARG((!bias_gate && !bias_value) || (cols > 0 && n % (size_t)cols == 0), "swiglu_bw: biases need cols > 0 dividing n");
    XL_CHECK_ARG((in_dtype == XLSTM_F32 || in_dtype == XLSTM_BF16) && (d_dtype == XLSTM_F32 || d_dtype == XLSTM_BF16),
                 "swiglu_bw: in_dtype / d_dtype");
    GLUE_CHECK("swiglu_bw")
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = can_vec(n, {d_mixed, gate_pre, value, d_gate, d_value}) && bias_vec_ok(bias_gate, bias_value, cols);
    if (cols <= 0) cols = 1;
    const unsigned nb = blocks_for(n, vec);
    const bool db = d_dtype == XLSTM_BF16, ib = in_dtype == XLSTM_BF16, ob = out_dtype == XLSTM_BF16;
#define XL_SWIGLU_BW(DT, IT, OT)                                                                                          \
    swiglu_bw_k<DT, IT, OT><<<nb, 256, 0, st>>>((const DT*)d_mixed, (const IT*)gate_pre, (const IT*)value, bias_gate, bias_value, \
                                                cols, (OT*)d_gate, (OT*)d_value, n, vec)
    // narrow inputs come with narrow outputs (a bf16 layer); the fp32 layer is fp32 throughout, with the outputs' width free
    if (db && ib && ob) XL_SWIGLU_BW(bf16, bf16, bf16);
    else if (!db && ib && ob) XL_SWIGLU_BW(float, bf16, bf16);
    else if (!db && !ib && ob) XL_SWIGLU_BW(float, float, bf16);
    else if (!db && !ib && !ob) XL_SWIGLU_BW(float, float, float);
    else XL_CHECK_ARG(false, "swiglu_bw: this combination of widths is not built (bf16 inputs need bf16 outputs)");
#undef XL_SWIGLU_BW
    XL_LAUNCH_OK("swiglu_bw");
    return XLSTM_OK;
}

extern "C" int xlstm_ogate_fw(void* stream, float* o, const float* yhat, const float* bias, int cols, void* hc, int out_dtype,
                              size_t n) {
    XL_CHECK_ARG(o && yhat && hc, "ogate_fw: null pointer");
    XL_CHECK_ARG(!bias || (cols > 0 && n % (size_t)cols == 0), "ogate_fw: a bias needs cols > 0 dividing n");
    GLUE_CHECK("ogate_fw")
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = can_vec(n, {o, yhat, hc}) && bias_vec_ok(bias, nullptr, cols);
    if (cols <= 0) cols = 1;
    if (out_dtype == XLSTM_BF16) ogate_fw_k<bf16><<<blocks_for(n, vec), 256, 0, st>>>(o, yhat, bias, cols, (bf16*)hc, n, vec);
    else ogate_fw_k<float><<<blocks_for(n, vec), 256, 0, st>>>(o, yhat, bias, cols, (float*)hc, n, vec);
    XL_LAUNCH_OK("ogate_fw");
    return XLSTM_OK;
}

extern "C" int xlstm_ogate_bw(void* stream, const float* d_hc, const float* o, const float* yhat, void* do_pre, int out_dtype,
                              float* d_yhat, size_t n) {
    XL_CHECK_ARG(d_hc && o && yhat && do_pre && d_yhat, "ogate_bw: null pointer");
    GLUE_CHECK("ogate_bw")
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = can_vec(n, {d_hc, o, yhat, do_pre, d_yhat});
    if (out_dtype == XLSTM_BF16) ogate_bw_k<bf16><<<blocks_for(n, vec), 256, 0, st>>>(d_hc, o, yhat, (bf16*)do_pre, d_yhat, n, vec);
    else ogate_bw_k<float><<<blocks_for(n, vec), 256, 0, st>>>(d_hc, o, yhat, (float*)do_pre, d_yhat, n, vec);
    XL_LAUNCH_OK("ogate_bw");
    return XLSTM_OK;
}

extern "C" int xlstm_embedding_scatter_add(void* stream, const float* d, const int* sorted_ids, const int* order, float* table_g,
                                           int n, int dm) {
    XL_CHECK_ARG(d && sorted_ids && order && table_g, "embedding_scatter_add: null pointer");
    XL_CHECK_ARG(n >= 0 && dm > 0, "embedding_scatter_add: bad shape n=%d dm=%d", n, dm);
    if (n == 0) return XLSTM_OK;
    // 16-byte pieces per row: the vector kernel takes them when they tile the CTA's 256 threads (64 pieces x 4 row lanes at
    // a row of 256 floats) or are a multiple of 256
    const int c4n = dm % 4 == 0 ? dm / 4 : 0;
    const int CL = c4n >= 256 ? 256 : c4n;
    const bool v4 = c4n > 0 && CL > 0 && 256 % CL == 0 && c4n % CL == 0 && !(((uintptr_t)d | (uintptr_t)table_g) & 15);
    if (v4) embedding_scatter_add_v4_k<<<(unsigned)n, 256, 0, (cudaStream_t)stream>>>(d, sorted_ids, order, table_g, n, dm, CL);
    else embedding_scatter_add_k<<<(unsigned)n, 256, 0, (cudaStream_t)stream>>>(d, sorted_ids, order, table_g, n, dm);
    XL_LAUNCH_OK("embedding_scatter_add");
    return XLSTM_OK;
}

extern "C" int xlstm_split3_bf16(void* stream, const float* x, void* hi, void* mid, void* lo, size_t n) {
    XL_CHECK_ARG(x && hi && mid && lo, "split3_bf16: null pointer");
    if (n == 0) return XLSTM_OK;
    const int vec = can_vec(n, {x}) && !(((uintptr_t)hi | (uintptr_t)mid | (uintptr_t)lo) & 7);
    split3_k<<<blocks_for(n, vec), 256, 0, (cudaStream_t)stream>>>(x, (bf16*)hi, (bf16*)mid, (bf16*)lo, n, vec);
    XL_LAUNCH_OK("split3_bf16");
    return XLSTM_OK;
}

extern "C" size_t xlstm_colsum_workspace_bytes(int rows, int cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return (size_t)colsum_parts(rows, cols) * cols * sizeof(float);
}

extern "C" int xlstm_colsum_narrow(void* stream, const void* x, int x_dtype, int rows, int cols, float scale, void* out_bf16,
                                   float* acc, void* workspace, size_t workspace_bytes) {
    XL_CHECK_ARG(x && acc, "colsum_narrow: null pointer");
    XL_CHECK_ARG(rows >= 0 && cols > 0, "colsum_narrow: bad shape %d x %d", rows, cols);
    XL_CHECK_ARG(x_dtype == XLSTM_F32 || x_dtype == XLSTM_BF16, "colsum_narrow: unknown storage type");
    if (rows == 0) return XLSTM_OK;
    const size_t need = xlstm_colsum_workspace_bytes(rows, cols);
    if (!workspace || workspace_bytes < need) {
        set_error("colsum_narrow: workspace of %zu B is smaller than the %zu B required", workspace_bytes, need);
        return XLSTM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* partial = (float*)workspace;
    int nparts = colsum_parts(rows, cols);
    const int rpp = (rows + nparts - 1) / nparts;
    nparts = (rows + rpp - 1) / rpp;
    const bool vec = cols % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)out_bf16 & 7) && !((uintptr_t)partial & 15);
    const dim3 grid((cols + 127) / 128, nparts);
    if (vec) {
        if (x_dtype == XLSTM_F32) colsum_narrow_k<float><<<grid, 256, 0, st>>>((const float*)x, (bf16*)out_bf16, partial, rows, cols, scale, rpp);
        else colsum_narrow_k<bf16><<<grid, 256, 0, st>>>((const bf16*)x, (bf16*)out_bf16, partial, rows, cols, scale, rpp);
    } else {
        if (x_dtype == XLSTM_F32) colsum_narrow_gen_k<float><<<grid, 128, 0, st>>>((const float*)x, (bf16*)out_bf16, partial, rows, cols, scale, rpp);
        else colsum_narrow_gen_k<bf16><<<grid, 128, 0, st>>>((const bf16*)x, (bf16*)out_bf16, partial, rows, cols, scale, rpp);
    }
    XL_LAUNCH_OK("colsum_narrow");
    merge_parts8<<<(cols + 31) / 32, 256, 0, st>>>(partial, acc, nparts, cols);
    XL_LAUNCH_OK("colsum_parts_merge");
    return XLSTM_OK;
}

extern "C" int xlstm_bias_rows(void* stream, const float* residual, const float* bias, float* out, int rows, int cols) {
    XL_CHECK_ARG(bias && out, "bias_rows: null pointer");
    XL_CHECK_ARG(rows >= 0 && cols > 0, "bias_rows: bad shape %d x %d", rows, cols);
    const size_t n = (size_t)rows * cols;
    if (n == 0) return XLSTM_OK;
    const int vec = can_vec(n, {residual, out}) && bias_vec_ok(bias, nullptr, cols);
    bias_rows_k<<<blocks_for(n, vec), 256, 0, (cudaStream_t)stream>>>(residual, bias, out, n, cols, vec);
    XL_LAUNCH_OK("bias_rows");
    return XLSTM_OK;
}
