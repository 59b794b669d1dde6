// Softmax cross-entropy, forward and backward in one pass over the logits.
//
// One CTA (wide rows) or one warp (narrow rows) owns a row: it streams the logits once
// from HBM while keeping them in shared memory / registers, reduces max and sum-exp, then
// writes dlogits = (softmax - onehot) * inv from the on-chip copy: 8*C bytes per row. Row
// losses go to a scratch vector and are summed on the device in a fixed order into
// *loss_accum, so no host read-back sits on the step's critical path.
//
// Math: src/nn2/loss.rs:10-53 (p_t floored at 1e-30); masked form: src/gpu/cuda/
// mlstm_ops.cu:332-370. Kernels replaced: src/gpu/cuda/common.cu:270-289.
#include "common.cuh"

namespace xl {

// Soft-cap cap*tanh(x/cap) of the flat LM's head (src/nn2/ops.rs:25-42), fused into the loss kernels when
// CAP: the input is then the pre-cap logit, and the gradient is taken through the cap,
// d/dx = (p - onehot) * inv * (1 - tanh^2).
template <bool CAP>
__device__ __forceinline__ float capped(float x, float cap, float icap) {
    if (!CAP) return x;
    return cap * (1.f - __fdividef(2.f, 1.f + __expf(2.f * x * icap)));
}
template <bool CAP>
__device__ __forceinline__ float through_cap(float g, float t, float icap) {
    if (!CAP) return g;
    const float u = t * icap;
    return g * (1.f - u * u);
}

// ---- wide rows: one CTA per row, row cached in shared memory ---------------------------------
template <bool CACHE, bool CAP>
__global__ void __launch_bounds__(1024) ce_row_cta(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                                                   const uint32_t* __restrict__ mask, float* __restrict__ dlogits,
                                                   float* __restrict__ row_loss, int rows, int C, float inv, float cap) {
    const float icap = CAP ? 1.f / cap : 0.f;
    extern __shared__ __align__(16) float srow[];  // [C] when CACHE
    __shared__ float red[32];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* z = logits + (size_t)r * C;
        float* d = dlogits + (size_t)r * C;
        if (mask && !mask[r]) {
            for (int j = threadIdx.x; j < C; j += blockDim.x) d[j] = 0.f;
            if (threadIdx.x == 0) row_loss[r] = 0.f;
            continue;
        }
        // pass 1: load + running max / sum-exp per thread (online softmax)
        float mx = -INFINITY, sum = 0.f;
        const bool v4 = (C % 4 == 0) && (((uintptr_t)z & 15) == 0) && (((uintptr_t)d & 15) == 0);
        if (v4) {
            const float4* z4 = reinterpret_cast<const float4*>(z);
            const int n4 = C / 4, stride = blockDim.x;
            // four independent 16-byte loads in flight per thread before any of them is consumed
            for (int j0 = threadIdx.x; j0 < n4; j0 += 4 * stride) {
                float4 t[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + u * stride;
                    t[u] = (j < n4) ? __ldcs(z4 + j) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + u * stride;
                    if (j < n4) {
                        if (CAP) {
                            t[u].x = capped<CAP>(t[u].x, cap, icap); t[u].y = capped<CAP>(t[u].y, cap, icap);
                            t[u].z = capped<CAP>(t[u].z, cap, icap); t[u].w = capped<CAP>(t[u].w, cap, icap);
                        }
                        if (CACHE) reinterpret_cast<float4*>(srow)[j] = t[u];
                        float m4 = fmaxf(fmaxf(t[u].x, t[u].y), fmaxf(t[u].z, t[u].w));
                        if (m4 > mx) { sum *= __expf(mx - m4); mx = m4; }
                        sum += __expf(t[u].x - mx) + __expf(t[u].y - mx) + __expf(t[u].z - mx) + __expf(t[u].w - mx);
                    }
                }
            }
        } else {
            for (int j = threadIdx.x; j < C; j += blockDim.x) {
                float t = capped<CAP>(z[j], cap, icap);
                if (CACHE) srow[j] = t;
                if (t > mx) { sum *= expf(mx - t); mx = t; }
                sum += expf(t - mx);
            }
        }
        if (CACHE && r + (int)gridDim.x < rows) {
            // pull this CTA's next row into L2 while this row is reduced and its gradient written, so that DRAM
            // keeps reading through those phases and the next pass 1 starts from L2
            const char* nz = reinterpret_cast<const char*>(logits + (size_t)(r + gridDim.x) * C);
            for (size_t o = (size_t)threadIdx.x * 128; o < (size_t)C * sizeof(float); o += (size_t)blockDim.x * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(nz + o));
        }
        float gmx = block_max(mx, red);
        sum = (mx == -INFINITY) ? 0.f : sum * expf(mx - gmx);
        float gsum = block_sum(sum, red);
        const float is = 1.f / gsum;
        const uint32_t tg = targets[r];
        if (threadIdx.x == 0) {
            float zt = CACHE ? srow[tg] : capped<CAP>(z[tg], cap, icap);
            float pt = expf(zt - gmx) * is;
            row_loss[r] = -logf(fmaxf(pt, 1e-30f));
        }
        if (!CACHE) __syncthreads();  // dlogits may alias logits: read z[target] before anyone overwrites it
        // pass 2: gradient from the on-chip copy
        if (v4) {
            float4* d4 = reinterpret_cast<float4*>(d);
            for (int j = threadIdx.x; j < C / 4; j += blockDim.x) {
                float4 t = CACHE ? reinterpret_cast<float4*>(srow)[j] : reinterpret_cast<const float4*>(z)[j];
                if (CAP && !CACHE) {
                    t.x = capped<CAP>(t.x, cap, icap); t.y = capped<CAP>(t.y, cap, icap);
                    t.z = capped<CAP>(t.z, cap, icap); t.w = capped<CAP>(t.w, cap, icap);
                }
                float4 o;
                o.x = __expf(t.x - gmx) * is; o.y = __expf(t.y - gmx) * is;
                o.z = __expf(t.z - gmx) * is; o.w = __expf(t.w - gmx) * is;
                uint32_t base = 4u * j;
                if (tg == base) o.x -= 1.f;
                else if (tg == base + 1u) o.y -= 1.f;
                else if (tg == base + 2u) o.z -= 1.f;
                else if (tg == base + 3u) o.w -= 1.f;
                o.x = through_cap<CAP>(o.x * inv, t.x, icap); o.y = through_cap<CAP>(o.y * inv, t.y, icap);
                o.z = through_cap<CAP>(o.z * inv, t.z, icap); o.w = through_cap<CAP>(o.w * inv, t.w, icap);
                __stcs(d4 + j, o);
            }
        } else {
            for (int j = threadIdx.x; j < C; j += blockDim.x) {
                float t = CACHE ? srow[j] : capped<CAP>(z[j], cap, icap);
                float o = expf(t - gmx) * is;
                if ((uint32_t)j == tg) o -= 1.f;
                d[j] = through_cap<CAP>(o * inv, t, icap);
            }
        }
        __syncthreads();  // srow is reused by the next row
    }
}

// ---- narrow rows (C <= 1024): one warp per row, row in registers -----------------------------
template <int VPL, bool CAP>
__global__ void __launch_bounds__(256) ce_row_warp(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                                                   const uint32_t* __restrict__ mask, float* __restrict__ dlogits,
                                                   float* __restrict__ row_loss, int rows, int C, float inv, float cap) {
    const float icap = CAP ? 1.f / cap : 0.f;
    const int lane = threadIdx.x & 31;
    const int wglobal = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int wstride = gridDim.x * (blockDim.x >> 5);
    for (int r = wglobal; r < rows; r += wstride) {
        const float* z = logits + (size_t)r * C;
        float* d = dlogits + (size_t)r * C;
        if (mask && !mask[r]) {
            for (int j = lane; j < C; j += 32) d[j] = 0.f;
            if (lane == 0) row_loss[r] = 0.f;
            continue;
        }
        float v[VPL];
        float tc[CAP ? VPL : 1];  // capped logits, needed again for the gradient through the cap
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int j = i * 32 + lane;
            v[i] = j < C ? capped<CAP>(z[j], cap, icap) : -INFINITY;
            if (CAP) tc[i] = j < C ? v[i] : 0.f;
            mx = fmaxf(mx, v[i]);
        }
        mx = warp_max(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            v[i] = expf(v[i] - mx);  // exp(-inf) = 0 for the padding
            sum += v[i];
        }
        sum = warp_sum(sum);
        const float is = 1.f / sum;
        const uint32_t tg = targets[r];
        float pt = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int j = i * 32 + lane;
            float p = v[i] * is;
            if ((uint32_t)j == tg) { pt = p; p -= 1.f; }
            if (j < C) d[j] = through_cap<CAP>(p * inv, CAP ? tc[i] : 0.f, icap);
        }
        pt = warp_sum(pt);
        if (lane == 0) row_loss[r] = -logf(fmaxf(pt, 1e-30f));
    }
}

// ---- narrow rows whose width is a multiple of 4 (a byte vocabulary, C = 256): one warp per PAIR of rows, 128-bit
// accesses, both rows' loads in flight before either is reduced.
template <int V4, bool CAP>
__global__ void __launch_bounds__(256) ce_row_warp4(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                                                    const uint32_t* __restrict__ mask, float* __restrict__ dlogits,
                                                    float* __restrict__ row_loss, int rows, int C, float inv, float cap) {
    const float icap = CAP ? 1.f / cap : 0.f;
    const int lane = threadIdx.x & 31;
    const int wglobal = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int wstride = gridDim.x * (blockDim.x >> 5);
    const int n4 = C / 4;
    for (int r0 = 2 * wglobal; r0 < rows; r0 += 2 * wstride) {
        float4 v[2][V4];
        bool live[2];
        uint32_t tg[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = r0 + e;
            live[e] = r < rows && !(mask && !mask[r]);
            tg[e] = live[e] ? targets[r] : 0u;
            const float4* z4 = reinterpret_cast<const float4*>(logits + (size_t)r * C);
#pragma unroll
            for (int i = 0; i < V4; ++i) {
                const int j = i * 32 + lane;
                v[e][i] = (live[e] && j < n4) ? __ldcs(z4 + j) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = r0 + e;
            if (r >= rows) break;
            float4* d4 = reinterpret_cast<float4*>(dlogits + (size_t)r * C);
            if (!live[e]) {
#pragma unroll
                for (int i = 0; i < V4; ++i) {
                    const int j = i * 32 + lane;
                    if (j < n4) __stcs(d4 + j, make_float4(0.f, 0.f, 0.f, 0.f));
                }
                if (lane == 0) row_loss[r] = 0.f;
                continue;
            }
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < V4; ++i) {
                if (CAP) {
                    v[e][i].x = capped<CAP>(v[e][i].x, cap, icap); v[e][i].y = capped<CAP>(v[e][i].y, cap, icap);
                    v[e][i].z = capped<CAP>(v[e][i].z, cap, icap); v[e][i].w = capped<CAP>(v[e][i].w, cap, icap);
                }
                mx = fmaxf(mx, fmaxf(fmaxf(v[e][i].x, v[e][i].y), fmaxf(v[e][i].z, v[e][i].w)));
            }
            mx = warp_max(mx);
            float sum = 0.f;
            float4 ex[V4];
#pragma unroll
            for (int i = 0; i < V4; ++i) {  // exp(-inf) = 0 for the padding (capped(-inf) = -cap is masked by j < n4 below)
                const bool in = i * 32 + lane < n4;
                ex[i].x = in ? __expf(v[e][i].x - mx) : 0.f; ex[i].y = in ? __expf(v[e][i].y - mx) : 0.f;
                ex[i].z = in ? __expf(v[e][i].z - mx) : 0.f; ex[i].w = in ? __expf(v[e][i].w - mx) : 0.f;
                sum += (ex[i].x + ex[i].y) + (ex[i].z + ex[i].w);
            }
            sum = warp_sum(sum);
            const float is = 1.f / sum;
            float pt = 0.f;
#pragma unroll
            for (int i = 0; i < V4; ++i) {
                const int j = i * 32 + lane;
                if (j >= n4) continue;
                float4 o = make_float4(ex[i].x * is, ex[i].y * is, ex[i].z * is, ex[i].w * is);
                const uint32_t base = 4u * j;
                if (tg[e] == base) { pt = o.x; o.x -= 1.f; }
                else if (tg[e] == base + 1u) { pt = o.y; o.y -= 1.f; }
                else if (tg[e] == base + 2u) { pt = o.z; o.z -= 1.f; }
                else if (tg[e] == base + 3u) { pt = o.w; o.w -= 1.f; }
                o.x = through_cap<CAP>(o.x * inv, v[e][i].x, icap); o.y = through_cap<CAP>(o.y * inv, v[e][i].y, icap);
                o.z = through_cap<CAP>(o.z * inv, v[e][i].z, icap); o.w = through_cap<CAP>(o.w * inv, v[e][i].w, icap);
                __stcs(d4 + j, o);
            }
            pt = warp_sum(pt);
            if (lane == 0) row_loss[r] = -logf(fmaxf(pt, 1e-30f));
        }
    }
}

// *loss_accum += inv * sum(row_loss), one CTA, fixed order.
__global__ void __launch_bounds__(1024) ce_loss_reduce(const float* __restrict__ row_loss, float* loss_accum, int rows, float inv) {
    __shared__ float red[32];
    float s = 0.f;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) s += row_loss[r];
    s = block_sum(s, red);
    if (threadIdx.x == 0) *loss_accum += s * inv;
}

}  // namespace xl

using namespace xl;

extern "C" size_t xlstm_ce_workspace_bytes(int rows) { return rows > 0 ? (size_t)rows * sizeof(float) : 0; }

template <bool CAP>
static int ce_run(void* stream, const float* logits, const uint32_t* targets, const uint32_t* mask, float* dlogits,
                  float* loss_accum, int rows, int C, float inv, float cap, void* workspace, size_t workspace_bytes) {
    XL_CHECK_ARG(logits && targets && dlogits && loss_accum, "ce_fw_bw: null pointer");
    XL_CHECK_ARG(rows >= 0 && C > 0, "ce_fw_bw: bad shape rows=%d C=%d", rows, C);
    if (rows == 0) return XLSTM_OK;
    if (!workspace || workspace_bytes < xlstm_ce_workspace_bytes(rows)) {
        set_error("ce_fw_bw: workspace of %zu B is smaller than the %zu B required", workspace_bytes,
                  xlstm_ce_workspace_bytes(rows));
        return XLSTM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* row_loss = (float*)workspace;
    const bool aligned16 = !(((uintptr_t)logits | (uintptr_t)dlogits) & 15);
    if (C <= 1024 && C % 4 == 0 && aligned16) {
        const int pairs = (rows + 1) / 2, nb = (pairs + 7) / 8, maxb = sm_count() * 8;
        const int grid = nb < maxb ? nb : maxb;
#define RUN4(V) ce_row_warp4<V, CAP><<<grid, 256, 0, st>>>(logits, targets, mask, dlogits, row_loss, rows, C, inv, cap)
        if (C <= 128) RUN4(1);
        else if (C <= 256) RUN4(2);
        else if (C <= 512) RUN4(4);
        else RUN4(8);
#undef RUN4
        XL_LAUNCH_OK("ce_row_warp4");
    } else if (C <= 1024) {
        int wpb = 8;
        int nb = (rows + wpb - 1) / wpb, maxb = sm_count() * 8;
        int grid = nb < maxb ? nb : maxb;
#define RUN(V) ce_row_warp<V, CAP><<<grid, 256, 0, st>>>(logits, targets, mask, dlogits, row_loss, rows, C, inv, cap)
        if (C <= 32) RUN(1);
        else if (C <= 64) RUN(2);
        else if (C <= 128) RUN(4);
        else if (C <= 256) RUN(8);
        else if (C <= 512) RUN(16);
        else RUN(32);
#undef RUN
        XL_LAUNCH_OK("ce_row_warp");
    } else {
        size_t smem = (size_t)C * sizeof(float);
        int threads = C >= 8192 ? 1024 : 256;
        if (smem <= 200 * 1024) {
            XL_CUDA(cudaFuncSetAttribute(ce_row_cta<true, CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            int per_sm = (int)((220 * 1024) / (smem + 1024));
            if (per_sm < 1) per_sm = 1;
            if (per_sm > 2048 / threads) per_sm = 2048 / threads;
            int maxb = sm_count() * per_sm;
            ce_row_cta<true, CAP><<<rows < maxb ? rows : maxb, threads, smem, st>>>(logits, targets, mask, dlogits, row_loss, rows, C, inv, cap);
        } else {
            int maxb = sm_count() * 2;
            ce_row_cta<false, CAP><<<rows < maxb ? rows : maxb, 1024, 0, st>>>(logits, targets, mask, dlogits, row_loss, rows, C, inv, cap);
        }
        XL_LAUNCH_OK("ce_row_cta");
    }
    ce_loss_reduce<<<1, 1024, 0, st>>>(row_loss, loss_accum, rows, inv);
    XL_LAUNCH_OK("ce_loss_reduce");
    return XLSTM_OK;
}

extern "C" int xlstm_ce_fw_bw(void* stream, const float* logits, const uint32_t* targets, const uint32_t* mask,
                              float* dlogits, float* loss_accum, int rows, int C, float inv, void* workspace,
                              size_t workspace_bytes) {
    return ce_run<false>(stream, logits, targets, mask, dlogits, loss_accum, rows, C, inv, 0.f, workspace, workspace_bytes);
}

extern "C" int xlstm_softcap_ce_fw_bw(void* stream, const float* pre_logits, const uint32_t* targets, const uint32_t* mask,
                                      float* d_pre, float* loss_accum, int rows, int C, float inv, float cap, void* workspace,
                                      size_t workspace_bytes) {
    XL_CHECK_ARG(cap > 0.f, "softcap_ce_fw_bw: cap must be positive (got %g)", (double)cap);
    return ce_run<true>(stream, pre_logits, targets, mask, d_pre, loss_accum, rows, C, inv, cap, workspace, workspace_bytes);
}

// ---- the same op for callers that cannot allocate device memory --------------------------------
//
// xlstm_ce_fw_bw needs one float of scratch per row and asks the caller for it. Some hosts have no
// way to supply that: the reference's own runtime hands every byte of device memory to its buffer
// pool up front, and a step loop that must never touch the CUDA allocator (because cudaMalloc and
// cudaFree can synchronise the whole device, or because the surrounding code runs where allocation
// calls are not allowed) has the same problem. For them the scratch lives inside the library, in a
// fixed array that every GPU loading the library keeps resident until the process exits.
//
// Limits and sharing rules, because the array is one per device and is never cleared:
//   - at most XLSTM_CE_NOALLOC_MAX_ROWS rows per call (256 KiB of scratch); more is refused;
//   - every element a call reads is written earlier in the same call, so stale contents from the
//     previous call are harmless and nothing needs zeroing;
//   - two calls whose kernels may overlap on the same device (different streams) race on the
//     array; serialise them on one stream.
// The first call on each device looks up the array's device address (cudaGetSymbolAddress, which
// is not an allocation); make that first call before starting any stream capture.
static constexpr int kCeNoAllocMaxRows = 65536;
static __device__ __align__(256) float g_ce_noalloc_scratch[kCeNoAllocMaxRows];

static float* ce_noalloc_scratch_ptr(int* rc) {
    // In host code the array's name is only a handle; the kernels need its device address.
    static std::atomic<float*> cached[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("ce_fw_bw_noalloc: cudaGetDevice failed or device index out of range: %s", cudaGetErrorString(e));
        *rc = XLSTM_ERR_CUDA;
        return nullptr;
    }
    float* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_ce_noalloc_scratch);
        if (e != cudaSuccess || !addr) {
            set_error("ce_fw_bw_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            *rc = XLSTM_ERR_CUDA;
            return nullptr;
        }
        p = (float*)addr;
        cached[dev].store(p, std::memory_order_release);
    }
    *rc = XLSTM_OK;
    return p;
}

extern "C" int xlstm_ce_fw_bw_noalloc(void* stream, const float* logits, const uint32_t* targets, const uint32_t* mask,
                                      float* dlogits, float* loss_accum, int rows, int C, float inv) {
    if (rows > kCeNoAllocMaxRows) {
        set_error("ce_fw_bw_noalloc: %d rows exceed the built-in scratch of %d rows; split the call or use xlstm_ce_fw_bw "
                  "with a caller-owned workspace", rows, kCeNoAllocMaxRows);
        return XLSTM_ERR_ARG;
    }
    int rc = XLSTM_OK;
    float* scratch = ce_noalloc_scratch_ptr(&rc);
    if (!scratch) return rc;
    return xlstm_ce_fw_bw(stream, logits, targets, mask, dlogits, loss_accum, rows, C, inv, scratch,
                          (size_t)kCeNoAllocMaxRows * sizeof(float));
}
