// Grouped RMSNorm forward / backward — bandwidth-bound streaming kernels.
//
// A team of threads (a warp, or a whole CTA for wide groups) owns one (row, group) at a time
// and keeps it in registers between the reduction and the write, so the forward moves
// 8 B/element (read x, write y) and the backward 12 B/element (read dy and x, write dx);
// x_hat is rebuilt from x and inv_rms instead of being stored. The column sums for dgamma
// are accumulated in registers across the rows a team visits and combined in a fixed order
// (teams of a CTA, then CTAs), never with floating-point atomics.
//
// Math: src/nn2/ops.rs:110-185; kernels replaced: src/gpu/cuda/common.cu:210-265.
#include "common.cuh"

namespace xl {

static constexpr int kWarpsPerCta = 8;

// ---- typed 4-element accesses: fp32 (16 bytes) or bf16 (8 bytes) storage ----------------------
__device__ __forceinline__ float4 ld4(const float* p, long long i4) { return __ldcs(reinterpret_cast<const float4*>(p) + i4); }
__device__ __forceinline__ float4 ld4(const bf16* p, long long i4) {
    const uint2 u = __ldcs(reinterpret_cast<const uint2*>(p) + i4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, long long i4, float4 v) { __stcs(reinterpret_cast<float4*>(p) + i4, v); }
__device__ __forceinline__ void st4(bf16* p, long long i4, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    __stcs(reinterpret_cast<uint2*>(p) + i4, u);
}

// ---- vector path: group % 4 == 0 -----------------------------------------------------------
// A "team" of TPG threads (a warp, or the whole 256-thread CTA for wide groups) owns one
// (row, group) at a time; each thread holds VPL float4 of it in registers.
template <int TPG>
__device__ __forceinline__ float team_sum(float v, float* red) {
    if (TPG == 32) return warp_sum(v);
    return block_sum(v, red);
}

template <int VPL, int TPG, typename XT, typename YT>
__global__ void __launch_bounds__(kWarpsPerCta * 32) rmsnorm_fw_vec(
    const XT* __restrict__ x, const float* __restrict__ gamma, YT* __restrict__ y,
    float* __restrict__ inv_rms, float* __restrict__ x_hat, long long ngroups, int F, int group, float eps) {
    __shared__ float red[32];
    constexpr int TEAMS = kWarpsPerCta * 32 / TPG;
    const int lane = threadIdx.x % TPG;
    const long long tglobal = (long long)blockIdx.x * TEAMS + threadIdx.x / TPG;
    const long long tstride = (long long)gridDim.x * TEAMS;
    const int gpr = F / group, g4 = group / 4;
    for (long long gi = tglobal; gi < ngroups; gi += tstride) {
        const long long row = gi / gpr;
        const int gc = (int)(gi % gpr);
        const XT* xp = x + row * F + (long long)gc * group;
        float4 r[VPL];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                r[i] = ld4(xp, idx);
                ss += r[i].x * r[i].x + r[i].y * r[i].y + r[i].z * r[i].z + r[i].w * r[i].w;
            }
        }
        ss = team_sum<TPG>(ss, red);
        const float inv = 1.f / sqrtf(ss / (float)group + eps);
        if (lane == 0) inv_rms[gi] = inv;
        const float4* gp = reinterpret_cast<const float4*>(gamma + (long long)gc * group);
        YT* yp = y + row * F + (long long)gc * group;
        float4* hp = x_hat ? reinterpret_cast<float4*>(x_hat + row * F + (long long)gc * group) : nullptr;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                float4 g = __ldg(gp + idx);
                float4 xh = make_float4(r[i].x * inv, r[i].y * inv, r[i].z * inv, r[i].w * inv);
                if (hp) __stcs(hp + idx, xh);
                st4(yp, idx, make_float4(g.x * xh.x, g.y * xh.y, g.z * xh.z, g.w * xh.w));
            }
        }
    }
}

// Backward: CTA c owns column group (c % gpr) and row slice (c / gpr); its teams stride
// over that slice's rows. partial [gridDim.x / gpr, F] receives the CTA's dgamma sums.
template <int VPL, int TPG, typename XT, typename DT>
__global__ void __launch_bounds__(kWarpsPerCta * 32) rmsnorm_bw_vec(
    const float* __restrict__ dy, const XT* __restrict__ x, const float* __restrict__ inv_rms,
    const float* __restrict__ gamma, const float* __restrict__ residual, DT* __restrict__ dx,
    float* __restrict__ partial, int rows, int F, int group) {
    extern __shared__ float sacc[];  // [group]
    __shared__ float red[32];
    constexpr int TEAMS = kWarpsPerCta * 32 / TPG;
    const int lane = threadIdx.x % TPG, team = threadIdx.x / TPG;
    const int gpr = F / group, g4 = group / 4;
    const int gc = blockIdx.x % gpr, part = blockIdx.x / gpr, nparts = gridDim.x / gpr;
    float4 acc[VPL];
    float4 gam[VPL];
    const float4* gp = reinterpret_cast<const float4*>(gamma + (long long)gc * group);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        int idx = i * TPG + lane;
        gam[i] = idx < g4 ? __ldg(gp + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (long long row = (long long)part * TEAMS + team; row < rows; row += (long long)nparts * TEAMS) {
        const long long off = row * F + (long long)gc * group;
        const float4* dyp = reinterpret_cast<const float4*>(dy + off);
        const XT* xp = x + off;
        const float inv = inv_rms[row * gpr + gc];
        float4 d[VPL], xh[VPL];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                d[i] = __ldcs(dyp + idx);
                float4 xv = ld4(xp, idx);
                xh[i] = make_float4(xv.x * inv, xv.y * inv, xv.z * inv, xv.w * inv);
                float4 p = make_float4(d[i].x * xh[i].x, d[i].y * xh[i].y, d[i].z * xh[i].z, d[i].w * xh[i].w);
                acc[i].x += p.x; acc[i].y += p.y; acc[i].z += p.z; acc[i].w += p.w;
                s += gam[i].x * p.x + gam[i].y * p.y + gam[i].z * p.z + gam[i].w * p.w;
            }
        }
        s = team_sum<TPG>(s, red) / (float)group;
        DT* dxp = dx + off;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                float4 o = make_float4(inv * (gam[i].x * d[i].x - xh[i].x * s), inv * (gam[i].y * d[i].y - xh[i].y * s),
                                       inv * (gam[i].z * d[i].z - xh[i].z * s), inv * (gam[i].w * d[i].w - xh[i].w * s));
                if (residual) {  // the residual branch's gradient joins here instead of in a pass of its own
                    const float4 rr = __ldcs(reinterpret_cast<const float4*>(residual + off) + idx);
                    o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w;
                }
                st4(dxp, idx, o);
            }
        }
    }
    // combine the CTA's teams in team order
    float4* sacc4 = reinterpret_cast<float4*>(sacc);
    for (int w = 0; w < TEAMS; ++w) {
        if (team == w) {
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                int idx = i * TPG + lane;
                if (idx < g4) {
                    float4 cur = (w == 0) ? make_float4(0.f, 0.f, 0.f, 0.f) : sacc4[idx];
                    sacc4[idx] = make_float4(cur.x + acc[i].x, cur.y + acc[i].y, cur.z + acc[i].z, cur.w + acc[i].w);
                }
            }
        }
        __syncthreads();
    }
    float* prow = partial + (long long)part * F + (long long)gc * group;
    for (int c = threadIdx.x; c < group; c += blockDim.x) prow[c] = sacc[c];
}


// ---- generic path: any group size -------------------------------------------------------
template <typename XT, typename YT>
__global__ void rmsnorm_fw_gen(const XT* __restrict__ x, const float* __restrict__ gamma, YT* __restrict__ y,
                               float* __restrict__ inv_rms, float* __restrict__ x_hat, long long ngroups, int F,
                               int group, float eps) {
    const int lane = threadIdx.x & 31;
    const long long wglobal = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
    const int gpr = F / group;
    for (long long gi = wglobal; gi < ngroups; gi += wstride) {
        const long long off = (gi / gpr) * F + (gi % gpr) * group;
        const int goff = (int)(gi % gpr) * group;
        float ss = 0.f;
        for (int i = lane; i < group; i += 32) ss += ldf(x, off + i) * ldf(x, off + i);
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)group + eps);
        if (lane == 0) inv_rms[gi] = inv;
        for (int i = lane; i < group; i += 32) {
            float xh = ldf(x, off + i) * inv;
            if (x_hat) x_hat[off + i] = xh;
            stf(y, off + i, gamma[goff + i] * xh);
        }
    }
}

template <typename XT, typename DT>
__global__ void rmsnorm_bw_gen(const float* __restrict__ dy, const XT* __restrict__ x,
                               const float* __restrict__ inv_rms, const float* __restrict__ gamma,
                               const float* __restrict__ residual, DT* __restrict__ dx, long long ngroups, int F, int group) {
    const int lane = threadIdx.x & 31;
    const long long wglobal = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
    const int gpr = F / group;
    for (long long gi = wglobal; gi < ngroups; gi += wstride) {
        const long long off = (gi / gpr) * F + (gi % gpr) * group;
        const int goff = (int)(gi % gpr) * group;
        const float inv = inv_rms[gi];
        float s = 0.f;
        for (int i = lane; i < group; i += 32) s += gamma[goff + i] * dy[off + i] * (ldf(x, off + i) * inv);
        s = warp_sum(s) / (float)group;
        for (int i = lane; i < group; i += 32)
            stf(dx, off + i, inv * (gamma[goff + i] * dy[off + i] - (ldf(x, off + i) * inv) * s) + (residual ? residual[off + i] : 0.f));
    }
}

// partial[part][c] = sum over the part's rows of dy*x*inv  (generic dgamma, stage 1)
template <typename XT>
__global__ void colsum_mul_gen(const float* __restrict__ dy, const XT* __restrict__ x,
                               const float* __restrict__ inv_rms, float* __restrict__ partial, int rows, int F,
                               int group, int rows_per_part) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= F) return;
    const int gpr = F / group, gc = c / group;
    int r0 = blockIdx.y * rows_per_part, r1 = min(rows, r0 + rows_per_part);
    float s = 0.f;
    for (int r = r0; r < r1; ++r) s += dy[(long long)r * F + c] * ldf(x, (size_t)r * F + c) * inv_rms[(long long)r * gpr + gc];
    partial[(long long)blockIdx.y * F + c] = s;
}

static bool vec_ok(const void* a, const void* b, const void* c, int F, int group) {
    auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    return group % 4 == 0 && F % 4 == 0 && group <= 256 * 4 * 4 && al(a) && al(b) && (c == nullptr || al(c));
}

static int bw_parts_vec(int rows, int F, int group) {
    int gpr = F / group;
    int teams = group / 4 <= 128 ? kWarpsPerCta : 1;
    int want = (sm_count() * 4 + gpr - 1) / gpr;
    int maxp = (rows + teams - 1) / teams;
    int p = want < maxp ? want : maxp;
    return p < 1 ? 1 : p;
}
static int bw_parts_gen(int rows) {
    int p = (rows + 63) / 64;
    return p > 512 ? 512 : (p < 1 ? 1 : p);
}

}  // namespace xl

using namespace xl;

template <typename XT, typename YT>
static int rmsnorm_fw_run(cudaStream_t st, const XT* x, const float* gamma, YT* y, float* inv_rms, float* x_hat, int rows,
                          int F, int group, float eps) {
    long long ngroups = (long long)rows * (F / group);
    int maxb = sm_count() * 8;
    if (vec_ok(x, y, x_hat, F, group) && ((uintptr_t)gamma & 15) == 0) {
        int g4 = group / 4;
        int teams = g4 <= 512 ? kWarpsPerCta : 1;  // forward: a warp keeps up to 2048 floats of a row in registers
        long long nb = (ngroups + teams - 1) / teams;
        int grid = (int)(nb < maxb ? nb : maxb);
#define RUN(V, TPG) rmsnorm_fw_vec<V, TPG, XT, YT><<<grid, kWarpsPerCta * 32, 0, st>>>(x, gamma, y, inv_rms, x_hat, ngroups, F, group, eps)
        if (g4 <= 32) RUN(1, 32);
        else if (g4 <= 64) RUN(2, 32);
        else if (g4 <= 128) RUN(4, 32);
        else if (g4 <= 256) RUN(8, 32);
        else if (g4 <= 512) RUN(16, 32);
        else RUN(4, 256);
#undef RUN
        XL_LAUNCH_OK("rmsnorm_fw_vec");
    } else {
        long long nb = (ngroups + 7) / 8;
        int grid = (int)(nb < maxb ? nb : maxb);
        rmsnorm_fw_gen<XT, YT><<<grid, 256, 0, st>>>(x, gamma, y, inv_rms, x_hat, ngroups, F, group, eps);
        XL_LAUNCH_OK("rmsnorm_fw_gen");
    }
    return XLSTM_OK;
}

extern "C" int xlstm_rmsnorm_fw(void* stream, const void* x, int x_dtype, const float* gamma, void* y, int y_dtype,
                                float* inv_rms, float* x_hat, int rows, int F, int group, float eps) {
    XL_CHECK_ARG(x && gamma && y && inv_rms, "rmsnorm_fw: null pointer");
    XL_CHECK_ARG(rows >= 0 && F > 0 && group > 0 && F % group == 0, "rmsnorm_fw: group %d does not divide width %d", group, F);
    XL_CHECK_ARG((x_dtype == XLSTM_F32 || x_dtype == XLSTM_BF16) && (y_dtype == XLSTM_F32 || y_dtype == XLSTM_BF16),
                 "rmsnorm_fw: unknown storage type");
    if (rows == 0) return XLSTM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == XLSTM_F32)
        return y_dtype == XLSTM_F32 ? rmsnorm_fw_run(st, (const float*)x, gamma, (float*)y, inv_rms, x_hat, rows, F, group, eps)
                                    : rmsnorm_fw_run(st, (const float*)x, gamma, (bf16*)y, inv_rms, x_hat, rows, F, group, eps);
    return y_dtype == XLSTM_F32 ? rmsnorm_fw_run(st, (const bf16*)x, gamma, (float*)y, inv_rms, x_hat, rows, F, group, eps)
                                : rmsnorm_fw_run(st, (const bf16*)x, gamma, (bf16*)y, inv_rms, x_hat, rows, F, group, eps);
}

extern "C" size_t xlstm_rmsnorm_bw_workspace_bytes(int rows, int F) {
    if (rows <= 0 || F <= 0) return 0;
    // enough for either path: parts <= max(4*SMs, 512)
    int parts = sm_count() * 4;
    if (parts < 512) parts = 512;
    return (size_t)parts * F * sizeof(float);
}

template <typename XT, typename DT>
static int rmsnorm_bw_run(cudaStream_t st, const float* dy, const XT* x, const float* inv_rms, const float* gamma,
                          const float* residual, DT* dx, float* dgamma, int rows, int F, int group, float* partial) {
    int nparts;
    if (vec_ok(dy, x, dx, F, group) && ((uintptr_t)gamma & 15) == 0 && ((uintptr_t)residual & 15) == 0 && F / group <= sm_count() * 4) {
        int gpr = F / group;
        nparts = bw_parts_vec(rows, F, group);
        int grid = nparts * gpr, g4 = group / 4;
        size_t smem = (size_t)group * sizeof(float);
#define RUN(V, TPG) rmsnorm_bw_vec<V, TPG, XT, DT><<<grid, kWarpsPerCta * 32, smem, st>>>(dy, x, inv_rms, gamma, residual, dx, partial, rows, F, group)
        if (g4 <= 32) RUN(1, 32);
        else if (g4 <= 64) RUN(2, 32);
        else if (g4 <= 128) RUN(4, 32);
        else if (g4 <= 256) RUN(1, 256);
        else if (g4 <= 512) RUN(2, 256);
        else RUN(4, 256);
#undef RUN
        XL_LAUNCH_OK("rmsnorm_bw_vec");
    } else {
        long long ngroups = (long long)rows * (F / group);
        long long nb = (ngroups + 7) / 8;
        int maxb = sm_count() * 8;
        rmsnorm_bw_gen<XT, DT><<<(int)(nb < maxb ? nb : maxb), 256, 0, st>>>(dy, x, inv_rms, gamma, residual, dx, ngroups, F, group);
        XL_LAUNCH_OK("rmsnorm_bw_gen");
        nparts = bw_parts_gen(rows);
        int rpp = (rows + nparts - 1) / nparts;
        nparts = (rows + rpp - 1) / rpp;
        dim3 grid((F + 127) / 128, nparts);
        colsum_mul_gen<XT><<<grid, 128, 0, st>>>(dy, x, inv_rms, partial, rows, F, group, rpp);
        XL_LAUNCH_OK("colsum_mul_gen");
    }
    merge_parts8<<<(F + 31) / 32, 256, 0, st>>>(partial, dgamma, nparts, F);
    XL_LAUNCH_OK("colsum_merge");
    return XLSTM_OK;
}

extern "C" int xlstm_rmsnorm_bw(void* stream, const float* dy, const void* x, int x_dtype, const float* inv_rms,
                                const float* gamma, const float* residual, void* dx, int dx_dtype, float* dgamma,
                                int rows, int F, int group, void* workspace, size_t workspace_bytes) {
    XL_CHECK_ARG(dy && x && inv_rms && gamma && dx && dgamma, "rmsnorm_bw: null pointer");
    XL_CHECK_ARG(rows >= 0 && F > 0 && group > 0 && F % group == 0, "rmsnorm_bw: group %d does not divide width %d", group, F);
    XL_CHECK_ARG((x_dtype == XLSTM_F32 || x_dtype == XLSTM_BF16) && (dx_dtype == XLSTM_F32 || dx_dtype == XLSTM_BF16),
                 "rmsnorm_bw: unknown storage type");
    if (rows == 0) return XLSTM_OK;
    if (!workspace || workspace_bytes < xlstm_rmsnorm_bw_workspace_bytes(rows, F)) {
        set_error("rmsnorm_bw: workspace of %zu B is smaller than the %zu B required", workspace_bytes,
                  xlstm_rmsnorm_bw_workspace_bytes(rows, F));
        return XLSTM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* partial = (float*)workspace;
    if (x_dtype == XLSTM_F32)
        return dx_dtype == XLSTM_F32
                   ? rmsnorm_bw_run(st, dy, (const float*)x, inv_rms, gamma, residual, (float*)dx, dgamma, rows, F, group, partial)
                   : rmsnorm_bw_run(st, dy, (const float*)x, inv_rms, gamma, residual, (bf16*)dx, dgamma, rows, F, group, partial);
    return dx_dtype == XLSTM_F32
               ? rmsnorm_bw_run(st, dy, (const bf16*)x, inv_rms, gamma, residual, (float*)dx, dgamma, rows, F, group, partial)
               : rmsnorm_bw_run(st, dy, (const bf16*)x, inv_rms, gamma, residual, (bf16*)dx, dgamma, rows, F, group, partial);
}
