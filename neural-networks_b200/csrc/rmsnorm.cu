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

// ---- vector path: group % 4 == 0 -----------------------------------------------------------
// A "team" of TPG threads (a warp, or the whole 256-thread CTA for wide groups) owns one
// (row, group) at a time; each thread holds VPL float4 of it in registers.
template <int TPG>
__device__ __forceinline__ float team_sum(float v, float* red) {
    if (TPG == 32) return warp_sum(v);
    return block_sum(v, red);
}

template <int VPL, int TPG>
__global__ void __launch_bounds__(kWarpsPerCta * 32) rmsnorm_fw_vec(
    const float* __restrict__ x, const float* __restrict__ gamma, float* __restrict__ y,
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
        const float4* xp = reinterpret_cast<const float4*>(x + row * F + (long long)gc * group);
        float4 r[VPL];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                r[i] = __ldcs(xp + idx);
                ss += r[i].x * r[i].x + r[i].y * r[i].y + r[i].z * r[i].z + r[i].w * r[i].w;
            }
        }
        ss = team_sum<TPG>(ss, red);
        const float inv = 1.f / sqrtf(ss / (float)group + eps);
        if (lane == 0) inv_rms[gi] = inv;
        const float4* gp = reinterpret_cast<const float4*>(gamma + (long long)gc * group);
        float4* yp = reinterpret_cast<float4*>(y + row * F + (long long)gc * group);
        float4* hp = x_hat ? reinterpret_cast<float4*>(x_hat + row * F + (long long)gc * group) : nullptr;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                float4 g = __ldg(gp + idx);
                float4 xh = make_float4(r[i].x * inv, r[i].y * inv, r[i].z * inv, r[i].w * inv);
                if (hp) __stcs(hp + idx, xh);
                __stcs(yp + idx, make_float4(g.x * xh.x, g.y * xh.y, g.z * xh.z, g.w * xh.w));
            }
        }
    }
}

// Backward: CTA c owns column group (c % gpr) and row slice (c / gpr); its teams stride
// over that slice's rows. partial [gridDim.x / gpr, F] receives the CTA's dgamma sums.
template <int VPL, int TPG>
__global__ void __launch_bounds__(kWarpsPerCta * 32) rmsnorm_bw_vec(
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ inv_rms,
    const float* __restrict__ gamma, float* __restrict__ dx, float* __restrict__ partial, int rows, int F,
    int group) {
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
        const float4* xp = reinterpret_cast<const float4*>(x + off);
        const float inv = inv_rms[row * gpr + gc];
        float4 d[VPL], xh[VPL];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4) {
                d[i] = __ldcs(dyp + idx);
                float4 xv = __ldcs(xp + idx);
                xh[i] = make_float4(xv.x * inv, xv.y * inv, xv.z * inv, xv.w * inv);
                float4 p = make_float4(d[i].x * xh[i].x, d[i].y * xh[i].y, d[i].z * xh[i].z, d[i].w * xh[i].w);
                acc[i].x += p.x; acc[i].y += p.y; acc[i].z += p.z; acc[i].w += p.w;
                s += gam[i].x * p.x + gam[i].y * p.y + gam[i].z * p.z + gam[i].w * p.w;
            }
        }
        s = team_sum<TPG>(s, red) / (float)group;
        float4* dxp = reinterpret_cast<float4*>(dx + off);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            int idx = i * TPG + lane;
            if (idx < g4)
                __stcs(dxp + idx, make_float4(inv * (gam[i].x * d[i].x - xh[i].x * s), inv * (gam[i].y * d[i].y - xh[i].y * s),
                                              inv * (gam[i].z * d[i].z - xh[i].z * s), inv * (gam[i].w * d[i].w - xh[i].w * s)));
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

// dgamma[c] += sum over parts (ascending) of partial[part][c]
__global__ void colsum_merge(const float* __restrict__ partial, float* __restrict__ dgamma, int nparts, int F) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= F) return;
    float s = 0.f;
    for (int p = 0; p < nparts; ++p) s += partial[(long long)p * F + c];
    dgamma[c] += s;
}

// ---- generic path: any group size -------------------------------------------------------
__global__ void rmsnorm_fw_gen(const float* __restrict__ x, const float* __restrict__ gamma, float* __restrict__ y,
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
        for (int i = lane; i < group; i += 32) ss += x[off + i] * x[off + i];
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)group + eps);
        if (lane == 0) inv_rms[gi] = inv;
        for (int i = lane; i < group; i += 32) {
            float xh = x[off + i] * inv;
            if (x_hat) x_hat[off + i] = xh;
            y[off + i] = gamma[goff + i] * xh;
        }
    }
}

__global__ void rmsnorm_bw_gen(const float* __restrict__ dy, const float* __restrict__ x,
                               const float* __restrict__ inv_rms, const float* __restrict__ gamma,
                               float* __restrict__ dx, long long ngroups, int F, int group) {
    const int lane = threadIdx.x & 31;
    const long long wglobal = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
    const int gpr = F / group;
    for (long long gi = wglobal; gi < ngroups; gi += wstride) {
        const long long off = (gi / gpr) * F + (gi % gpr) * group;
        const int goff = (int)(gi % gpr) * group;
        const float inv = inv_rms[gi];
        float s = 0.f;
        for (int i = lane; i < group; i += 32) s += gamma[goff + i] * dy[off + i] * (x[off + i] * inv);
        s = warp_sum(s) / (float)group;
        for (int i = lane; i < group; i += 32)
            dx[off + i] = inv * (gamma[goff + i] * dy[off + i] - (x[off + i] * inv) * s);
    }
}

// partial[part][c] = sum over the part's rows of dy*x*inv  (generic dgamma, stage 1)
__global__ void colsum_mul_gen(const float* __restrict__ dy, const float* __restrict__ x,
                               const float* __restrict__ inv_rms, float* __restrict__ partial, int rows, int F,
                               int group, int rows_per_part) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= F) return;
    const int gpr = F / group, gc = c / group;
    int r0 = blockIdx.y * rows_per_part, r1 = min(rows, r0 + rows_per_part);
    float s = 0.f;
    for (int r = r0; r < r1; ++r) s += dy[(long long)r * F + c] * x[(long long)r * F + c] * inv_rms[(long long)r * gpr + gc];
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

extern "C" int xlstm_rmsnorm_fw(void* stream, const float* x, const float* gamma, float* y, float* inv_rms,
                                float* x_hat, int rows, int F, int group, float eps) {
    XL_CHECK_ARG(x && gamma && y && inv_rms, "rmsnorm_fw: null pointer");
    XL_CHECK_ARG(rows >= 0 && F > 0 && group > 0 && F % group == 0, "rmsnorm_fw: group %d does not divide width %d", group, F);
    if (rows == 0) return XLSTM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    long long ngroups = (long long)rows * (F / group);
    int maxb = sm_count() * 8;
    if (vec_ok(x, y, x_hat, F, group) && ((uintptr_t)gamma & 15) == 0) {
        int g4 = group / 4;
        int teams = g4 <= 512 ? kWarpsPerCta : 1;  // forward: a warp keeps up to 2048 floats of a row in registers
        long long nb = (ngroups + teams - 1) / teams;
        int grid = (int)(nb < maxb ? nb : maxb);
#define RUN(V, TPG) rmsnorm_fw_vec<V, TPG><<<grid, kWarpsPerCta * 32, 0, st>>>(x, gamma, y, inv_rms, x_hat, ngroups, F, group, eps)
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
        rmsnorm_fw_gen<<<grid, 256, 0, st>>>(x, gamma, y, inv_rms, x_hat, ngroups, F, group, eps);
        XL_LAUNCH_OK("rmsnorm_fw_gen");
    }
    return XLSTM_OK;
}

extern "C" size_t xlstm_rmsnorm_bw_workspace_bytes(int rows, int F) {
    if (rows <= 0 || F <= 0) return 0;
    // enough for either path: parts <= max(4*SMs, 512)
    int parts = sm_count() * 4;
    if (parts < 512) parts = 512;
    return (size_t)parts * F * sizeof(float);
}

extern "C" int xlstm_rmsnorm_bw(void* stream, const float* dy, const float* x, const float* inv_rms,
                                const float* gamma, float* dx, float* dgamma, int rows, int F, int group,
                                void* workspace, size_t workspace_bytes) {
    XL_CHECK_ARG(dy && x && inv_rms && gamma && dx && dgamma, "rmsnorm_bw: null pointer");
    XL_CHECK_ARG(rows >= 0 && F > 0 && group > 0 && F % group == 0, "rmsnorm_bw: group %d does not divide width %d", group, F);
    if (rows == 0) return XLSTM_OK;
    if (!workspace || workspace_bytes < xlstm_rmsnorm_bw_workspace_bytes(rows, F)) {
        set_error("rmsnorm_bw: workspace of %zu B is smaller than the %zu B required", workspace_bytes,
                  xlstm_rmsnorm_bw_workspace_bytes(rows, F));
        return XLSTM_ERR_WORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* partial = (float*)workspace;
    int nparts;
    if (vec_ok(dy, x, dx, F, group) && ((uintptr_t)gamma & 15) == 0 && F / group <= sm_count() * 4) {
        int gpr = F / group;
        nparts = bw_parts_vec(rows, F, group);
        int grid = nparts * gpr, g4 = group / 4;
        size_t smem = (size_t)group * sizeof(float);
#define RUN(V, TPG) rmsnorm_bw_vec<V, TPG><<<grid, kWarpsPerCta * 32, smem, st>>>(dy, x, inv_rms, gamma, dx, partial, rows, F, group)
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
        rmsnorm_bw_gen<<<(int)(nb < maxb ? nb : maxb), 256, 0, st>>>(dy, x, inv_rms, gamma, dx, ngroups, F, group);
        XL_LAUNCH_OK("rmsnorm_bw_gen");
        nparts = bw_parts_gen(rows);
        int rpp = (rows + nparts - 1) / nparts;
        nparts = (rows + rpp - 1) / rpp;
        dim3 grid((F + 127) / 128, nparts);
        colsum_mul_gen<<<grid, 128, 0, st>>>(dy, x, inv_rms, partial, rows, F, group, rpp);
        XL_LAUNCH_OK("colsum_mul_gen");
    }
    colsum_merge<<<(F + 127) / 128, 128, 0, st>>>(partial, dgamma, nparts, F);
    XL_LAUNCH_OK("colsum_merge");
    return XLSTM_OK;
}
