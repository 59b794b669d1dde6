// Forward of the chunkwise mLSTM core on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Shape covered: dqk = dhv = 128, chunk L = 64, bf16 storage. One CTA owns one (batch, head) pair
// and walks its chunks in order; the matrix memory C lives in tensor memory for the whole call as a
// 128 x 128 fp32 accumulator, pre-scaled by the next chunk's decay in the same pass that emits its
// bf16 operand copy and the record the backward reads. Sixteen math warps own the epilogues, a
// control warp issues every TMA load and tcgen05.mma and computes the gate vectors one chunk ahead.
//
// Per chunk, with entering state (C, n, m_prev) (src/gpu/cuda/mlstm_fused.cu:12-19):
//   S = Q K^T ; P = Dbar . S ;  H^T[v,t] = sum_j V[j,v] P[t,j] + b_t sum_c C[v,c] Q[t,c]
//   qn_t = rowsum(P)_t + b_t (q_t . n) ; psi_t = max(|qn_t|, exp(-m_t)) ; ytil = H / psi
//   C' = g C + (a.V)^T K ; n' = g n + sum_j a_j k_j
// H is accumulated feature-major (M = 128 lanes = v, 64 columns = positions), which runs the
// tensor core at its full M and makes the global stores of ytil coalesced along v.
#include <cuda.h>

#include "common.cuh"
#include "mlstm.cuh"
#include "tc.cuh"

namespace xl {

using namespace tc;

int* tc_status_ptr();
bool tc_make_map3(CUtensorMap* m, const void* base, int B, int T, int W);
bool tc_make_map2(CUtensorMap* m, const void* base, uint64_t rows, int W, int box_rows);

namespace fw {

static constexpr int D = 128;
static constexpr int L = 64;
static constexpr int kMathWarps = 16;
static constexpr int kMathThreads = kMathWarps * 32;
static constexpr int kThreads = kMathThreads + 32;
static constexpr uint32_t kTileBytes = L * D * 2;
static constexpr uint32_t kBoxBytes = L * 128;
static constexpr uint32_t kStateBox = D * 128;

struct Gates {
    float rowt[L];  // fc_t - m_t
    float colt[L];  // i_j - fc_j  (-inf past a ragged end)
    float m[L];
    float b[L];
    float a[L];
    float g;        // exp(fc_L + m_prev - m_L)
    float pad[3];
};

struct Params {
    CUtensorMap tmq, tmk, tmv;
    CUtensorMap tmy;  // ytil [B][T][H*dhv] bf16, box {64, 64, 1}: the output tile is stored from shared memory
    CUtensorMap tmc;  // the bf16 C record as rows of 128: [sub-heads * (NC+1) * 128][128], box {64, 128} (when a record is kept)
    const float *ig, *fg;
    const float *cC, *cn, *cm;
    bf16* ytil;
    float *msv, *psiv, *qnv;
    bf16* savedC;   // [BH][NC+1][128][128]
    float* savedn;  // [BH][NC+1][128]
    float *oC, *on, *om;
    int B, H, T, NC;
    int states_only;  // 1: walk the state recurrence only (the backward's recompute pass)
    // Heads wider than 128 run as nq x nv sub-heads of 128 x 128, one CTA each: sub-head (qh, vh) takes
    // columns qh*128.. of q and k, vh*128.. of v, and owns block (vh, qh) of the matrix memory. The
    // numerator of the output is additive over qh and q.n likewise, so with nq > 1 the CTAs write
    // unnormalised partials (num, qnpart) and a small second kernel sums and normalises them.
    int nq, nv;
    float* num;     // [nq][B*T][H*nv*128] fp32 numerators (nq > 1 only)
    float* qnpart;  // [nq][B*H][T] partial q.n (nq > 1 only)
    int* status;
};

struct Smem {
    static constexpr uint32_t q0 = 0;                         // 2 stages x (Q, K, V)
    static constexpr uint32_t va = 6 * kTileBytes;            // a (.) V
    static constexpr uint32_t cb = va + kTileBytes;           // bf16 C_k, [128 x 128]
    static constexpr uint32_t p = cb + 2 * kStateBox;         // P, [64 x 64]
    static constexpr uint32_t gates = p + kBoxBytes;          // 2 x Gates
    static constexpr uint32_t nvec = gates + 2 * sizeof(Gates);  // n [128]
    static constexpr uint32_t npart = nvec + D * 4;           // n partial sums [4][128]
    static constexpr uint32_t rpart = npart + 4 * D * 4;      // row-sum partials [4][64]
    static constexpr uint32_t qn = rpart + 4 * L * 4;         // q.n [64]
    static constexpr uint32_t ipsi = qn + L * 4;              // 1/psi [64]
    static constexpr uint32_t misc = ipsi + L * 4;
    static constexpr uint32_t yt = (misc + 256 + 1023) & ~1023u;  // output tile [64 x 128] bf16 (two swizzled boxes)
    static constexpr uint32_t total = yt + kTileBytes;
};

__device__ __forceinline__ uint4 pack8(const float* v) {
    uint4 pk;
    pk.x = pack_bf16(v[0], v[1]); pk.y = pack_bf16(v[2], v[3]); pk.z = pack_bf16(v[4], v[5]); pk.w = pack_bf16(v[6], v[7]);
    return pk;
}

// Control warp: raw gate inputs of a chunk (two positions per lane), read one chunk ahead.
struct GateRaw {
    float fr[2], iv[2];
};
__device__ __forceinline__ void gates_load(const Params& p, int b, int h, int ch, GateRaw& r) {
    const int lane = threadIdx.x & 31;
    const int t0 = ch * L, Lc = min(L, p.T - t0);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        int t = lane + 32 * e;
        r.fr[e] = INFINITY;  // log_sigmoid(+inf) = 0
        r.iv[e] = -INFINITY;
        if (t < Lc) {
            size_t gi = ((size_t)b * p.T + t0 + t) * p.H + h;
            r.fr[e] = p.fg[gi];
            r.iv[e] = p.ig[gi];
        }
    }
}
// fc = cumsum(log sigmoid f); m_t = fc_t + max(m_prev, max_{j<=t}(i_j - fc_j)). Returns m of the last position.
__device__ __forceinline__ float gates_compute(const GateRaw& r, float m_prev, Gates* G) {
    const int lane = threadIdx.x & 31;
    float fc0 = log_sigmoid(r.fr[0]), fc1 = log_sigmoid(r.fr[1]);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float y0 = __shfl_up_sync(0xffffffffu, fc0, o), y1 = __shfl_up_sync(0xffffffffu, fc1, o);
        if (lane >= o) { fc0 += y0; fc1 += y1; }
    }
    fc1 += __shfl_sync(0xffffffffu, fc0, 31);
    float u0 = r.iv[0] - fc0, u1 = r.iv[1] - fc1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float y0 = __shfl_up_sync(0xffffffffu, u0, o), y1 = __shfl_up_sync(0xffffffffu, u1, o);
        if (lane >= o) { u0 = fmaxf(u0, y0); u1 = fmaxf(u1, y1); }
    }
    u1 = fmaxf(u1, __shfl_sync(0xffffffffu, u0, 31));
    const float m0 = fc0 + fmaxf(m_prev, u0), m1 = fc1 + fmaxf(m_prev, u1);
    const float fcL = __shfl_sync(0xffffffffu, fc1, 31), mL = __shfl_sync(0xffffffffu, m1, 31);
    float fc[2] = {fc0, fc1}, mt[2] = {m0, m1};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        int t = lane + 32 * e;
        G->rowt[t] = fc[e] - mt[e];
        G->colt[t] = r.iv[e] - fc[e];
        G->m[t] = mt[e];
        G->b[t] = expf(fc[e] + m_prev - mt[e]);
        G->a[t] = expf(fcL - fc[e] + r.iv[e] - mL);
    }
    if (lane == 0) G->g = expf(fcL + m_prev - mL);
    return mL;
}

// WIDE: heads split into sub-heads; the 128 x 128 instantiation folds all of that indexing away.
template <bool WIDE>
__global__ void __launch_bounds__(kThreads, 1) mlstm_fw_tc(const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_ctrl = warp == kMathWarps;
    const int nq = WIDE ? p.nq : 1, nv = WIDE ? p.nv : 1;
    const int nsub = nq * nv;
    const int sbh = blockIdx.x, bh = sbh / nsub, sub = sbh % nsub, qh = sub / nv, vh = sub % nv;
    const int b = bh / p.H, h = bh % p.H;
    const int qcol = (h * nq + qh) * D, vcol = (h * nv + vh) * D;  // first column of this sub-head in q/k and in v/ytil
    const int dqk = nq * D, dhv = nv * D;
    const bool unnorm = nq > 1;
    const int qd = warp & 3, cq = (warp >> 2) & 3;
    const uint32_t lane_base = (uint32_t)(32 * qd) << 16;
    const int x = 32 * qd + lane;            // lane of a 128-lane accumulator
    const int srow = 16 * qd + (lane & 15);  // row of the M = 64 tile S (lanes 0-15 of the quadrant)
    const int prow = 4 * warp + (lane >> 3), l8 = lane & 7;  // q.n pass: 8 lanes per position
    const bool full = !p.states_only;

    Gates* G = (Gates*)(sm + Smem::gates);
    float* nvec = (float*)(sm + Smem::nvec);
    float* npart = (float*)(sm + Smem::npart);
    float* rpart = (float*)(sm + Smem::rpart);
    float* sqn = (float*)(sm + Smem::qn);
    float* sipsi = (float*)(sm + Smem::ipsi);
    uint64_t* bars = (uint64_t*)(sm + Smem::misc);  // [0],[1] tile stages, [2] S, [3] S + He + dC, [4] Hi
    uint32_t* tmem_slot = (uint32_t*)(sm + Smem::misc + 64);
    int* abort_flag = (int*)(sm + Smem::misc + 72);
    unsigned char* sVa = sm + Smem::va;
    unsigned char* sCb = sm + Smem::cb;
    unsigned char* sP = sm + Smem::p;
    unsigned char* sY = sm + Smem::yt;

    if (tid == 0) {
        for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (is_ctrl) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem + 0, tHi = tmem + 64, tHe = tmem + 128, tC = tmem + 256;

    auto issue_tiles = [&](int ch, int stage) {
        unsigned char* base = sm + Smem::q0 + (uint32_t)stage * 3 * kTileBytes;
        mbar_expect_tx(&bars[stage], (full ? 3 : 2) * kTileBytes);
        for (int cbx = 0; cbx < 2; ++cbx) {
            if (full) tma_load_3d(base + 0 * kTileBytes + cbx * kBoxBytes, &p.tmq, &bars[stage], qcol + 64 * cbx, ch * L, b);
            tma_load_3d(base + 1 * kTileBytes + cbx * kBoxBytes, &p.tmk, &bars[stage], qcol + 64 * cbx, ch * L, b);
            tma_load_3d(base + 2 * kTileBytes + cbx * kBoxBytes, &p.tmv, &bars[stage], vcol + 64 * cbx, ch * L, b);
        }
    };

    // ---- prologue: gates of chunk 0, n, and C into TMEM (pre-scaled by g_0) + bf16 copy + record slot 0
    GateRaw graw;
    float m_prev = p.cm ? p.cm[bh] : 0.f;  // control warp carries the stabiliser chain
    if (is_ctrl) {
        if (lane == 0) issue_tiles(0, 0);
        gates_load(p, b, h, 0, graw);
        m_prev = gates_compute(graw, m_prev, &G[0]);
        if (p.NC > 1) gates_load(p, b, h, 1, graw);
    } else if (tid < D) {
        nvec[tid] = p.cn ? p.cn[(size_t)bh * dqk + qh * D + tid] : 0.f;
        if (p.savedn) p.savedn[((size_t)sbh * (p.NC + 1) + 0) * D + tid] = nvec[tid];
    }
    __syncthreads();
    if (!is_ctrl) {
        const float g0 = G[0].g;
        const int c0 = 32 * cq;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = p.cC ? p.cC[((size_t)bh * dhv + vh * D + x) * dqk + qh * D + c0 + i] : 0.f;
        bf16* rec = p.savedC ? p.savedC + ((size_t)sbh * (p.NC + 1) + 0) * D * D + (size_t)x * D + c0 : nullptr;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 pk = pack8(v + 8 * q);
            *reinterpret_cast<uint4*>(sCb + (cq >> 1) * kStateBox + swz(x, 4 * (cq & 1) + q)) = pk;
            if (rec) *reinterpret_cast<uint4*>(rec + 8 * q) = pk;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= g0;
        tmem_st32(tC + lane_base + c0, v);
        tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    const uint64_t dK_ = smem_desc(0, 16, 1024);
    const uint64_t dM1 = smem_desc(0, kBoxBytes, 1024);
    constexpr uint32_t id64_kk = instr_desc(64, 64, 0, 0);     // S
    constexpr uint32_t id_kk = instr_desc(128, 64, 0, 0);      // He^T = C Q^T
    constexpr uint32_t id_mk = instr_desc(128, 64, 1, 0);      // Hi^T = V^T P^T
    constexpr uint32_t id_mm128 = instr_desc(128, 128, 1, 1);  // dC = (a.V)^T K

    bool ok = true;
    for (int ch = 0; ch < p.NC; ++ch) {
        const int st = ch & 1;
        const int t0 = ch * L, Lc = min(L, p.T - t0);
        const bool last = (ch + 1 == p.NC);
        Gates* Gc = &G[st];
        unsigned char* sQ = sm + Smem::q0 + (uint32_t)st * 3 * kTileBytes;
        unsigned char* sK = sQ + kTileBytes;
        unsigned char* sV = sK + kTileBytes;

        // =============== phase 1: a.V copy and q.n (math) | next tiles (control) =======================
        if (is_ctrl) {
            if (lane == 0 && !last) issue_tiles(ch + 1, st ^ 1);
            if (!mbar_wait(&bars[st], (ch >> 1) & 1)) *abort_flag = 1;
        } else {
            if (!mbar_wait(&bars[st], (ch >> 1) & 1)) *abort_flag = 1;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t off = (uint32_t)(tid + kMathThreads * i) * 16;
                const float aj = Gc->a[(off & (kBoxBytes - 1)) >> 7];
                uint4 v4 = *reinterpret_cast<const uint4*>(sV + off);
                float2 f0 = unpack_bf16(v4.x), f1 = unpack_bf16(v4.y), f2 = unpack_bf16(v4.z), f3 = unpack_bf16(v4.w);
                v4.x = pack_bf16(f0.x * aj, f0.y * aj); v4.y = pack_bf16(f1.x * aj, f1.y * aj);
                v4.z = pack_bf16(f2.x * aj, f2.y * aj); v4.w = pack_bf16(f3.x * aj, f3.y * aj);
                *reinterpret_cast<uint4*>(sVa + off) = v4;
            }
            if (full) {
                // q_t . n : eight lanes per position, sixteen columns each
                float acc = 0.f;
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2) {
                    uint4 v4 = *reinterpret_cast<const uint4*>(sQ + (l8 >> 2) * kBoxBytes + swz(prow, 2 * (l8 & 3) + q2));
                    const float* nn = nvec + 16 * l8 + 8 * q2;
                    float2 f0 = unpack_bf16(v4.x), f1 = unpack_bf16(v4.y), f2 = unpack_bf16(v4.z), f3 = unpack_bf16(v4.w);
                    acc += f0.x * nn[0] + f0.y * nn[1] + f1.x * nn[2] + f1.y * nn[3] + f2.x * nn[4] + f2.y * nn[5] + f3.x * nn[6] + f3.y * nn[7];
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                if (l8 == 0) sqn[prow] = acc;
            }
            fence_async_smem();
        }
        __syncthreads();  // #1
        if (*abort_flag) { ok = false; break; }

        // =============== phase 2: MMAs (control) | S epilogue (math) ====================================
        if (is_ctrl) {
            if (lane == 0) {
                tc_fence_after();
                const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aVa = smem_u32(sVa), aC = smem_u32(sCb);
                if (full) {
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                        mma_ss(tS, desc_at(dK_, aQ + ko), desc_at(dK_, aK + ko), id64_kk, ks > 0);  // S = Q K^T
                    }
                    mma_commit(&bars[2]);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                        const uint32_t kc = (ks >> 2) * kStateBox + (ks & 3) * 32;
                        // He^T[v,t] = sum_c C[v,c] Q[t,c]
                        mma_ss(tHe, desc_at(dK_, aC + kc), desc_at(dK_, aQ + ko), id_kk, ks > 0);
                    }
                }
                // C += (a.V)^T K : M = v, N = c, K = j in 4 steps of 16 rows
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_ss(tC, desc_at(dM1, aVa + ks * 2048), desc_at(dM1, aK + ks * 2048), id_mm128, 1);
                mma_commit(&bars[3]);
            }
            __syncwarp();
            if (!last) {
                m_prev = gates_compute(graw, m_prev, &G[st ^ 1]);
                if (ch + 2 < p.NC) gates_load(p, b, h, ch + 2, graw);
            }
            if (lane == 0) tma_store_wait_read();  // the previous chunk's stores have read sCb and the output tile: phase 3 may overwrite them
        } else if (full) {
            if (!mbar_wait(&bars[2], ch & 1)) *abort_flag = 2;
            tc_fence_after();
            float s[16];
            tmem_ld16(tS + lane_base + 16 * cq, s);
            tmem_ld_wait();
            float rs = 0.f;
            {
                // branch-free and on all lanes (lanes 16-31 hold no rows of an M = 64 tile; their values are not stored)
                const float rt = Gc->rowt[srow];
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const float4 c4 = *reinterpret_cast<const float4*>(Gc->colt + 16 * cq + 4 * i4);
                    const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 4 * i4 + e, j = 16 * cq + i;
                        const float dbar = __expf((j <= srow) ? rt + cc[e] : -INFINITY);
                        s[i] *= dbar;
                        rs += s[i];
                    }
                }
            }
            if (lane < 16) {
                *reinterpret_cast<uint4*>(sP + swz(srow, 2 * cq)) = pack8(s);
                *reinterpret_cast<uint4*>(sP + swz(srow, 2 * cq + 1)) = pack8(s + 8);
                rpart[cq * L + srow] = rs;
            }
            fence_async_smem();
            tc_fence_before();
        }
        __syncthreads();  // #2
        if (*abort_flag) { ok = false; break; }

        // =============== phase 3: P V (control) | psi, state pass, n, H epilogue (math) ==================
        if (is_ctrl) {
            if (lane == 0 && full) {
                tc_fence_after();
                const uint32_t aP = smem_u32(sP), aV = smem_u32(sV);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)  // Hi^T[v,t] = sum_j V[j,v] P[t,j]
                    mma_ss(tHi, desc_at(dM1, aV + ks * 2048), desc_at(dK_, aP + ks * 32), id_mk, ks > 0);
                mma_commit(&bars[4]);
            }
            __syncwarp();
        } else {
            if (full && tid < L) {
                const float qn = rpart[tid] + rpart[L + tid] + rpart[2 * L + tid] + rpart[3 * L + tid] + Gc->b[tid] * sqn[tid];
                const float mt = Gc->m[tid];
                const float psi = fmaxf(fabsf(qn), expf(-mt));
                sipsi[tid] = unnorm ? 1.f : 1.f / psi;
                if (tid < Lc && vh == 0) {
                    const size_t o = (size_t)bh * p.T + t0 + tid;
                    if (unnorm) {
                        p.qnpart[(size_t)qh * p.B * p.H * p.T + o] = qn;
                        if (qh == 0) p.msv[o] = mt;
                    } else {
                        p.msv[o] = mt; p.psiv[o] = psi; p.qnv[o] = qn;
                    }
                }
            }
            {   // n partial over this quarter of the positions: sum_j a_j K[j,x]
                const uint32_t xoff = (uint32_t)(x >> 6) * kBoxBytes + (x & 7) * 2, xch8 = (x & 63) >> 3;
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int j = 16 * cq + i;
                    acc += Gc->a[j] * __bfloat162float(*reinterpret_cast<const bf16*>(sK + xoff + swz(j, xch8)));
                }
                npart[cq * D + x] = acc;
            }
            if (!mbar_wait(&bars[3], ch & 1)) *abort_flag = 3;
            tc_fence_after();
            {   // state pass: C_{k+1} -> bf16 operand copy + record (+ final state), then pre-scale by the next decay
                const int c0 = 32 * cq;
                const float gn = last ? 1.f : G[st ^ 1].g;
                float v[32];
                tmem_ld32(tC + lane_base + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q)  // the record of this state is stored from this copy by TMA, after the barrier
                    *reinterpret_cast<uint4*>(sCb + (cq >> 1) * kStateBox + swz(x, 4 * (cq & 1) + q)) = pack8(v + 8 * q);
                if (last && p.oC) {
                    float* oc = p.oC + ((size_t)bh * dhv + vh * D + x) * dqk + qh * D + c0;
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(oc + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                if (!last) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= gn;
                    tmem_st32(tC + lane_base + c0, v);
                    tmem_st_wait();
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kMathThreads) : "memory");  // npart, sipsi complete
            if (tid < D) {
                const float nn = Gc->g * nvec[tid] + (npart[tid] + npart[D + tid]) + (npart[2 * D + tid] + npart[3 * D + tid]);
                nvec[tid] = nn;
                if (p.savedn) p.savedn[((size_t)sbh * (p.NC + 1) + ch + 1) * D + tid] = nn;
            }
            if (full) {
                if (!mbar_wait(&bars[4], ch & 1)) *abort_flag = 4;
                tc_fence_after();
                float hi[16], he[16];
                tmem_ld16(tHi + lane_base + 16 * cq, hi);
                tmem_ld16(tHe + lane_base + 16 * cq, he);
                tmem_ld_wait();
                const size_t ystride = (size_t)p.H * dhv;
                const size_t yoff = ((size_t)b * p.T + t0 + 16 * cq) * ystride + vcol + x;
                const int nlive = min(16, Lc - 16 * cq);
                if (unnorm) {
                    float* no = p.num + (size_t)qh * p.B * p.T * ystride + yoff;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (i < nlive) no[(size_t)i * ystride] = hi[i] + Gc->b[16 * cq + i] * he[i];
                } else {
                    // into the shared output tile (feature x of positions 16*cq..+15); TMA stores it after the barrier
                    // and clips the rows past a ragged end
                    unsigned char* ydst = sY + (uint32_t)(x >> 6) * kBoxBytes + (x & 7) * 2;
                    const uint32_t xch8 = (x & 63) >> 3;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int pos = 16 * cq + i;
                        *reinterpret_cast<bf16*>(ydst + swz(pos, xch8)) = __float2bfloat16_rn((hi[i] + Gc->b[pos] * he[i]) * sipsi[pos]);
                    }
                }
            }
            fence_async_smem();
            tc_fence_before();
        }
        __syncthreads();  // #3
        if (*abort_flag) { ok = false; break; }
        if (tid == kMathThreads && (p.savedC || (full && !unnorm))) {
            if (p.savedC) {
                // record slot ch+1 <- the bf16 state copy, straight from shared memory (two 64-column boxes)
                const int row0 = (sbh * (p.NC + 1) + ch + 1) * D;
                tma_store_2d(&p.tmc, sCb, 0, row0);
                tma_store_2d(&p.tmc, sCb + kStateBox, 64, row0);
            }
            if (full && !unnorm) {
                tma_store_3d(&p.tmy, sY, vcol, t0, b);
                tma_store_3d(&p.tmy, sY + kBoxBytes, vcol + 64, t0, b);
            }
            tma_store_commit();
        }
    }
    if (tid == kMathThreads) tma_store_wait_all();

    if (ok) {
        if (p.on && tid < D && vh == 0) p.on[(size_t)bh * dqk + qh * D + tid] = nvec[tid];
        if (p.om && tid == kMathThreads && sub == 0) p.om[bh] = m_prev;
    } else if (tid == 0) {
        atomicCAS(p.status, 0, 100 + *abort_flag);
    }
    tc_fence_before();
    __syncthreads();
    if (is_ctrl) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// Sum of the sub-heads' numerators and q.n partials, normaliser, output: one warp per (position, head).
__global__ void __launch_bounds__(256) mlstm_fw_combine(const float* __restrict__ num, const float* __restrict__ qnpart,
                                                        const float* __restrict__ msv, bf16* __restrict__ ytil,
                                                        float* __restrict__ psiv, float* __restrict__ qnv, int B, int H,
                                                        int T, int dhv, int nq) {
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // (b*T + t)*H + h
    if (row >= (size_t)B * T * H) return;
    const int h = (int)(row % H);
    const size_t bt = row / H;
    const int t = (int)(bt % T), b = (int)(bt / T);
    const size_t o = ((size_t)b * H + h) * T + t;
    float qn = 0.f;
    for (int q = 0; q < nq; ++q) qn += qnpart[(size_t)q * B * H * T + o];
    const float psi = fmaxf(fabsf(qn), expf(-msv[o]));
    if (lane == 0) { psiv[o] = psi; qnv[o] = qn; }
    const float ipsi = 1.f / psi;
    const size_t plane = (size_t)B * T * H * dhv;
    for (int c = 4 * lane; c < dhv; c += 128) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < nq; ++q) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(num + (size_t)q * plane + row * dhv + c));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        uint2 pk;
        pk.x = pack_bf16(acc.x * ipsi, acc.y * ipsi);
        pk.y = pack_bf16(acc.z * ipsi, acc.w * ipsi);
        *reinterpret_cast<uint2*>(ytil + row * dhv + c) = pk;
    }
}

}  // namespace fw

size_t mlstm_tc_fw_workspace_bytes(int B, int H, int T, int dqk, int dhv) {
    const int nq = dqk / fw::D;
    if (nq <= 1) return 0;
    return align_up((size_t)nq * B * T * H * dhv * sizeof(float), 256) + align_up((size_t)nq * B * H * T * sizeof(float), 256);
}

int mlstm_fw_ws_launch(cudaStream_t st, const MlstmFwArgs& a, void* saved);  // 128 x 128 heads: the warp-specialised kernel

int mlstm_fw_tc_launch(cudaStream_t st, const MlstmFwArgs& a, void* saved, void* workspace, size_t workspace_bytes) {
    using namespace fw;
    if (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.ytil | (uintptr_t)saved) & 15) {
        set_error("mlstm_fw (tensor-core path): q, k, v, ytil and the state record must be 16-byte aligned");
        return XLSTM_ERR_ARG;
    }
    if (a.dqk == D && a.dhv == D) return mlstm_fw_ws_launch(st, a, saved);  // heads wider than 128 run below as sub-heads
    Params p = {};
    p.nq = a.dqk / D; p.nv = a.dhv / D;
    const int nsub = p.nq * p.nv;
    if (p.nq > 1 && !a.states_only) {
        const size_t need = mlstm_tc_fw_workspace_bytes(a.B, a.H, a.T, a.dqk, a.dhv);
        if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15)) {
            set_error("mlstm_fw: heads wider than 128 in q/k need a 16-byte aligned workspace of %zu B (got %zu)", need, workspace_bytes);
            return XLSTM_ERR_WORKSPACE;
        }
        p.num = (float*)workspace;
        p.qnpart = (float*)((char*)workspace + align_up((size_t)p.nq * a.B * a.T * a.H * a.dhv * sizeof(float), 256));
    }
    if (!tc_make_map3(&p.tmq, a.q, a.B, a.T, a.H * a.dqk) || !tc_make_map3(&p.tmk, a.k, a.B, a.T, a.H * a.dqk) ||
        !tc_make_map3(&p.tmv, a.v, a.B, a.T, a.H * a.dhv)) {
        set_error("mlstm_fw: cuTensorMapEncodeTiled failed");
        return XLSTM_ERR_CUDA;
    }
    p.ig = a.ig; p.fg = a.fg; p.cC = a.cC; p.cn = a.cn; p.cm = a.cm;
    p.ytil = (bf16*)a.ytil; p.msv = a.msv; p.psiv = a.psiv; p.qnv = a.qnv;
    if (!a.states_only && p.nq == 1 && !tc_make_map3(&p.tmy, a.ytil, a.B, a.T, a.H * a.dhv)) {
        set_error("mlstm_fw: cuTensorMapEncodeTiled failed for the output");
        return XLSTM_ERR_CUDA;
    }
    if (saved) {
        if (!tc_make_map2(&p.tmc, saved, (uint64_t)a.B * a.H * nsub * (a.NC + 1) * D, D, D)) {
            set_error("mlstm_fw: cuTensorMapEncodeTiled failed for the state record");
            return XLSTM_ERR_CUDA;
        }
        p.savedC = (bf16*)saved;
        p.savedn = (float*)((char*)saved + mlstm_tc_saved_C_bytes(a.B * a.H * nsub, a.NC));
    }
    p.oC = a.oC; p.on = a.on; p.om = a.om;
    p.B = a.B; p.H = a.H; p.T = a.T; p.NC = a.NC;
    p.states_only = a.states_only;
    p.status = tc_status_ptr();
    if (!p.status) { set_error("mlstm_fw: cannot resolve the device status word"); return XLSTM_ERR_CUDA; }
    // the opt-in to large dynamic shared memory is a per-device function attribute: one flag per device
    static std::atomic<bool> attr_set[64];
    const size_t smem = Smem::total + 1024;
    int dev = 0;
    XL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        XL_CUDA(cudaFuncSetAttribute(mlstm_fw_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        XL_CUDA(cudaFuncSetAttribute(mlstm_fw_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    if (nsub == 1) mlstm_fw_tc<false><<<a.B * a.H, kThreads, smem, st>>>(p);
    else mlstm_fw_tc<true><<<a.B * a.H * nsub, kThreads, smem, st>>>(p);
    XL_LAUNCH_OK("mlstm_fw_tc");
    if (p.nq > 1 && !a.states_only) {
        const size_t rows = (size_t)a.B * a.T * a.H;
        mlstm_fw_combine<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(p.num, p.qnpart, a.msv, (bf16*)a.ytil, a.psiv, a.qnv, a.B, a.H,
                                                                     a.T, a.dhv, p.nq);
        XL_LAUNCH_OK("mlstm_fw_combine");
    }
    return XLSTM_OK;
}

}  // namespace xl
