// Chunkwise mLSTM core on the Blackwell tensor cores (tcgen05 + TMEM, operands staged by TMA).
//
// Shape covered: dqk = dhv = 128, chunk L = 64, bf16 storage (the configuration the layer
// benchmark is quoted on). One CTA owns one (batch, head) pair and walks its chunks in order;
// the matrix memory C (forward) / its gradient dC (backward) lives in tensor memory for the
// whole call as a 128 x 128 fp32 accumulator, so chunk states never make an HBM round trip
// inside a call — only the bf16 record of the state entering each chunk is written for the
// backward to read.
//
// All contractions are bf16 x bf16 -> fp32 tcgen05.mma; gate, stabiliser and normaliser math is
// fp32 on the CUDA cores. Position-indexed accumulators use M = 64 tiles whose two column halves
// are interleaved on the TMEM lanes (half 0 on lanes 0-15 of each 32-lane quadrant, half 1 on
// lanes 16-31), so thread (row, half) of a warp owns one row-half and every per-row scale
// (1/psi_t, b_t, a_j) is a per-thread scalar in the epilogue.
//
// Math: src/gpu/cuda/mlstm_fused.cu:12-19 (forward), :830-858 (backward); the gate gradients use
// the identity dF_r = dq_r.q_r - dk_r.k_r, d(i)_r = dk_r.k_r, which equals the reference's
// row/column-sum form term by term (checked against the CPU oracle in tests/).
#include <cuda.h>

#include "common.cuh"
#include "mlstm.cuh"
#include "tc.cuh"

namespace xl {

using namespace tc;

__device__ int g_tc_status = 0;  // 0 ok, else the code of the first wait that ran out of budget

static constexpr int D = 128;        // dqk = dhv
static constexpr int L = 64;         // chunk length
static constexpr int kThreads = 128;
static constexpr uint32_t kTileBytes = L * D * 2;   // 16 KB: one [64 x 128] bf16 tile = two 8 KB boxes
static constexpr uint32_t kBoxBytes = L * 128;      // 8 KB: [64 rows x 64 cols]
static constexpr uint32_t kStateBox = D * 128;      // 16 KB: [128 rows x 64 cols]

// Inclusive scans over the 64 positions of a chunk held by threads 0..63 (warps 0 and 1).
// `xchg` is a 4-float shared scratch. All 128 threads must call (contains __syncthreads).
__device__ __forceinline__ float scan64_add(float x, float* xchg, bool reverse) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!reverse) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            float y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        if (warp < 2 && lane == 31) xchg[warp] = x;
        __syncthreads();
        if (warp == 1) x += xchg[0];
    } else {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            float y = __shfl_down_sync(0xffffffffu, x, o);
            if (lane + o < 32) x += y;
        }
        if (warp < 2 && lane == 0) xchg[warp] = x;
        __syncthreads();
        if (warp == 0) x += xchg[1];
    }
    __syncthreads();
    return x;
}
__device__ __forceinline__ float scan64_max(float x, float* xchg) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x = fmaxf(x, y);
    }
    if (warp < 2 && lane == 31) xchg[warp] = x;
    __syncthreads();
    if (warp == 1) x = fmaxf(x, xchg[0]);
    __syncthreads();
    return x;
}

// Per-chunk gate vectors in shared memory.
struct Gates {
    float rowt[L];  // fc_t - m_t
    float colt[L];  // i_j - fc_j   (-inf past the end of a ragged chunk)
    float m[L];
    float b[L];
    float a[L];
    float fg[L];
    float g;        // exp(fc_L + m_prev - m_L)
    float mlast;
    float pad[2];
};

// ---------------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------------
struct TcFwParams {
    CUtensorMap tmq, tmk, tmv;  // [B][T][H*128] bf16, box {64 cols, 64 rows, 1}
    const float *ig, *fg;
    const float *cC, *cn, *cm;
    bf16* ytil;
    float *msv, *psiv, *qnv;
    bf16* savedC;   // [BH][NC+1][128][128]
    float* savedn;  // [BH][NC+1][128]
    float *oC, *on, *om;
    int B, H, T, NC;
    long long* prof;  // optional: per-phase cycle counts of CTA 0 (development aid; null in production)
};

struct FwSmem {
    // offsets from the 1024-aligned base
    static constexpr uint32_t q0 = 0;                       // 2 stages x (Q, K, V)
    static constexpr uint32_t va = 6 * kTileBytes;          // a (.) V
    static constexpr uint32_t cb = va + kTileBytes;         // bf16 C_k, [128 x 128]
    static constexpr uint32_t p = cb + 2 * kStateBox;       // P, [64 x 64]
    static constexpr uint32_t gates = p + kBoxBytes;        // 2 x Gates
    static constexpr uint32_t nvec = gates + 2 * sizeof(Gates);
    static constexpr uint32_t misc = nvec + D * 4;          // barriers etc.
    static constexpr uint32_t total = misc + 256;
};

// Forward-direction gates of chunk `ch` into *G. m_prev is the stabiliser entering the chunk.
// All threads call. Writes msv-independent data only.
__device__ __forceinline__ void fw_gates(const TcFwParams& p, int b, int h, int ch, float m_prev, Gates* G, float* xchg) {
    const int tid = threadIdx.x;
    const int t0 = ch * L, Lc = min(L, p.T - t0);
    float lf = 0.f, iv = -INFINITY, fraw = 0.f;
    if (tid < Lc) {
        size_t gi = ((size_t)b * p.T + t0 + tid) * p.H + h;
        fraw = p.fg[gi];
        lf = log_sigmoid(fraw);
        iv = p.ig[gi];
    }
    float fc = scan64_add(lf, xchg, false);
    float u = scan64_max(iv - fc, xchg + 2);
    if (tid < L) {
        float mt = fc + fmaxf(m_prev, u);
        G->rowt[tid] = fc - mt;
        G->colt[tid] = iv - fc;
        G->m[tid] = mt;
        G->b[tid] = expf(fc + m_prev - mt);
        G->fg[tid] = fraw;
        if (tid == L - 1) {
            G->g = expf(fc + m_prev - mt);
            G->mlast = mt;
            xchg[0] = fc;
            xchg[1] = mt;
        }
    }
    __syncthreads();
    if (tid < L) G->a[tid] = expf(xchg[0] - fc + iv - xchg[1]);  // exp(-inf) = 0 past a ragged end
    __syncthreads();
}

__global__ void __launch_bounds__(kThreads, 1) mlstm_fw_tc(const __grid_constant__ TcFwParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
    const int row = 16 * warp + (lane & 15), hf = lane >> 4;  // M=64 epilogue ownership

    Gates* G = (Gates*)(sm + FwSmem::gates);
    float* nvec = (float*)(sm + FwSmem::nvec);
    uint64_t* bars = (uint64_t*)(sm + FwSmem::misc);  // [0],[1] tile stages, [2] mma1, [3] mma2
    uint32_t* tmem_slot = (uint32_t*)(sm + FwSmem::misc + 64);
    int* abort_flag = (int*)(sm + FwSmem::misc + 72);
    float* xchg = (float*)(sm + FwSmem::misc + 96);  // 8 floats

    if (tid == 0) {
        mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[2], 1); mbar_init(&bars[3], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem + 0, tHi = tmem + 64, tHe = tmem + 128, tC = tmem + 256;
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;

    auto issue_tiles = [&](int ch, int stage) {
        unsigned char* base = sm + FwSmem::q0 + (uint32_t)stage * 3 * kTileBytes;
        mbar_expect_tx(&bars[stage], 3 * kTileBytes);
        for (int cbx = 0; cbx < 2; ++cbx) {
            tma_load_3d(base + 0 * kTileBytes + cbx * kBoxBytes, &p.tmq, &bars[stage], h * D + 64 * cbx, ch * L, b);
            tma_load_3d(base + 1 * kTileBytes + cbx * kBoxBytes, &p.tmk, &bars[stage], h * D + 64 * cbx, ch * L, b);
            tma_load_3d(base + 2 * kTileBytes + cbx * kBoxBytes, &p.tmv, &bars[stage], h * D + 64 * cbx, ch * L, b);
        }
    };
    if (tid == 0) issue_tiles(0, 0);

    // ---- initial state: n, m; C into TMEM (pre-scaled by g_0) and as bf16 into Cb + record slot 0
    float m_prev = p.cm ? p.cm[bh] : 0.f;
    nvec[tid] = p.cn ? p.cn[(size_t)bh * D + tid] : 0.f;
    fw_gates(p, b, h, 0, m_prev, &G[0], xchg);
    {
        const float g0 = G[0].g;
        unsigned char* cb = sm + FwSmem::cb;
        bf16* rec = p.savedC ? p.savedC + ((size_t)bh * (p.NC + 1) + 0) * D * D + (size_t)tid * D : nullptr;
        for (int c0 = 0; c0 < D; c0 += 32) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = p.cC ? p.cC[(size_t)bh * D * D + (size_t)tid * D + c0 + i] : 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 pk;
                pk.x = pack_bf16(v[8 * q + 0], v[8 * q + 1]); pk.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
                pk.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]); pk.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
                int col = c0 + 8 * q;
                *reinterpret_cast<uint4*>(cb + (col >> 6) * kStateBox + swz(tid, (col & 63) >> 3)) = pk;
                if (rec) *reinterpret_cast<uint4*>(rec + col) = pk;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= g0;
            tmem_st32(tC + lane_base + c0, v);
        }
        tmem_st_wait();
        if (p.savedn) p.savedn[((size_t)bh * (p.NC + 1) + 0) * D + tid] = nvec[tid];
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    constexpr uint32_t idS = instr_desc(64, 32, 0, 0);
    constexpr uint32_t idHe = instr_desc(64, 64, 0, 0);
    constexpr uint32_t idHi = instr_desc(64, 64, 0, 1);
    constexpr uint32_t idC = instr_desc(128, 128, 1, 1);

    bool ok = true;
#ifdef XL_TC_PROFILE
    long long tprev = clock64();
    long long pacc[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) pacc[i] = 0;
#define PROF(i) { long long tn = clock64(); pacc[i] += tn - tprev; tprev = tn; }
#else
#define PROF(i)
#endif
    for (int ch = 0; ch < p.NC; ++ch) {
        const int st = ch & 1;
        const int t0 = ch * L, Lc = min(L, p.T - t0);
        Gates* Gc = &G[st];
        unsigned char* sQ = sm + FwSmem::q0 + (uint32_t)st * 3 * kTileBytes;
        unsigned char* sK = sQ + kTileBytes;
        unsigned char* sV = sK + kTileBytes;
        unsigned char* sVa = sm + FwSmem::va;
        unsigned char* sCb = sm + FwSmem::cb;
        unsigned char* sP = sm + FwSmem::p;

        PROF(0)
        if (!mbar_wait(&bars[st], (ch >> 1) & 1)) { *abort_flag = 1; }
        PROF(1)
        // ---- Va = a (.) V, chunk-for-chunk in the tile's physical order
        for (int i = 0; i < 8; ++i) {
            uint32_t off = (uint32_t)(tid + kThreads * i) * 16;
            int j = (off & (kBoxBytes - 1)) >> 7;
            float aj = Gc->a[j];
            uint4 x = *reinterpret_cast<const uint4*>(sV + off);
            float2 f0 = unpack_bf16(x.x), f1 = unpack_bf16(x.y), f2 = unpack_bf16(x.z), f3 = unpack_bf16(x.w);
            x.x = pack_bf16(f0.x * aj, f0.y * aj); x.y = pack_bf16(f1.x * aj, f1.y * aj);
            x.z = pack_bf16(f2.x * aj, f2.y * aj); x.w = pack_bf16(f3.x * aj, f3.y * aj);
            *reinterpret_cast<uint4*>(sVa + off) = x;
        }
        fence_async_smem();
        __syncthreads();
        if (*abort_flag) { ok = false; break; }
        PROF(2)

        if (tid == 0) {
            tc_fence_after();
            if (ch + 1 < p.NC) issue_tiles(ch + 1, st ^ 1);
            const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sVa), aC = smem_u32(sCb);
            // S = Q K^T : two N=32 halves on interleaved lanes, K = 128 in 8 steps
            for (int hh = 0; hh < 2; ++hh)
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                    mma_ss(tS + ((uint32_t)(16 * hh) << 16), smem_desc(aQ + ko, 16, 1024),
                           smem_desc(aK + ko + hh * 32 * 128, 16, 1024), idS, ks > 0);
                }
            // He = Q C_k^T : halves over v (rows of Cb), K = c = 128
            for (int hh = 0; hh < 2; ++hh)
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t koq = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                    uint32_t koc = (ks >> 2) * kStateBox + (ks & 3) * 32 + hh * 64 * 128;
                    mma_ss(tHe + ((uint32_t)(16 * hh) << 16), smem_desc(aQ + koq, 16, 1024), smem_desc(aC + koc, 16, 1024),
                           idHe, ks > 0);
                }
            // C += (a.V)^T K : M = v (MN-major A), N = c (MN-major B), K = j = 64 in 4 steps of 16 rows
            for (int ks = 0; ks < 4; ++ks)
                mma_ss(tC, smem_desc(aV + ks * 2048, kBoxBytes, 1024), smem_desc(aK + ks * 2048, kBoxBytes, 1024), idC, 1);
            mma_commit(&bars[2]);
        }
        PROF(3)
        if (!mbar_wait(&bars[2], ch & 1)) { *abort_flag = 2; }
        tc_fence_after();
        PROF(4)

        // ---- S epilogue: decay mask, P (bf16, K-major tile), row sums, q.n, psi
        float ipsi, bt = Gc->b[row];
        {
            float s[32];
            tmem_ld32(tS + lane_base, s);
            tmem_ld_wait();
            const float rt = Gc->rowt[row];
            float rs = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                int j = 32 * hf + i;
                float d = (j <= row) ? __expf(rt + Gc->colt[j]) : 0.f;
                s[i] *= d;
                rs += s[i];
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 pk;
                pk.x = pack_bf16(s[8 * q + 0], s[8 * q + 1]); pk.y = pack_bf16(s[8 * q + 2], s[8 * q + 3]);
                pk.z = pack_bf16(s[8 * q + 4], s[8 * q + 5]); pk.w = pack_bf16(s[8 * q + 6], s[8 * q + 7]);
                *reinterpret_cast<uint4*>(sP + swz(row, 4 * hf + q)) = pk;
            }
            // q_t . n over this thread's 64 columns
            float qn = 0.f;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                uint4 x = *reinterpret_cast<const uint4*>(sQ + hf * kBoxBytes + swz(row, c8));
                const float* nn = nvec + 64 * hf + 8 * c8;
                float2 f0 = unpack_bf16(x.x), f1 = unpack_bf16(x.y), f2 = unpack_bf16(x.z), f3 = unpack_bf16(x.w);
                qn += f0.x * nn[0] + f0.y * nn[1] + f1.x * nn[2] + f1.y * nn[3] + f2.x * nn[4] + f2.y * nn[5] + f3.x * nn[6] + f3.y * nn[7];
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 16);
            qn += __shfl_xor_sync(0xffffffffu, qn, 16);
            const float qnt = rs + bt * qn;
            const float mt = Gc->m[row];
            const float psi = fmaxf(fabsf(qnt), expf(-mt));
            ipsi = 1.f / psi;
            if (hf == 0 && row < Lc) {
                size_t o = (size_t)bh * p.T + t0 + row;
                p.msv[o] = mt; p.psiv[o] = psi; p.qnv[o] = qnt;
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (*abort_flag) { ok = false; break; }
        PROF(5)

        if (tid == 0) {
            tc_fence_after();
            const uint32_t aP = smem_u32(sP), aV = smem_u32(sV);
            // Hi = P V : halves over v (V boxes), K = j = 64: A K-major in 4 steps of 32 B, B MN-major in steps of 16 rows
            for (int hh = 0; hh < 2; ++hh)
                for (int ks = 0; ks < 4; ++ks)
                    mma_ss(tHi + ((uint32_t)(16 * hh) << 16), smem_desc(aP + ks * 32, 16, 1024),
                           smem_desc(aV + hh * kBoxBytes + ks * 2048, kBoxBytes, 1024), idHi, ks > 0);
            mma_commit(&bars[3]);
        }

        PROF(6)
        // ---- while P V runs: record and advance n, gates of the next chunk, C pass
        {
            const float g = Gc->g;
            float acc = 0.f;
            const int cbx = tid >> 6, cc = tid & 63;
#pragma unroll 8
            for (int j = 0; j < L; ++j) {
                bf16 kv = *reinterpret_cast<const bf16*>(sK + cbx * kBoxBytes + swz(j, cc >> 3) + (cc & 7) * 2);
                acc += Gc->a[j] * __bfloat162float(kv);
            }
            float nn = g * nvec[tid] + acc;
            __syncthreads();  // every q.n read of the old n is done (same phase as the S epilogue above)
            nvec[tid] = nn;
            if (p.savedn) p.savedn[((size_t)bh * (p.NC + 1) + ch + 1) * D + tid] = nn;
        }
        PROF(7)
        m_prev = Gc->mlast;
        const bool last = (ch + 1 == p.NC);
        if (!last) fw_gates(p, b, h, ch + 1, m_prev, &G[st ^ 1], xchg);
        PROF(8)
        {
            const float gn = last ? 1.f : G[st ^ 1].g;
            bf16* rec = p.savedC ? p.savedC + ((size_t)bh * (p.NC + 1) + ch + 1) * D * D + (size_t)tid * D : nullptr;
            float* oc = (last && p.oC) ? p.oC + (size_t)bh * D * D + (size_t)tid * D : nullptr;
            for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                tmem_ld32(tC + lane_base + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 pk;
                    pk.x = pack_bf16(v[8 * q + 0], v[8 * q + 1]); pk.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
                    pk.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]); pk.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
                    int col = c0 + 8 * q;
                    *reinterpret_cast<uint4*>(sCb + (col >> 6) * kStateBox + swz(tid, (col & 63) >> 3)) = pk;
                    if (rec) *reinterpret_cast<uint4*>(rec + col) = pk;
                }
                if (oc) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(oc + c0 + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                if (!last) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= gn;
                    tmem_st32(tC + lane_base + c0, v);
                }
            }
            tmem_st_wait();
        }

        PROF(9)
        if (!mbar_wait(&bars[3], ch & 1)) { *abort_flag = 3; }
        tc_fence_after();
        PROF(10)
        // ---- H epilogue: y = (Hi + b_t He) / psi_t, this thread's 64 columns of its row
        {
            bf16* yrow = p.ytil + (((size_t)b * p.T + t0 + row) * p.H + h) * D + 64 * hf;
            for (int c0 = 0; c0 < 64; c0 += 32) {
                float hi[32], he[32];
                tmem_ld32(tHi + lane_base + c0, hi);
                tmem_ld32(tHe + lane_base + c0, he);
                tmem_ld_wait();
                if (row < Lc) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float y[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) y[i] = (hi[8 * q + i] + bt * he[8 * q + i]) * ipsi;
                        uint4 pk;
                        pk.x = pack_bf16(y[0], y[1]); pk.y = pack_bf16(y[2], y[3]);
                        pk.z = pack_bf16(y[4], y[5]); pk.w = pack_bf16(y[6], y[7]);
                        *reinterpret_cast<uint4*>(yrow + c0 + 8 * q) = pk;
                    }
                }
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (*abort_flag) { ok = false; break; }
        PROF(11)
    }
#undef PROF
#ifdef XL_TC_PROFILE
    if (p.prof && bh == 0 && tid == 0)
        for (int i = 0; i < 12; ++i) p.prof[i] = pacc[i];
#endif

    if (ok) {
        if (p.on) p.on[(size_t)bh * D + tid] = nvec[tid];
        if (p.om && tid == 0) p.om[bh] = m_prev;
    } else if (tid == 0) {
        atomicCAS(&g_tc_status, 0, 100 + *abort_flag);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

static long long* g_prof = nullptr;
extern "C" void xlstm_debug_set_prof(void* p) { g_prof = (long long*)p; }
long long* tc_debug_prof() { return g_prof; }
int* tc_status_ptr() {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_status) != cudaSuccess) return nullptr;
    return (int*)p;
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

bool mlstm_tc_supported(int L_, int dqk, int dhv, int dtype) {
    return L_ == L && dqk == D && dhv == D && dtype == XLSTM_BF16;
}

size_t mlstm_tc_saved_C_bytes(int BH, int NC) { return align_up((size_t)BH * (NC + 1) * D * D * sizeof(bf16), 256); }
size_t mlstm_tc_saved_n_bytes(int BH, int NC) { return align_up((size_t)BH * (NC + 1) * D * sizeof(float), 256); }

int mlstm_fw_tc_launch(cudaStream_t st, const MlstmFwArgs& a, void* saved) {
    if (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.ytil) & 15) {
        set_error("mlstm_fw (tensor-core path): q, k, v, ytil must be 16-byte aligned");
        return XLSTM_ERR_ARG;
    }
    TcFwParams p = {};
    if (!tc_make_map3(&p.tmq, a.q, a.B, a.T, a.H * D) || !tc_make_map3(&p.tmk, a.k, a.B, a.T, a.H * D) ||
        !tc_make_map3(&p.tmv, a.v, a.B, a.T, a.H * D)) {
        set_error("mlstm_fw: cuTensorMapEncodeTiled failed");
        return XLSTM_ERR_CUDA;
    }
    p.ig = a.ig; p.fg = a.fg; p.cC = a.cC; p.cn = a.cn; p.cm = a.cm;
    p.ytil = (bf16*)a.ytil; p.msv = a.msv; p.psiv = a.psiv; p.qnv = a.qnv;
    if (saved) {
        p.savedC = (bf16*)saved;
        p.savedn = (float*)((char*)saved + mlstm_tc_saved_C_bytes(a.B * a.H, a.NC));
    }
    p.oC = a.oC; p.on = a.on; p.om = a.om;
    p.B = a.B; p.H = a.H; p.T = a.T; p.NC = a.NC;
    p.prof = g_prof;
    size_t smem = FwSmem::total + 1024;
    XL_CUDA(cudaFuncSetAttribute(mlstm_fw_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mlstm_fw_tc<<<a.B * a.H, kThreads, smem, st>>>(p);
    XL_LAUNCH_OK("mlstm_fw_tc");
    return XLSTM_OK;
}

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
