// Forward of the chunkwise mLSTM core for 128 x 128 heads as a warp-specialised pipeline (tcgen05 + TMEM + TMA).
//
// Same contract and arithmetic as the phase-synchronous forward (mlstm_tc_fw.cu; chunk algebra of
// src/gpu/cuda/mlstm_fused.cu:12-19): one CTA owns one (batch, head) pair, walks its chunks of 64 positions in
// order and keeps the matrix memory C in tensor memory for the whole call. What differs is how the work of a chunk is
// spread: instead of sixteen warps that run each phase together between block barriers, five groups of warps each own
// one kind of work and hand results to one another through mbarriers, so that the S epilogue of chunk k+1, the state
// pass that turns C_k into C_{k+1}, the output epilogue of chunk k and the loads of chunk k+2 run at the same time.
// Only the state recurrence C_k -> (MMA) -> state pass -> C_{k+1} is sequential.
//
//   warps 0-3   C group   state pass: C (TMEM, fp32) -> bf16 operand copy (+ record, + final state), x next decay
//   warps 4-7   H group   q.n and psi, then the output epilogue: (Hi + b He) / psi -> bf16 tile -> TMA store
//   warps 8-15  S group   S epilogue: P = Dbar . S (bf16 tile) and its row sums; the a-scaled copy of V one chunk ahead
//   warp 16     loads     TMA loads of Q, K, V two chunks ahead; gate vectors (cumulative log-sigmoid, stabiliser chain)
//   warp 17     MMA       every tcgen05.mma, issued from the converged warp
//   warps 18-19 n         n_{k+1} = g n_k + sum_j a_j k_j (half of the rows each; warp 19 carries the chain)
// (q_t . n, the normaliser psi and the per-position scalars the backward reads are the H group's, ahead of its epilogue)
//
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, every role leaves its loop (their own
// waits run out or see the flag), tensor memory is freed and the code of the first failed wait goes to the device
// status word.
#include <cuda.h>

#include "common.cuh"
#include "mlstm.cuh"
#include "tc.cuh"

namespace xl {

using namespace tc;

int* tc_status_ptr();
bool tc_make_map3(CUtensorMap* m, const void* base, int B, int T, int W);
bool tc_make_map2(CUtensorMap* m, const void* base, uint64_t rows, int W, int box_rows);

namespace fw2 {

static constexpr int D = 128;
static constexpr int L = 64;
static constexpr int kWarps = 20;
static constexpr int kThreads = kWarps * 32;
static constexpr uint32_t kTileBytes = L * D * 2;   // one 64 x 128 bf16 tile (two swizzled 64-column boxes)
static constexpr uint32_t kBoxBytes = L * 128;
static constexpr uint32_t kStateBox = D * 128;      // one 128-row x 64-column box of the bf16 state copy
static constexpr int kGateRing = 4;

struct Gates {
    float rowt[L];  // fc_t - m_t
    float colt[L];  // i_j - fc_j  (-inf past a ragged end)
    float m[L];
    float b[L];     // exp(fc_t + m_prev - m_t)
    float a[L];     // exp(fc_L - fc_j + i_j - m_L)
    float g;        // exp(fc_L + m_prev - m_L)
    float pad[3];
};

struct Params {
    CUtensorMap tmq, tmk, tmv;
    CUtensorMap tmy;  // ytil [B][T][H*128] bf16, box {64, 64, 1}
    CUtensorMap tmc;  // bf16 C record as rows of 128: [BH * (NC+1) * 128][128], box {64, 128}
    const float *ig, *fg;
    const float *cC, *cn, *cm;
    float *msv, *psiv, *qnv;
    bf16* savedC;   // [BH][NC+1][128][128] (nullptr: no record)
    float* savedn;  // [BH][NC+1][128]
    float *oC, *on, *om;
    int B, H, T, NC;
    int states_only;  // 1: the state recurrence only (no S, no outputs)
    // Packed mode (seg > 0): a "sequence" of this launch is npack independent sequences of seg <= 32 positions each laid
    // end to end (T = npack * seg <= 64: one chunk), none with a carry. Gate scans restart at every multiple of seg, the
    // decay mask is block-diagonal, the state stays zero, and msv / psiv / qnv keep the caller's [sequence][head][seg]
    // layout. A 9-position sequence then costs a seventh of a chunk tile instead of a whole one.
    int seg, npack;
    int* status;
};

// barrier indices ([n]: n consecutive barriers, indexed by chunk parity, or by chunk % 4 for the gate ring)
enum Bar {
    kFull = 0,       // [2] tiles of a stage have landed (TMA transaction bytes)
    kEmpty = 2,      // [2] everyone is done with a stage's tiles
    kGates = 4,      // [4] gate vectors of a chunk are in their ring slot
    kSFull = 8,      // [2] S accumulator written
    kSFree = 10,     // [2] S accumulator read out
    kPFull = 12,     // [2] P tile and row sums written
    kAVFull = 14,    // [2] a-scaled V written
    kCDone = 16,     // [2] C += (a V)^T K of a chunk has completed (and every MMA issued before it)
    kCReady = 18,    // state pass done: bf16 copy in shared memory, C in TMEM scaled for the chunk
    kHFull = 19,     // [2] Hi (and He) accumulators written
    kHFree = 21,     // [2] output epilogue of the chunk finished (q.n, 1/psi and the gate vectors no longer needed either)
    kNPart = 23,     // [2] the first half of the n update's row sum written
    kNReady = 25,    // [2] n entering the chunk written
    kNFree = 27,     // [2] q.n of the chunk no longer needs n
    kNumBars = 29
};

struct Smem {
    static constexpr uint32_t tiles = 0;                                   // 2 stages x (Q, K, V)
    static constexpr uint32_t va = tiles + 2 * 3 * kTileBytes;             // 2 x (a . V)
    static constexpr uint32_t cb = va + 2 * kTileBytes;                    // bf16 C_k, [128 x 128]
    static constexpr uint32_t p = cb + 2 * kStateBox;                      // 2 x P [64 x 64]
    static constexpr uint32_t yt = p + 2 * kBoxBytes;                      // 2 x output tile [64 x 128] bf16
    static constexpr uint32_t gates = yt + 2 * kTileBytes;                 // ring of gate vectors
    static constexpr uint32_t nvec = gates + kGateRing * sizeof(Gates);    // 2 x n [128]
    static constexpr uint32_t rpart = nvec + 2 * D * 4;                    // row-sum halves [2][2][64]
    static constexpr uint32_t ipsi = rpart + 2 * 2 * L * 4 + 2 * D * 4;    // 1/psi [2][64] (behind the n partials [2][128])
    static constexpr uint32_t bars = ipsi + 2 * L * 4;
    static constexpr uint32_t misc = bars + kNumBars * 8;                  // tmem slot, abort flag
    static constexpr uint32_t total = misc + 32;
};
static_assert(Smem::total + 1024 <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ uint4 pack8(const float* v) {
    uint4 pk;
    pk.x = pack_bf16(v[0], v[1]); pk.y = pack_bf16(v[2], v[3]); pk.z = pack_bf16(v[4], v[5]); pk.w = pack_bf16(v[6], v[7]);
    return pk;
}

// Gate vectors of one chunk by one warp (two positions per lane): fc = cumsum(log sigmoid f),
// m_t = fc_t + max(m_prev, max_{j<=t}(i_j - fc_j)). Returns m of the chunk's last position.
template <bool PACKED>
__device__ __forceinline__ float gates_compute(const Params& p, int b, int h, int ch, float m_prev, Gates* G) {
    const int lane = threadIdx.x & 31;
    const int t0 = ch * L, Lc = min(L, p.T - t0);
    float fr[2], iv[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int t = lane + 32 * e;
        fr[e] = INFINITY;  // log_sigmoid(+inf) = 0: positions past a ragged end leave fc unchanged
        iv[e] = -INFINITY;
        if (t < Lc) {
            const size_t gi = ((size_t)b * p.T + t0 + t) * p.H + h;
            fr[e] = p.fg[gi];
            iv[e] = p.ig[gi];
        }
    }
    const int seg = PACKED ? p.seg : 0;  // packed mode: every sequence of the tile starts from the empty state (m_prev = 0 here)
    float fc0 = log_sigmoid(fr[0]), fc1 = log_sigmoid(fr[1]);
    seg_prefix64<false>(fc0, fc1, lane, seg);
    float u0 = iv[0] - fc0, u1 = iv[1] - fc1;
    seg_prefix64<true>(u0, u1, lane, seg);
    const float m0 = fc0 + fmaxf(m_prev, u0), m1 = fc1 + fmaxf(m_prev, u1);
    const float fcL = __shfl_sync(0xffffffffu, fc1, 31), mL = __shfl_sync(0xffffffffu, m1, 31);
    const float fc[2] = {fc0, fc1}, mt[2] = {m0, m1};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int t = lane + 32 * e;
        G->rowt[t] = fc[e] - mt[e];
        G->colt[t] = iv[e] - fc[e];
        G->m[t] = mt[e];
        G->b[t] = expf(fc[e] + m_prev - mt[e]);
        G->a[t] = seg ? 0.f : expf(fcL - fc[e] + iv[e] - mL);  // packed: no state leaves the tile
    }
    if (lane == 0) G->g = seg ? 0.f : expf(fcL + m_prev - mL);
    return mL;
}

// Bounded wait that also gives up when another role has raised the CTA's abort flag.
// Called by all 32 lanes of a warp; the answer is the same on every lane, so a role never splits a warp on it.
__device__ __noinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    bool ok = false;
    for (int i = 0; i < kWaitBudget; ++i) {
        if (mbar_try_wait(bar, parity)) { ok = true; break; }
        if ((i & 255) == 255 && *abort_flag) break;
        if (i > 64) __nanosleep(32);
    }
    return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// chunk c uses barrier (base + c % 2) for the (c / 2)-th time
#define WS_WAIT2(base, c, code)                                                                   \
    if (!wait_or_abort(&bars[(base) + ((c) & 1)], (uint32_t)(((c) >> 1) & 1), abort_flag)) {      \
        if (*abort_flag == 0) *abort_flag = (code);                                               \
        break;                                                                                    \
    }
#define WS_WAIT_GATES(c, code)                                                                    \
    if (!wait_or_abort(&bars[kGates + ((c) & 3)], (uint32_t)(((c) >> 2) & 1), abort_flag)) {      \
        if (*abort_flag == 0) *abort_flag = (code);                                               \
        break;                                                                                    \
    }
#define WS_WAIT1(idx, c, code)                                                                    \
    if (!wait_or_abort(&bars[idx], (uint32_t)((c) & 1), abort_flag)) {                            \
        if (*abort_flag == 0) *abort_flag = (code);                                               \
        break;                                                                                    \
    }

// PACKED: the instantiation that packed launches use; the plain one carries none of their index arithmetic (the extra
// compare per element of the decay mask alone cost the forward 6 %).
template <bool PACKED>
__global__ void __launch_bounds__(kThreads, 1) mlstm_fw_ws(const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
    const int col0 = h * D;  // first column of this head in q, k, v, ytil
    const int NC = p.NC;
    const bool full = !p.states_only;

    Gates* G = (Gates*)(sm + Smem::gates);
    float* nvec = (float*)(sm + Smem::nvec);
    float* rpart = (float*)(sm + Smem::rpart);
    float* sipsi = (float*)(sm + Smem::ipsi);
    uint64_t* bars = (uint64_t*)(sm + Smem::bars);
    uint32_t* tmem_slot = (uint32_t*)(sm + Smem::misc);
    volatile int* abort_flag = (volatile int*)(sm + Smem::misc + 8);
    unsigned char* sCb = sm + Smem::cb;

    if (tid == 0) {
        // arrivals per phase. A stage's tiles are released by the MMA warp's commit, the eight S-group warps (they
        // read V), the two n warps (K) and, with outputs, the four H-group warps (Q).
        const uint32_t e = full ? 15u : 11u;
        const uint32_t cnt[kNumBars] = {1, 1, e, e, 1, 1, 1, 1, 1, 1, 8, 8, 8, 8, 8, 8, 1, 1, 4, 1, 1, 4, 4, 1, 1, 1, 1, 4, 4};
        for (int i = 0; i < kNumBars; ++i) mbar_init(&bars[i], cnt[i]);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 17) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem + 0, tHi = tmem + 128, tHe = tmem + 256, tC = tmem + 384;  // S, Hi, He: two buffers of 64 columns each

    if (warp == 16) {
        // ================= loads + gate vectors ==================================================================
        float m_prev = p.cm ? p.cm[bh] : 0.f;
        int c = 0;
        for (; c < NC; ++c) {
            const int s = c & 1;
            if (c >= 2) WS_WAIT2(kEmpty, c - 2, 11)
            if (lane == 0) {
                unsigned char* base = sm + Smem::tiles + (uint32_t)s * 3 * kTileBytes;
                mbar_expect_tx(&bars[kFull + s], (full ? 3 : 2) * kTileBytes);
                for (int cbx = 0; cbx < 2; ++cbx) {
                    if (full) tma_load_3d(base + 0 * kTileBytes + cbx * kBoxBytes, &p.tmq, &bars[kFull + s], col0 + 64 * cbx, c * L, b);
                    tma_load_3d(base + 1 * kTileBytes + cbx * kBoxBytes, &p.tmk, &bars[kFull + s], col0 + 64 * cbx, c * L, b);
                    tma_load_3d(base + 2 * kTileBytes + cbx * kBoxBytes, &p.tmv, &bars[kFull + s], col0 + 64 * cbx, c * L, b);
                }
            }
            m_prev = gates_compute<PACKED>(p, b, h, c, m_prev, &G[c & 3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kGates + (c & 3)]);
        }
        if (c == NC && p.om && lane == 0) p.om[bh] = m_prev;
    } else if (warp == 17) {
        // ================= MMA issue ===============================================================================
        const uint64_t dK_ = smem_desc(0, 16, 1024);          // K-major operand
        const uint64_t dM1 = smem_desc(0, kBoxBytes, 1024);   // MN-major operand over a 64-row tile
        constexpr uint32_t id64_kk = instr_desc(64, 64, 0, 0);     // S = Q K^T
        constexpr uint32_t id_kk = instr_desc(128, 64, 0, 0);      // He^T = C Q^T
        constexpr uint32_t id_mk = instr_desc(128, 64, 1, 0);      // Hi^T = V^T P^T
        constexpr uint32_t id_mm128 = instr_desc(128, 128, 1, 1);  // C += (a.V)^T K
        const uint32_t aTiles = smem_u32(sm + Smem::tiles), aVa0 = smem_u32(sm + Smem::va), aC = smem_u32(sCb),
                       aP0 = smem_u32(sm + Smem::p);
        auto issue_S = [&](int c) {
            const uint32_t aQ = aTiles + (uint32_t)(c & 1) * 3 * kTileBytes, aK = aQ + kTileBytes;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                mma_ss_w(tS + 64 * (c & 1), desc_at(dK_, aQ + ko), desc_at(dK_, aK + ko), id64_kk, ks > 0);
            }
            mma_commit_w(&bars[kSFull + (c & 1)]);
        };
        // iteration k: the state products of chunk k, S of chunk k + 1, then P V of chunk k; k = -1 only issues S of chunk 0.
        // One call site for each group of instructions: the kernel's code size matters (seven roles share the
        // instruction caches).
        for (int k = full ? -1 : 0; k < NC; ++k) {
            const int s = k & 1;
            const uint32_t aQ = aTiles + (uint32_t)s * 3 * kTileBytes, aK = aQ + kTileBytes, aV = aK + kTileBytes;
            const uint32_t aVa = aVa0 + (uint32_t)s * kTileBytes;
            if (k >= 0) {
                WS_WAIT1(kCReady, k, 22)
                if (full) {
                    if (k >= 2) WS_WAIT2(kHFree, k - 2, 23)
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {  // He^T[v,t] = sum_c C[v,c] Q[t,c]
                        const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                        const uint32_t kc = (ks >> 2) * kStateBox + (ks & 3) * 32;
                        mma_ss_w(tHe + 64 * s, desc_at(dK_, aC + kc), desc_at(dK_, aQ + ko), id_kk, ks > 0);
                    }
                } else {
                    WS_WAIT2(kFull, k, 24)
                }
                WS_WAIT2(kAVFull, k, 25)
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)  // C += (a.V)^T K : M = v, N = c, K = j in 4 steps of 16 rows
                    mma_ss_w(tC, desc_at(dM1, aVa + ks * 2048), desc_at(dM1, aK + ks * 2048), id_mm128, 1);
                mma_commit_w(&bars[kCDone + s]);
                if (!full) {
                    mma_commit_w(&bars[kEmpty + s]);
                    continue;
                }
            }
            if (k + 1 < NC) {
                WS_WAIT2(kFull, k + 1, 26)
                if (k + 1 >= 2) WS_WAIT2(kSFree, k - 1, 27)
                tc_fence_after();
                issue_S(k + 1);
            }
            if (k < 0) continue;
            WS_WAIT2(kPFull, k, 28)
            tc_fence_after();
            const uint32_t aP = aP0 + (uint32_t)s * kBoxBytes;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)  // Hi^T[v,t] = sum_j V[j,v] P[t,j]
                mma_ss_w(tHi + 64 * s, desc_at(dM1, aV + ks * 2048), desc_at(dK_, aP + ks * 32), id_mk, ks > 0);
            mma_commit_w(&bars[kHFull + s]);
            mma_commit_w(&bars[kEmpty + s]);
        }
    } else if (warp >= 8 && warp < 16) {
        // ================= S group: a-scaled V one chunk ahead, S epilogue =======================================
        const int stid = tid - 256, qd = warp & 3, half = (warp - 8) >> 2;
        const uint32_t lane_base = (uint32_t)(32 * qd) << 16;
        const int row = 16 * qd + (lane & 15);  // the M = 64 tile keeps row r on lane (r / 16) * 32 + r % 16
        // a-scaled copy of V for chunk c (the operand of the state update); returns false when a wait gave up
        auto scaled_v = [&](int c) -> bool {
            const int s = c & 1;
            bool ok = false;
            do {
                WS_WAIT_GATES(c, 31)
                WS_WAIT2(kFull, c, 32)
                if (c >= 2) WS_WAIT2(kCDone, c - 2, 33)  // the MMAs that read this buffer two chunks ago have completed
                ok = true;
            } while (false);
            if (!ok) return false;
            const Gates* Gc = &G[c & 3];
            const unsigned char* sV = sm + Smem::tiles + (uint32_t)s * 3 * kTileBytes + 2 * kTileBytes;
            unsigned char* sVa = sm + Smem::va + (uint32_t)s * kTileBytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t off = (uint32_t)(stid + 256 * i) * 16;
                const float aj = Gc->a[(off & (kBoxBytes - 1)) >> 7];
                uint4 v4 = *reinterpret_cast<const uint4*>(sV + off);
                float2 f0 = unpack_bf16(v4.x), f1 = unpack_bf16(v4.y), f2 = unpack_bf16(v4.z), f3 = unpack_bf16(v4.w);
                v4.x = pack_bf16(f0.x * aj, f0.y * aj); v4.y = pack_bf16(f1.x * aj, f1.y * aj);
                v4.z = pack_bf16(f2.x * aj, f2.y * aj); v4.w = pack_bf16(f3.x * aj, f3.y * aj);
                *reinterpret_cast<uint4*>(sVa + off) = v4;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars[kAVFull + s]); mbar_arrive(&bars[kEmpty + s]); }
            return true;
        };
        // iteration k: the S epilogue of chunk k (none for k = -1), then the scaled V of chunk k + 1. One call site each:
        // the kernel's code size matters (seven roles share the instruction caches)
        bool live = true;
        for (int k = -1; live && k < NC; ++k) {
            const int s = k & 1;
            if (full && k >= 0) {
                WS_WAIT2(kSFull, k, 34)
                tc_fence_after();
                float sv[32];
                tmem_ld32(tS + 64 * s + lane_base + 32 * half, sv);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[kSFree + s]);
                const Gates* Gc = &G[k & 3];  // its barrier was waited for by scaled_v(k)
                // branch-free and on all lanes (lanes 16-31 hold no rows of an M = 64 tile; their results are not stored):
                // the mask goes into the exponent's argument, exp(-inf) = 0
                float rs0 = 0.f, rs1 = 0.f;
                {
                    const float rt = Gc->rowt[row];
                    const int jmin = PACKED ? seg_first(row, p.seg) : 0;  // packed mode: the row's own sequence only
#pragma unroll
                    for (int i4 = 0; i4 < 8; ++i4) {
                        const float4 c4 = *reinterpret_cast<const float4*>(Gc->colt + 32 * half + 4 * i4);
                        const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = 4 * i4 + e, j = 32 * half + i;
                            const float dbar = __expf((j <= row && (!PACKED || j >= jmin)) ? rt + cc[e] : -INFINITY);
                            sv[i] *= dbar;
                            if (e & 1) rs1 += sv[i]; else rs0 += sv[i];
                        }
                    }
                }
                const float rs = rs0 + rs1;
                // the P buffer and the row sums of two chunks ago are free once that chunk's output epilogue has ended
                if (k >= 2) WS_WAIT2(kHFree, k - 2, 35)
                if (lane < 16) {
                    unsigned char* sP = sm + Smem::p + (uint32_t)s * kBoxBytes;
#pragma unroll
                    for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(sP + swz(row, 4 * half + q)) = pack8(sv + 8 * q);
                    rpart[(s * 2 + half) * L + row] = rs;
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[kPFull + s]);
            }
            if (k + 1 < NC) live = scaled_v(k + 1);
        }
    } else if (warp < 4) {
        // ================= C group: state pass ====================================================================
        const int x = 32 * warp + lane;  // row v of C held by this thread (lane x of the 128-lane accumulator)
        const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
        for (int k = 0; k <= NC; ++k) {  // pass k produces the state ENTERING chunk k (k = NC: the final state)
            const bool last = (k == NC);
            bool bad = false;
            if (k >= 1) bad = !wait_or_abort(&bars[kCDone + ((k - 1) & 1)], (uint32_t)(((k - 1) >> 1) & 1), abort_flag);
            if (!bad && !last) bad = !wait_or_abort(&bars[kGates + (k & 3)], (uint32_t)((k >> 2) & 1), abort_flag);
            // the record store of the previous pass has finished reading the bf16 copy
            if (p.savedC && k >= 1 && tid == 0) tma_store_wait_read();
            // one answer for the whole group (its sub-block barriers must be reached by all 128 threads or by none)
            if (named_barrier_or(1, 128, bad || *abort_flag != 0)) {
                if (*abort_flag == 0) *abort_flag = 41;
                break;
            }
            tc_fence_after();
            const float gk = last ? 1.f : G[k & 3].g;
#pragma unroll 1
            for (int q4 = 0; q4 < 4; ++q4) {
                const int c0 = 32 * q4;
                float v[32];
                if (k == 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = p.cC ? p.cC[((size_t)bh * D + x) * D + c0 + i] : 0.f;
                } else {
                    tmem_ld32(tC + lane_base + c0, v);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<uint4*>(sCb + (q4 >> 1) * kStateBox + swz(x, 4 * (q4 & 1) + q)) = pack8(v + 8 * q);
                if (last && p.oC) {
                    float* oc = p.oC + ((size_t)bh * D + x) * D + c0;
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(oc + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                if (!last) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= gk;
                    tmem_st32(tC + lane_base + c0, v);
                }
            }
            fence_async_smem();
            if (!last) {
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[kCReady]);
            }
            if (p.savedC) {
                named_barrier(1, 128);
                if (tid == 0) {
                    const int row0 = (bh * (NC + 1) + k) * D;
                    tma_store_2d(&p.tmc, sCb, 0, row0);
                    tma_store_2d(&p.tmc, sCb + kStateBox, 64, row0);
                    tma_store_commit();
                }
            }
        }
        if (tid == 0) tma_store_wait_all();
    } else if (warp < 8) {
        // ================= H group: q.n and psi, then the output epilogue =========================================
        const int hx = tid - 128;                     // feature v of this thread in the epilogue
        const uint32_t lane_base = (uint32_t)(32 * (warp - 4)) << 16;
        const uint32_t xoff = (uint32_t)(hx >> 6) * kBoxBytes + (hx & 7) * 2, xch8 = (hx & 63) >> 3;
        const int qt = hx >> 1, qhf = hx & 1;         // q.n: position qt, columns 64 * qhf .. + 63 (two threads per position)
        for (int k = 0; full && k < NC; ++k) {
            const int s = k & 1;
            const int t0 = k * L, Lc = min(L, p.T - t0);
            const Gates* Gc = &G[k & 3];
            bool bad = !wait_or_abort(&bars[kGates + (k & 3)], (uint32_t)((k >> 2) & 1), abort_flag);
            if (!bad) bad = !wait_or_abort(&bars[kFull + s], (uint32_t)((k >> 1) & 1), abort_flag);
            if (!bad) bad = !wait_or_abort(&bars[kNReady + s], (uint32_t)((k >> 1) & 1), abort_flag);
            float acc = 0.f;
            if (!bad) {
                const unsigned char* sQ = sm + Smem::tiles + (uint32_t)s * 3 * kTileBytes + (uint32_t)qhf * kBoxBytes;
                const float* nn = nvec + s * D + 64 * qhf;
#pragma unroll 2
                for (int cb = 0; cb < 8; ++cb) {
                    const float4 n0 = *reinterpret_cast<const float4*>(nn + 8 * cb), n1 = *reinterpret_cast<const float4*>(nn + 8 * cb + 4);
                    const uint4 v4 = *reinterpret_cast<const uint4*>(sQ + swz(qt, cb));
                    const float2 f0 = unpack_bf16(v4.x), f1 = unpack_bf16(v4.y), f2 = unpack_bf16(v4.z), f3 = unpack_bf16(v4.w);
                    acc += f0.x * n0.x + f0.y * n0.y + f1.x * n0.z + f1.y * n0.w + f2.x * n1.x + f2.y * n1.y + f3.x * n1.z + f3.y * n1.w;
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            if (lane == 0) { mbar_arrive(&bars[kNFree + s]); mbar_arrive(&bars[kEmpty + s]); }  // done with n and the Q tile
            if (!bad) bad = !wait_or_abort(&bars[kPFull + s], (uint32_t)((k >> 1) & 1), abort_flag);
            if (!bad && qhf == 0) {
                const float qn = rpart[(s * 2 + 0) * L + qt] + rpart[(s * 2 + 1) * L + qt] + Gc->b[qt] * acc;
                const float mt = Gc->m[qt];
                const float psi = fmaxf(fabsf(qn), expf(-mt));
                sipsi[s * L + qt] = 1.f / psi;
                if (qt < Lc) {
                    const size_t o = PACKED ? ((size_t)(b * p.npack + qt / p.seg) * p.H + h) * p.seg + qt % p.seg
                                           : (size_t)bh * p.T + t0 + qt;
                    p.msv[o] = mt; p.psiv[o] = psi; p.qnv[o] = qn;
                }
            }
            if (!bad) bad = !wait_or_abort(&bars[kHFull + s], (uint32_t)((k >> 1) & 1), abort_flag);
            // the store of two chunks ago has finished reading this output buffer
            if (hx == 0) tma_store_wait_read1();
            // one answer for the whole group; the barrier also publishes 1/psi to the group
            if (named_barrier_or(2, 128, bad || *abort_flag != 0)) {
                if (*abort_flag == 0) *abort_flag = 51;
                break;
            }
            tc_fence_after();
            const float* ips = sipsi + s * L;
            unsigned char* ydst = sm + Smem::yt + (uint32_t)s * kTileBytes + xoff;
#pragma unroll 1
            for (int q4 = 0; q4 < 4; ++q4) {
                float hi[16], he[16];
                tmem_ld16(tHi + 64 * s + lane_base + 16 * q4, hi);
                tmem_ld16(tHe + 64 * s + lane_base + 16 * q4, he);
                tmem_ld_wait();
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(Gc->b + 16 * q4 + 4 * i4);
                    const float4 p4 = *reinterpret_cast<const float4*>(ips + 16 * q4 + 4 * i4);
                    const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 4 * i4 + e, pos = 16 * q4 + i;
                        *reinterpret_cast<bf16*>(ydst + swz(pos, xch8)) = __float2bfloat16_rn((hi[i] + bb[e] * he[i]) * pp[e]);
                    }
                }
            }
            fence_async_smem();
            tc_fence_before();
            named_barrier(2, 128);
            if (hx == 0) {
                unsigned char* sY = sm + Smem::yt + (uint32_t)s * kTileBytes;
                tma_store_3d(&p.tmy, sY, col0, k * L, b);
                tma_store_3d(&p.tmy, sY + kBoxBytes, col0 + 64, k * L, b);
                tma_store_commit();
            }
            if (lane == 0) mbar_arrive(&bars[kHFree + s]);
        }
        if (hx == 0) tma_store_wait_all();
    } else if (warp == 18 || warp == 19) {
        // ================= n chain: n_{k+1} = g n_k + sum_j a_j k_j, rows 0-31 by warp 18, rows 32-63 and the chain by 19 ===
        const bool chain = warp == 19;
        const int c = 4 * lane;  // features c .. c + 3
        float* npart = rpart + 2 * 2 * L;  // [2][128] partial sums of warp 18 (behind the row-sum halves)
        float nv[4] = {0.f, 0.f, 0.f, 0.f};
        if (chain) {
#pragma unroll
            for (int i = 0; i < 4; ++i) nv[i] = p.cn ? p.cn[(size_t)bh * D + c + i] : 0.f;
            if (full) *reinterpret_cast<float4*>(nvec + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
            if (p.savedn) *reinterpret_cast<float4*>(p.savedn + ((size_t)bh * (NC + 1) + 0) * D + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
            __syncwarp();
            if (full && lane == 0) mbar_arrive(&bars[kNReady + 0]);
        }
        const uint32_t koff = (uint32_t)(lane >> 4) * kBoxBytes + (lane & 1) * 8, kch = (lane & 15) >> 1;
        const int j0 = chain ? 32 : 0;
        int k = 0;
        for (; k < NC; ++k) {
            const int s = k & 1;
            WS_WAIT_GATES(k, 71)
            WS_WAIT2(kFull, k, 72)
            const Gates* Gc = &G[k & 3];
            const unsigned char* sK = sm + Smem::tiles + (uint32_t)s * 3 * kTileBytes + kTileBytes + koff;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int j = j0; j < j0 + 32; ++j) {
                const uint2 v2 = *reinterpret_cast<const uint2*>(sK + swz(j, kch));
                const float aj = Gc->a[j];
                const float2 f0 = unpack_bf16(v2.x), f1 = unpack_bf16(v2.y);
                acc[0] += aj * f0.x; acc[1] += aj * f0.y; acc[2] += aj * f1.x; acc[3] += aj * f1.y;
            }
            if (!chain) {
                // the chain warp read this buffer two chunks ago before it released that chunk's tiles, and this chunk's
                // tiles could only land after that release
                *reinterpret_cast<float4*>(npart + s * D + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                __syncwarp();
                if (lane == 0) { mbar_arrive(&bars[kNPart + s]); mbar_arrive(&bars[kEmpty + s]); }
                continue;
            }
            WS_WAIT2(kNPart, k, 74)
            const float4 pp = *reinterpret_cast<const float4*>(npart + s * D + c);
            const float g = Gc->g;
            nv[0] = g * nv[0] + (pp.x + acc[0]); nv[1] = g * nv[1] + (pp.y + acc[1]);
            nv[2] = g * nv[2] + (pp.z + acc[2]); nv[3] = g * nv[3] + (pp.w + acc[3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kEmpty + s]);
            if (p.savedn) *reinterpret_cast<float4*>(p.savedn + ((size_t)bh * (NC + 1) + k + 1) * D + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
            if (full && k + 1 < NC) {
                const int s1 = (k + 1) & 1;
                if (k + 1 >= 2) WS_WAIT2(kNFree, k - 1, 73)   // q.n of chunk k-1 has read the buffer this overwrites
                *reinterpret_cast<float4*>(nvec + s1 * D + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[kNReady + s1]);
            }
        }
        if (chain && k == NC && p.on) *reinterpret_cast<float4*>(p.on + (size_t)bh * D + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
    }

    // ---- every role ends here -----------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicCAS(p.status, 0, 100 + *abort_flag);
    if (warp == 17) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace fw2

int mlstm_fw_ws_launch(cudaStream_t st, const MlstmFwArgs& a, void* saved) {
    using namespace fw2;
    Params p = {};
    if (!tc_make_map3(&p.tmq, a.q, a.B, a.T, a.H * a.dqk) || !tc_make_map3(&p.tmk, a.k, a.B, a.T, a.H * a.dqk) ||
        !tc_make_map3(&p.tmv, a.v, a.B, a.T, a.H * a.dhv)) {
        set_error("mlstm_fw: cuTensorMapEncodeTiled failed");
        return XLSTM_ERR_CUDA;
    }
    if (!a.states_only && !tc_make_map3(&p.tmy, a.ytil, a.B, a.T, a.H * a.dhv)) {
        set_error("mlstm_fw: cuTensorMapEncodeTiled failed for the output");
        return XLSTM_ERR_CUDA;
    }
    if (saved) {
        if (!tc_make_map2(&p.tmc, saved, (uint64_t)a.B * a.H * (a.NC + 1) * D, D, D)) {
            set_error("mlstm_fw: cuTensorMapEncodeTiled failed for the state record");
            return XLSTM_ERR_CUDA;
        }
        p.savedC = (bf16*)saved;
        p.savedn = (float*)((char*)saved + mlstm_tc_saved_C_bytes(a.B * a.H, a.NC));
    }
    p.ig = a.ig; p.fg = a.fg; p.cC = a.cC; p.cn = a.cn; p.cm = a.cm;
    p.msv = a.msv; p.psiv = a.psiv; p.qnv = a.qnv;
    p.oC = a.oC; p.on = a.on; p.om = a.om;
    p.B = a.B; p.H = a.H; p.T = a.T; p.NC = a.NC;
    p.states_only = a.states_only;
    p.seg = a.seg; p.npack = a.npack;
    if (a.seg && (a.NC != 1 || a.T != a.seg * a.npack || a.T > L || a.seg > 32 || a.cC || a.oC)) {
        set_error("mlstm_fw: packed mode takes npack * seg <= 64 positions per tile, seg <= 32, no carry and no state out");
        return XLSTM_ERR_ARG;
    }
    p.status = tc_status_ptr();
    if (!p.status) { set_error("mlstm_fw: cannot resolve the device status word"); return XLSTM_ERR_CUDA; }
    // the opt-in to large dynamic shared memory is a per-device function attribute: one flag per device
    static std::atomic<bool> attr_set[64];
    const size_t smem = Smem::total + 1024;
    int dev = 0;
    XL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        XL_CUDA(cudaFuncSetAttribute(mlstm_fw_ws<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        XL_CUDA(cudaFuncSetAttribute(mlstm_fw_ws<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    if (a.seg) mlstm_fw_ws<true><<<a.B * a.H, kThreads, smem, st>>>(p);
    else mlstm_fw_ws<false><<<a.B * a.H, kThreads, smem, st>>>(p);
    XL_LAUNCH_OK("mlstm_fw_ws");
    return XLSTM_OK;
}

}  // namespace xl
