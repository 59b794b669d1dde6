// Backward of the chunkwise mLSTM core on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Same shape contract as the forward (dqk = dhv = 128, L = 64, bf16 storage). One CTA owns one
// (batch, head) pair and walks its chunks right to left with dC resident in tensor memory as a
// 128 x 128 fp32 accumulator. Eight math warps own the epilogues (thread = one row-half-quarter
// of a position-indexed accumulator, or one row-half of dC); a ninth control warp issues every
// TMA load and tcgen05.mma and computes the gate vectors one chunk ahead.
//
// Per chunk, with entering state (C, n), leaving-state gradient (dC+, dn+), dN = dy/psi:
//   S = Q K^T, dds = dN V^T + dqn            ->  DS = Dbar.S, dS = Dbar.dds
//   dV = DS^T dN + a (K dC+^T)                   dQ = dS K + (b.dN) C + b dqn n
//   dK = dS^T Q + a (V dC+ + dn+)                dC = g dC+ + (b.dN)^T Q
//   d(i)_r = dK_r.K_r,  dF_r = dQ_r.Q_r - dK_r.K_r,  d(f)_j = (sum_{r>=j} dF_r)(1 - sigmoid(f_j))
// (src/gpu/cuda/mlstm_fused.cu:830-858 with the stabiliser held constant; the gate-gradient
// identity replaces the reference's row/column sums and is checked against the CPU oracle.)
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "mlstm.cuh"
#include "tc.cuh"

namespace xl {

using namespace tc;

int* tc_status_ptr();  // device address of the library's status word

namespace bw {

static constexpr int D = 128;
static constexpr int L = 64;
static constexpr int kMathWarps = 16;
static constexpr int kMathThreads = kMathWarps * 32;
static constexpr int kThreads = kMathThreads + 32;  // + 1 control warp
static constexpr uint32_t kTileBytes = L * D * 2;
static constexpr uint32_t kBoxBytes = L * 128;
static constexpr uint32_t kStateBox = D * 128;

struct Gates {
    float rowt[L];  // fc_t - m_t
    float colt[L];  // i_j - fc_j  (-inf past a ragged end)
    float b[L];
    float a[L];
    float fg[L];
    float emm[L];   // exp(-m_t), the floor of psi
    float g;
    float pad[3];
};

struct Params {
    CUtensorMap tmq, tmk, tmv;  // [B][T][H*128] bf16, box {64, 64, 1}
    CUtensorMap tmc;            // saved C: [BH*(NC+1)*128][128] bf16, box {64, 128}
    const float *ig, *fg;
    const float* cm;
    const bf16* ytil;
    const float *msv, *psiv, *qnv;
    const bf16* savedC;
    const float* savedn;
    const void* dy;
    const float *cdC, *cdn;
    void *dq, *dk, *dv;
    float *dig, *dfg;
    float *odC, *odn;
    int B, H, T, NC;
    int gbf16;
    // Heads wider than 128 run as nq x nv sub-heads of 128 x 128, one CTA each (see the forward kernel).
    // Every gradient is linear in the sub-heads' contributions once dN = dy/psi and dqn are formed from
    // the whole head, so the CTAs write fp32 partials and a second kernel sums them: dq, dk over vh
    // (planes `qk_plane` apart), dv over qh (`v_plane`), the gate gradients over all (`g_plane`). The
    // terms that belong to the normaliser branch (dqn) are taken by the vh = 0 sub-heads only.
    int nq, nv;
    const float* dotv;  // [B*H][T] dy_t . ytil_t over the whole head (nv > 1; else the CTA forms it itself)
    size_t qk_plane, v_plane, g_plane;
    // Packed mode (seg > 0), as in the forward kernel: npack independent sequences of seg positions per tile, one chunk,
    // no carry: segmented scans, block-diagonal decay mask, zero state; msv / psiv / qnv in [sequence][head][seg] order.
    int seg, npack;
    int* status;      // device status word (first bounded wait that ran out)
};

// Index of position t0 + t of (b, h) in msv / psiv / qnv (and dotv).
// (`seg` is the kernel's segment length: the compile-time 0 of the plain instantiations removes the packed arithmetic.)
__device__ __forceinline__ size_t vec_index(const Params& p, int b, int h, int bh, int pos, int seg) {
    return seg ? ((size_t)(b * p.npack + pos / seg) * p.H + h) * seg + pos % seg : (size_t)bh * p.T + pos;
}

static constexpr int kVecFloats = 3 * L + D;
struct Smem {
    static constexpr uint32_t q = 0;                       // 2 stages
    static constexpr uint32_t k = q + 2 * kTileBytes;      // 2 stages
    static constexpr uint32_t v = k + 2 * kTileBytes;
    static constexpr uint32_t ck = v + kTileBytes;         // [128 x 128] entering state, bf16
    static constexpr uint32_t dn_ = ck + 2 * kStateBox;    // dN  = dy/psi
    static constexpr uint32_t dnb = dn_ + kTileBytes;      // dNb = b . dN
    static constexpr uint32_t dcb = dnb + kTileBytes;      // bf16 dC+
    static constexpr uint32_t ds_ = dcb + 2 * kStateBox;   // DS  [64 x 64]
    static constexpr uint32_t dS = ds_ + kBoxBytes;        // dS  [64 x 64]
    static constexpr uint32_t gates = dS + kBoxBytes;      // 2 x Gates
    static constexpr uint32_t graw = gates + 2 * sizeof(Gates);   // 2 x GateRawS
    static constexpr uint32_t vec = graw + 2 * 784;  // 2 x [psi 64 | qn 64 | n entering the chunk 128 | dy.ytil 64]
    static constexpr uint32_t dnv = vec + 2 * kVecFloats * 4;             // dn, double buffered [2][128]
    static constexpr uint32_t dnp = dnv + 2 * D * 4;       // dn partial sums [4][128]
    static constexpr uint32_t part = dnp + 4 * D * 4;      // partial sums [12][64]: dot(4), u(4), w(4)
    static constexpr uint32_t dqn = part + 12 * L * 4;     // [64]
    static constexpr uint32_t misc = dqn + L * 4;
    static constexpr uint32_t total = misc + 256;
};

template <typename G>
__device__ __forceinline__ void load16(const G* p, float* v);
template <>
__device__ __forceinline__ void load16<float>(const float* p, float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 t = __ldcs(reinterpret_cast<const float4*>(p) + i);
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
}
template <>
__device__ __forceinline__ void load16<bf16>(const bf16* p, float* v) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 t = __ldcs(reinterpret_cast<const uint4*>(p) + i);
        float2 a = unpack_bf16(t.x), b = unpack_bf16(t.y), c = unpack_bf16(t.z), d = unpack_bf16(t.w);
        v[8 * i] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = b.x; v[8 * i + 3] = b.y;
        v[8 * i + 4] = c.x; v[8 * i + 5] = c.y; v[8 * i + 6] = d.x; v[8 * i + 7] = d.y;
    }
}
template <typename G>
__device__ __forceinline__ void store16(G* p, const float* v);
template <>
__device__ __forceinline__ void store16<float>(float* p, const float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        __stcs(reinterpret_cast<float4*>(p) + i, make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
}
template <>
__device__ __forceinline__ void store16<bf16>(bf16* p, const float* v) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 t;
        t.x = pack_bf16(v[8 * i], v[8 * i + 1]); t.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
        t.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]); t.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
        __stcs(reinterpret_cast<uint4*>(p) + i, t);
    }
}

__device__ __forceinline__ uint4 pack8(const float* v) {
    uint4 pk;
    pk.x = pack_bf16(v[0], v[1]); pk.y = pack_bf16(v[2], v[3]); pk.z = pack_bf16(v[4], v[5]); pk.w = pack_bf16(v[6], v[7]);
    return pk;
}
// N floats (N = 8 * chunks) -> swizzled 16-byte chunks of row `row`, starting at logical chunk `chunk0`.
template <int CHUNKS>
__device__ __forceinline__ void put_row(unsigned char* tile, uint32_t row, uint32_t chunk0, const float* v) {
#pragma unroll
    for (int q = 0; q < CHUNKS; ++q) *reinterpret_cast<uint4*>(tile + swz(row, chunk0 + q)) = pack8(v + 8 * q);
}
// dot of 16 floats with 16 bf16 of row `row` (chunks chunk0, chunk0+1) of a swizzled tile
__device__ __forceinline__ float dot_row16(const unsigned char* tile, uint32_t row, uint32_t chunk0, const float* v) {
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        uint4 x = *reinterpret_cast<const uint4*>(tile + swz(row, chunk0 + q));
        float2 f0 = unpack_bf16(x.x), f1 = unpack_bf16(x.y), f2 = unpack_bf16(x.z), f3 = unpack_bf16(x.w);
        acc += v[8 * q] * f0.x + v[8 * q + 1] * f0.y + v[8 * q + 2] * f1.x + v[8 * q + 3] * f1.y + v[8 * q + 4] * f2.x +
               v[8 * q + 5] * f2.y + v[8 * q + 6] * f3.x + v[8 * q + 7] * f3.y;
    }
    return acc;
}

// 4-byte asynchronous global -> shared copy (no register staging, no stall at issue).
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Raw gate inputs of one chunk as the control warp stages them in shared memory.
struct GateRawS {
    float fr[L], iv[L], mt[L];
    float m_prev;
    float pad[3];
};
// Control warp: start the asynchronous copy of a chunk's raw gate inputs (two positions per lane).
__device__ __forceinline__ void gates_fetch(const Params& p, int b, int h, int bh, int ch, GateRawS* r, int seg) {
    const int lane = threadIdx.x & 31;
    const int t0 = ch * L, Lc = min(L, p.T - t0);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        int t = lane + 32 * e;
        if (t < Lc) {
            size_t gi = ((size_t)b * p.T + t0 + t) * p.H + h;
            cp_async4(&r->fr[t], p.fg + gi);
            cp_async4(&r->iv[t], p.ig + gi);
        } else {
            r->fr[t] = INFINITY;   // log_sigmoid(+inf) = 0: positions past a ragged end leave fc unchanged
            r->iv[t] = -INFINITY;
        }
        cp_async4(&r->mt[t], p.msv + vec_index(p, b, h, bh, t0 + min(t, Lc - 1), seg));
    }
    if (lane == 0) {
        if (ch == 0) {
            if (p.cm) cp_async4(&r->m_prev, p.cm + bh); else r->m_prev = 0.f;
        } else {
            cp_async4(&r->m_prev, p.msv + (size_t)bh * p.T + t0 - 1);
        }
    }
}
// Control warp: gate vectors of a chunk from its staged raw inputs.
__device__ __forceinline__ void gates_compute(const GateRawS* r, Gates* G, int seg) {
    const int lane = threadIdx.x & 31;
    const float fr[2] = {r->fr[lane], r->fr[lane + 32]}, iv[2] = {r->iv[lane], r->iv[lane + 32]};
    const float mt[2] = {r->mt[lane], r->mt[lane + 32]};
    const float m_prev = r->m_prev;
    float fc0 = log_sigmoid(fr[0]), fc1 = log_sigmoid(fr[1]);
    seg_prefix64<false>(fc0, fc1, lane, seg);
    const float fcL = __shfl_sync(0xffffffffu, fc1, 31);
    const float mL = __shfl_sync(0xffffffffu, mt[1], 31);
    float fc[2] = {fc0, fc1};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        int t = lane + 32 * e;
        G->rowt[t] = fc[e] - mt[e];
        G->colt[t] = iv[e] - fc[e];
        G->b[t] = expf(fc[e] + m_prev - mt[e]);
        G->a[t] = seg ? 0.f : expf(fcL - fc[e] + iv[e] - mL);  // packed: no state crosses the tile
        G->fg[t] = fr[e];
        G->emm[t] = expf(-mt[e]);
    }
    if (lane == 0) G->g = seg ? 0.f : expf(fcL + m_prev - mL);
}
// Control warp: start the asynchronous copy of a chunk's psi, qn (64 each) and entering normaliser n (128)
// straight into their shared-memory slot [psi 64 | qn 64 | n 128].
__device__ __forceinline__ void vec_fetch(const Params& p, int bh, int sbh, int ch, float* dst, int seg) {
    const int lane = threadIdx.x & 31;
    const int t0 = ch * L, Lc = min(L, p.T - t0);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const size_t o = vec_index(p, bh / p.H, bh % p.H, bh, t0 + min(lane + 32 * e, Lc - 1), seg);
        cp_async4(dst + lane + 32 * e, p.psiv + o);
        cp_async4(dst + L + lane + 32 * e, p.qnv + o);
        if (p.dotv) cp_async4(dst + 2 * L + D + lane + 32 * e, p.dotv + o);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) cp_async4(dst + 2 * L + lane + 32 * e, p.savedn + ((size_t)sbh * (p.NC + 1) + ch) * D + lane + 32 * e);
}

// Sum 16 per-lane values across the 32 lanes of a warp with a reduce-scatter butterfly (16
// shuffles instead of 80). On return lane l holds, in the result, the warp-wide sum of element
// index ((l >> 1) & 15) remapped by `butterfly_index`.
__device__ __forceinline__ float butterfly16(float* v, int lane) {
    // stage xor 16: keep 8
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const bool up = lane & 16;
        float keep = up ? v[k + 8] : v[k], send = up ? v[k] : v[k + 8];
        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const bool up = lane & 8;
        float keep = up ? v[k + 4] : v[k], send = up ? v[k] : v[k + 4];
        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const bool up = lane & 4;
        float keep = up ? v[k + 2] : v[k], send = up ? v[k] : v[k + 2];
        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    {
        const bool up = lane & 2;
        float keep = up ? v[1] : v[0], send = up ? v[0] : v[1];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
    return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}
// Which of the 16 elements lane `lane` ends up holding after butterfly16.
__device__ __forceinline__ int butterfly_index(int lane) {
    return ((lane & 16) ? 8 : 0) + ((lane & 8) ? 4 : 0) + ((lane & 4) ? 2 : 0) + ((lane & 2) ? 1 : 0);
}

// GT: type of the upstream gradient dy; OT: type the gradients are written in (fp32 for sub-head partials).
// WIDE: heads split into sub-heads; the 128 x 128 instantiation folds all of that indexing away.
// PACKED: the instantiation packed launches use; in the others the segment length is the constant 0 and the segmented
// scans, the mask's second test and the vector index arithmetic fold away (left in, they cost the plain kernel 3 %).
template <typename GT, typename OT, bool WIDE, bool PACKED>
__global__ void __launch_bounds__(kThreads, 1) mlstm_bw_tc(const __grid_constant__ Params p) {
    const int seg = PACKED ? p.seg : 0;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_ctrl = warp == kMathWarps;
    const int nq = WIDE ? p.nq : 1, nv = WIDE ? p.nv : 1;
    const int nsub = nq * nv;
    const int sbh = blockIdx.x, bh = sbh / nsub, sub = sbh % nsub, qh = sub / nv, vh = sub % nv;
    const int b = bh / p.H, h = bh % p.H;
    const int qcol = (h * nq + qh) * D, vcol = (h * nv + vh) * D;
    const int dqk = nq * D, dhv = nv * D;
    const size_t qk_plane = WIDE ? p.qk_plane : 0, v_plane = WIDE ? p.v_plane : 0, g_plane = WIDE ? p.g_plane : 0;
    const float* dotv = WIDE ? p.dotv : nullptr;
    const bool once = vh == 0;  // this sub-head carries the normaliser-branch terms of its q/k columns
    const int qd = warp & 3, cq = (warp >> 2) & 3;
    const uint32_t lane_base = (uint32_t)(32 * qd) << 16;
    const int x = 32 * qd + lane;          // this thread's lane of a 128-lane (feature-indexed) accumulator
    const int srow = 16 * qd + (lane & 15);  // its row of the M = 64 tiles S and dds (lanes 0-15 of the quadrant)
    // dN pass ownership: warp w owns positions 4w .. 4w+3, eight lanes per position
    const int prow = 4 * warp + (lane >> 3), l8 = lane & 7;

    Gates* G = (Gates*)(sm + Smem::gates);
    GateRawS* GR = (GateRawS*)(sm + Smem::graw);
    static_assert(sizeof(GateRawS) == 784, "GateRawS layout");
    float* svec = (float*)(sm + Smem::vec);
    float* sdn = (float*)(sm + Smem::dnv);
    float* sdnp = (float*)(sm + Smem::dnp);
    float* part = (float*)(sm + Smem::part);
    float* sdqn = (float*)(sm + Smem::dqn);
    float* sbq = part;  // [64] b_t dqn_t (row 0 of `part`)
    uint64_t* bars = (uint64_t*)(sm + Smem::misc);  // [0],[1] Q/K stages, [2] V, [3] Ck, [4] group A, [5] group B, [6] S and dds only
    uint32_t* tmem_slot = (uint32_t*)(sm + Smem::misc + 64);
    int* abort_flag = (int*)(sm + Smem::misc + 72);
    float* srun = (float*)(sm + Smem::misc + 80);
    float* sred = (float*)(sm + Smem::misc + 96);  // 16 floats

    unsigned char* sV = sm + Smem::v;
    unsigned char* sCk = sm + Smem::ck;
    unsigned char* sdN = sm + Smem::dn_;
    unsigned char* sdNb = sm + Smem::dnb;
    unsigned char* sdCb = sm + Smem::dcb;
    unsigned char* sDS = sm + Smem::ds_;
    unsigned char* sdS = sm + Smem::dS;

    if (tid == 0) {
        for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (is_ctrl) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // S and dds are dead once DS/dS are in shared memory; dVi and dKi reuse their columns.
    const uint32_t tS = tmem + 0, tDds = tmem + 64, tVi = tmem + 0, tKi = tmem + 64, tVe = tmem + 128, tKe = tmem + 192,
                   tQ = tmem + 256, tC = tmem + 384;

    auto issue_qk = [&](int ch, int stage) {
        mbar_expect_tx(&bars[stage], 2 * kTileBytes);
        for (int cbx = 0; cbx < 2; ++cbx) {
            tma_load_3d(sm + Smem::q + stage * kTileBytes + cbx * kBoxBytes, &p.tmq, &bars[stage], qcol + 64 * cbx, ch * L, b);
            tma_load_3d(sm + Smem::k + stage * kTileBytes + cbx * kBoxBytes, &p.tmk, &bars[stage], qcol + 64 * cbx, ch * L, b);
        }
    };
    auto issue_v_ck = [&](int ch) {
        mbar_expect_tx(&bars[2], kTileBytes);
        mbar_expect_tx(&bars[3], 2 * kStateBox);
        for (int cbx = 0; cbx < 2; ++cbx) {
            tma_load_3d(sV + cbx * kBoxBytes, &p.tmv, &bars[2], vcol + 64 * cbx, ch * L, b);
            tma_load_2d(sCk + cbx * kStateBox, &p.tmc, &bars[3], 64 * cbx, (sbh * (p.NC + 1) + ch) * D);
        }
    };

    // Operands of the dN pass, prefetched one chunk ahead into registers. Piece i of a thread covers
    // columns 4*(l8 + 8i) .. +3 of its position, so eight lanes read one contiguous run per instruction.
    // The dN pass reads dy and ytil straight from global memory; one chunk ahead its lines are pulled into
    // L2 (no registers held across phases). Piece i of a thread covers columns 4*(l8 + 8i) .. +3 of its
    // position, so eight lanes read one contiguous run per instruction.
    auto prefetch_dy = [&](int ch) {
        const int t0 = ch * L, Lc = min(L, p.T - t0);
        if (prow < Lc && l8 < 4) {
            const size_t o = ((size_t)b * p.T + t0 + prow) * p.H * dhv + vcol;
            const char* pdy = reinterpret_cast<const char*>(p.dy) + o * sizeof(GT) + l8 * 128;
            if (l8 * 128 < (int)(D * sizeof(GT))) asm volatile("prefetch.global.L2 [%0];" ::"l"(pdy));
            if (l8 < 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.ytil + o) + l8 * 128));
        }
    };
    auto load_dy = [&](int ch, uint32_t* dyraw, uint32_t* yraw) {
        const int t0 = ch * L;
        const size_t o = ((size_t)b * p.T + t0 + prow) * p.H * dhv + vcol;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = 4 * (l8 + 8 * i);
            if (sizeof(GT) == 4) {
                uint4 t = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p.dy) + o + c));
                dyraw[4 * i] = t.x; dyraw[4 * i + 1] = t.y; dyraw[4 * i + 2] = t.z; dyraw[4 * i + 3] = t.w;
            } else {
                uint2 t = __ldcs(reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p.dy) + o + c));
                dyraw[2 * i] = t.x; dyraw[2 * i + 1] = t.y;
            }
            uint2 ty = __ldcs(reinterpret_cast<const uint2*>(p.ytil + o + c));
            yraw[2 * i] = ty.x; yraw[2 * i + 1] = ty.y;
        }
    };

    // ---- prologue -------------------------------------------------------------------------------
    if (is_ctrl) {
        if (lane == 0) { issue_qk(p.NC - 1, 0); issue_v_ck(p.NC - 1); }
        gates_fetch(p, b, h, bh, p.NC - 1, &GR[(p.NC - 1) & 1], seg);
        vec_fetch(p, bh, sbh, p.NC - 1, svec + ((p.NC - 1) & 1) * kVecFloats, seg);
        cp_async_commit();
        cp_async_wait_all();
        __syncwarp();
        gates_compute(&GR[(p.NC - 1) & 1], &G[(p.NC - 1) & 1], seg);
        if (p.NC > 1) { gates_fetch(p, b, h, bh, p.NC - 2, &GR[(p.NC - 2) & 1], seg); cp_async_commit(); }
    } else {
        prefetch_dy(p.NC - 1);
        // carry term of the forget-gate gradient: <dC_in, C_end> + dn_in . n_end
        float acc = 0.f;
        if (p.cdC) {
            const bf16* Ce = p.savedC + ((size_t)sbh * (p.NC + 1) + p.NC) * D * D;
            const float* dCi = p.cdC + ((size_t)bh * dhv + vh * D) * dqk + qh * D;  // block (vh, qh), rows dqk apart
            for (int i = tid; i < D * D; i += kMathThreads) acc += dCi[(size_t)(i >> 7) * dqk + (i & 127)] * __bfloat162float(Ce[i]);
            if (tid < D && once)
                acc += p.cdn[(size_t)bh * dqk + qh * D + tid] * p.savedn[((size_t)sbh * (p.NC + 1) + p.NC) * D + tid];
        }
        acc = warp_sum(acc);
        if (lane == 0) sred[warp] = acc;
        if (tid < D) sdn[tid] = (p.cdn && once) ? p.cdn[(size_t)bh * dqk + qh * D + tid] : 0.f;
    }
    __syncthreads();
    if (tid == 0) {
        float r = 0.f;
        for (int w = 0; w < kMathWarps; ++w) r += sred[w];
        *srun = r;
    }
    if (!is_ctrl) {
        // dC+ into TMEM (pre-scaled by g of the last chunk) and as bf16 into dCb
        const float g0 = G[(p.NC - 1) & 1].g;
        const int c0 = 32 * cq;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = p.cdC ? p.cdC[((size_t)bh * dhv + vh * D + x) * dqk + qh * D + c0 + i] : 0.f;
        put_row<4>(sdCb + (cq >> 1) * kStateBox, x, 4 * (cq & 1), v);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= g0;
        tmem_st32(tC + lane_base + c0, v);
        tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // descriptor templates
    const uint64_t dK_ = smem_desc(0, 16, 1024);          // K-major operand
    const uint64_t dM1 = smem_desc(0, kBoxBytes, 1024);   // MN-major, 64-element groups kBoxBytes apart ([64-row] tiles)
    const uint64_t dM2 = smem_desc(0, kStateBox, 1024);   // MN-major over a [128-row] state tile
    constexpr uint32_t id64_kk = instr_desc(64, 64, 0, 0);     // S, dds
    constexpr uint32_t id_kk = instr_desc(128, 64, 0, 0);      // feature-major outputs, 64 positions wide
    constexpr uint32_t id_mk = instr_desc(128, 64, 1, 0);
    constexpr uint32_t id_mm = instr_desc(128, 64, 1, 1);
    constexpr uint32_t id_mm128 = instr_desc(128, 128, 1, 1);

    bool ok = true;
    int it = 0;
    for (int ch = p.NC - 1; ch >= 0; --ch, ++it) {
        const int t0 = ch * L, Lc = min(L, p.T - t0);
        const int stg = it & 1;
        Gates* Gc = &G[ch & 1];
        float* dn_in = sdn + stg * D;          // dn+
        float* dn_out = sdn + (stg ^ 1) * D;
        unsigned char* sQ = sm + Smem::q + stg * kTileBytes;
        unsigned char* sK = sm + Smem::k + stg * kTileBytes;
        const float* spsi = svec + (ch & 1) * kVecFloats;
        const float* sqn = spsi + L;
        const float* nk = spsi + 2 * L;

        // =============== phase 1: dN, dNb tiles and the dy.ytil row dots (math) =======================
        if (!is_ctrl) {
            const float bt = Gc->b[prow];
            const float psi_r = spsi[prow];
            float dot = 0.f;
            float dyv[16];
            uint32_t dyraw[sizeof(GT) == 4 ? 16 : 8], yraw[8];
            if (prow < Lc) load_dy(ch, dyraw, yraw);
            if (prow < Lc) {
                const float ipsi = 1.f / psi_r;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float d[4];
                    if (sizeof(GT) == 4) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) d[e] = __uint_as_float(dyraw[4 * i + e]);
                    } else {
                        float2 a0 = unpack_bf16(dyraw[2 * i]), a1 = unpack_bf16(dyraw[2 * i + 1]);
                        d[0] = a0.x; d[1] = a0.y; d[2] = a1.x; d[3] = a1.y;
                    }
                    float2 y0 = unpack_bf16(yraw[2 * i]), y1 = unpack_bf16(yraw[2 * i + 1]);
                    dot += d[0] * y0.x + d[1] * y0.y + d[2] * y1.x + d[3] * y1.y;
#pragma unroll
                    for (int e = 0; e < 4; ++e) dyv[4 * i + e] = d[e] * ipsi;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) dyv[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // columns 4*(l8 + 8i) .. +3: box i/2, 16-byte chunk (l8 + 8(i&1))/2, half (l8 & 1)
                const uint32_t off = (uint32_t)(i >> 1) * kBoxBytes + swz(prow, (l8 + 8 * (i & 1)) >> 1) + (l8 & 1) * 8;
                uint2 a, bb;
                a.x = pack_bf16(dyv[4 * i], dyv[4 * i + 1]); a.y = pack_bf16(dyv[4 * i + 2], dyv[4 * i + 3]);
                bb.x = pack_bf16(dyv[4 * i] * bt, dyv[4 * i + 1] * bt); bb.y = pack_bf16(dyv[4 * i + 2] * bt, dyv[4 * i + 3] * bt);
                *reinterpret_cast<uint2*>(sdN + off) = a;
                *reinterpret_cast<uint2*>(sdNb + off) = bb;
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if (l8 == 0) {
                // dqn_t = sign(qn)(-dot/psi) where the q.n term, not the floor, set psi
                float r = 0.f;
                if (dotv) dot = spsi[2 * L + D + prow];  // the row dot over all of the head's v columns
                if (prow < Lc && once) {
                    const float qn = sqn[prow];
                    if (fabsf(qn) > Gc->emm[prow]) r = (qn > 0.f ? -1.f : 1.f) * dot / psi_r;
                }
                sdqn[prow] = r;
                sbq[prow] = bt * r;
            }
            fence_async_smem();
        } else {
            if (lane == 0 && ch > 0) issue_qk(ch - 1, stg ^ 1);
            bool w = mbar_wait(&bars[stg], (it >> 1) & 1) && mbar_wait(&bars[2], it & 1) && mbar_wait(&bars[3], it & 1);
            if (!w) *abort_flag = 1;
            // the two products that need only the tiles and dC+ start now, under the dN pass
            if (w && lane == 0) {
                tc_fence_after();
                const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), adC = smem_u32(sdCb);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;  // K-major step in a [64-row] tile
                    const uint32_t kc = (ks >> 2) * kStateBox + (ks & 3) * 32;  // K-major step in a [128-row] tile
                    // dVe^T[v,j] = sum_c dC+[v,c] K[j,c]
                    mma_ss(tVe, desc_at(dK_, adC + kc), desc_at(dK_, aK + ko), id_kk, ks > 0);
                    // dKe^T[c,j] = sum_v dC+[v,c] V[j,v] : A = dCb^T (MN-major over c, K = v rows), B = V K-major
                    mma_ss(tKe, desc_at(dM2, adC + ks * 2048), desc_at(dK_, aV + ko), id_mk, ks > 0);
                }
            }
            __syncwarp();
        }
        __syncthreads();  // #1
        if (*abort_flag) { ok = false; break; }

        // =============== phase 2: group A MMAs (control) | S/dds epilogue (math) ======================
        if (is_ctrl) {
            if (lane == 0) {
                tc_fence_after();
                const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aCk = smem_u32(sCk),
                               adN = smem_u32(sdN), adNb = smem_u32(sdNb);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                    mma_ss(tS, desc_at(dK_, aQ + ko), desc_at(dK_, aK + ko), id64_kk, ks > 0);      // S = Q K^T
                    mma_ss(tDds, desc_at(dK_, adN + ko), desc_at(dK_, aV + ko), id64_kk, ks > 0);   // dds = dN V^T
                }
                mma_commit(&bars[6]);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t ko = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                    // dQ^T[c,t] = sum_v C_k[v,c] dNb[t,v] : A = Ck^T (MN-major), B = dNb K-major
                    mma_ss(tQ, desc_at(dM2, aCk + ks * 2048), desc_at(dK_, adNb + ko), id_mk, ks > 0);
                }
                // dC += dNb^T Q : M = v, N = c, K = t (needs neither DS nor dS, so it does not wait for them)
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_ss(tC, desc_at(dM1, adNb + ks * 2048), desc_at(dM1, aQ + ks * 2048), id_mm128, 1);
                mma_commit(&bars[4]);
            }
            __syncwarp();
            if (!mbar_wait(&bars[4], it & 1)) *abort_flag = 2;
            // V and C_k are read by group A only: refill them for the next chunk as soon as it is done
            if (lane == 0 && ch > 0) issue_v_ck(ch - 1);
        } else {
            if (ch > 0) prefetch_dy(ch - 1);  // lands during the rest of this chunk
            if (!mbar_wait(&bars[6], it & 1)) *abort_flag = 2;
            tc_fence_after();
            // ---- S / dds epilogue: rows live on lanes 0-15 of each quadrant; 16 columns j per thread
            float s[16], dd[16];
            tmem_ld16(tS + lane_base + 16 * cq, s);
            tmem_ld16(tDds + lane_base + 16 * cq, dd);
            tmem_ld_wait();
            {
                // branch-free and on all lanes (lanes 16-31 hold no rows of an M = 64 tile; their values are not stored):
                // the causal mask goes into the exponent's argument, exp(-inf) = 0
                const float rt = Gc->rowt[srow], dq_t = sdqn[srow];
                const int jmin = seg_first(srow, seg);  // packed mode: the row's own sequence only
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const float4 c4 = *reinterpret_cast<const float4*>(Gc->colt + 16 * cq + 4 * i4);
                    const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 4 * i4 + e, j = 16 * cq + i;
                        const float dbar = __expf((j <= srow && (!PACKED || j >= jmin)) ? rt + cc[e] : -INFINITY);
                        s[i] *= dbar;
                        dd[i] = dbar * (dd[i] + dq_t);
                    }
                }
            }
            if (lane < 16) {
                put_row<2>(sDS, srow, 2 * cq, s);
                put_row<2>(sdS, srow, 2 * cq, dd);
            }
            fence_async_smem();
            tc_fence_before();
        }
        __syncthreads();  // #2
        if (*abort_flag) { ok = false; break; }

        // =============== phase 3: group B MMAs (control) | feature-major epilogues (math) ==============
        if (is_ctrl) {
            if (lane == 0) {
                tc_fence_after();
                const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), adN = smem_u32(sdN), aDS = smem_u32(sDS), adS = smem_u32(sdS);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    // dVi^T[v,j] = sum_t dN[t,v] DS[t,j] : both MN-major, K = t rows
                    mma_ss(tVi, desc_at(dM1, adN + ks * 2048), desc_at(dM1, aDS + ks * 2048), id_mm, ks > 0);
                    // dQ^T[c,t] += sum_j K[j,c] dS[t,j] : A = K^T MN-major (K = j rows), B = dS K-major over j
                    mma_ss(tQ, desc_at(dM1, aK + ks * 2048), desc_at(dK_, adS + ks * 32), id_mk, 1);
                    // dKi^T[c,j] = sum_t Q[t,c] dS[t,j] : both MN-major, K = t rows
                    mma_ss(tKi, desc_at(dM1, aQ + ks * 2048), desc_at(dM1, adS + ks * 2048), id_mm, ks > 0);
                }
                mma_commit(&bars[5]);
            }
            __syncwarp();
            if (ch > 0) {
                cp_async_wait_all();  // raw gates of chunk ch-1, fetched during the previous chunk
                __syncwarp();
                gates_compute(&GR[(ch - 1) & 1], &G[(ch - 1) & 1], seg);
                vec_fetch(p, bh, sbh, ch - 1, svec + ((ch - 1) & 1) * kVecFloats, seg);
                if (ch > 1) gates_fetch(p, b, h, bh, ch - 2, &GR[ch & 1], seg);
                cp_async_commit();
            }
        } else {
            // this thread's feature x, positions 16*cq .. +15
            const uint32_t xoff = (uint32_t)(x >> 6) * kBoxBytes + (x & 7) * 2;
            const uint32_t xch8 = (x & 63) >> 3;
            auto tile_at = [&](const unsigned char* tile, int pos) {
                return __bfloat162float(*reinterpret_cast<const bf16*>(tile + xoff + swz(pos, xch8)));
            };
            const float n_x = nk[x], dn_x = dn_in[x];
            auto load16 = [&](const float* src, float* dst) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 t4 = *reinterpret_cast<const float4*>(src + 16 * cq + 4 * i);
                    dst[4 * i] = t4.x; dst[4 * i + 1] = t4.y; dst[4 * i + 2] = t4.z; dst[4 * i + 3] = t4.w;
                }
            };
            {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) acc += sbq[16 * cq + i] * tile_at(sQ, 16 * cq + i);
                sdnp[cq * D + x] = acc;  // dn partial over this quarter of the positions
            }
            if (!mbar_wait(&bars[5], it & 1)) *abort_flag = 3;
            tc_fence_after();
            const size_t rowbase = (size_t)b * p.T + t0 + 16 * cq;
            const size_t qstride = (size_t)p.H * dqk, vstride = (size_t)p.H * dhv;
            const size_t qbase = (size_t)vh * qk_plane + rowbase * qstride + qcol + x;
            const int nlive = min(16, Lc - 16 * cq);  // positions of this quarter inside the sequence
            float a1[16], a2[16];
            // per-position scale factors are read four at a time right where they are used (short live ranges)
            auto quad = [&](const float* src, int i4) { return *reinterpret_cast<const float4*>(src + 16 * cq + 4 * i4); };
            // dV = dVi + a dVe
            tmem_ld16(tVi + lane_base + 16 * cq, a1);
            tmem_ld16(tVe + lane_base + 16 * cq, a2);
            tmem_ld_wait();
            {
                OT* o = reinterpret_cast<OT*>(p.dv) + (size_t)qh * v_plane + rowbase * vstride + vcol + x;
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const float4 c4 = quad(Gc->a, i4);
                    const float cfv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 4 * i4 + e;
                        if (i < nlive) stf(o, (size_t)i * vstride, a1[i] + cfv[e] * a2[i]);
                    }
                }
            }
            // dQ = acc + b dqn n ;  u = dQ . q. (u also equals dy.ytil + dqn (q.n), but taking it from the same
            // rounded dS that forms dK keeps the errors of u and w correlated, so they cancel in the suffix
            // sums of u - w as the exact terms do.)
            tmem_ld16(tQ + lane_base + 16 * cq, a1);
            tmem_ld_wait();
            {
                OT* o = reinterpret_cast<OT*>(p.dq) + qbase;
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const float4 c4 = quad(sbq, i4);
                    const float cfv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 4 * i4 + e;
                        const float v = a1[i] + cfv[e] * n_x;
                        if (i < nlive) stf(o, (size_t)i * qstride, v);
                        a1[i] = v * tile_at(sQ, 16 * cq + i);
                    }
                }
            }
            const float usum = butterfly16(a1, lane);
            if ((lane & 1) == 0) part[(4 + qd) * L + 16 * cq + butterfly_index(lane)] = usum;
            // dK = dKi + a (dKe + dn+) ;  w = dK . k
            tmem_ld16(tKi + lane_base + 16 * cq, a1);
            tmem_ld16(tKe + lane_base + 16 * cq, a2);
            tmem_ld_wait();
            {
                OT* o = reinterpret_cast<OT*>(p.dk) + qbase;
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const float4 c4 = quad(Gc->a, i4);
                    const float cfv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = 4 * i4 + e;
                        const float v = a1[i] + cfv[e] * (a2[i] + dn_x);
                        if (i < nlive) stf(o, (size_t)i * qstride, v);
                        a1[i] = v * tile_at(sK, 16 * cq + i);
                    }
                }
            }
            const float wsum = butterfly16(a1, lane);
            if ((lane & 1) == 0) {
                const int pos = 16 * cq + butterfly_index(lane);
                part[(8 + qd) * L + pos] = wsum;
            }
        }
        __syncthreads();  // #3
        if (*abort_flag) { ok = false; break; }

        // =============== phase 4: gate gradients (control) | dC pass, dn (math) =======================
        if (is_ctrl) {
            float dF[2], wv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int t = lane + 32 * e;
                float u = part[4 * L + t] + part[5 * L + t] + part[6 * L + t] + part[7 * L + t];
                wv[e] = part[8 * L + t] + part[9 * L + t] + part[10 * L + t] + part[11 * L + t];
                dF[e] = (t < Lc) ? (u - wv[e]) : 0.f;
            }
            // suffix sums over the 64 positions
            float s0 = dF[0], s1 = dF[1];
            seg_suffix64(s0, s1, lane, seg);
            const float tot = __shfl_sync(0xffffffffu, s0, 0);
            const float run = *srun;
            float sf[2] = {s0, s1};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int t = lane + 32 * e;
                if (t < Lc) {
                    size_t gi = (size_t)sub * g_plane + ((size_t)b * p.T + t0 + t) * p.H + h;
                    p.dfg[gi] = (run + sf[e]) * (1.f - stable_sigmoid(Gc->fg[t]));
                    p.dig[gi] = wv[e];
                }
            }
            __syncwarp();
            if (lane == 0) *srun = run + tot;
            cp_async_wait_all();  // psi, qn, n of the next chunk are in their slot before the block barrier
        } else {
            if (tid < D) dn_out[tid] = Gc->g * dn_in[tid] + (sdnp[tid] + sdnp[D + tid]) + (sdnp[2 * D + tid] + sdnp[3 * D + tid]);
            const int c0 = 32 * cq;
            const float gn = (ch > 0) ? G[(ch - 1) & 1].g : 1.f;
            float v[32];
            tmem_ld32(tC + lane_base + c0, v);
            tmem_ld_wait();
            put_row<4>(sdCb + (cq >> 1) * kStateBox, x, 4 * (cq & 1), v);
            if (ch == 0 && p.odC) {
                float* oc = p.odC + ((size_t)bh * dhv + vh * D + x) * dqk + qh * D + c0;
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4)
                    *reinterpret_cast<float4*>(oc + 4 * q4) = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
            }
            if (ch > 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= gn;
                tmem_st32(tC + lane_base + c0, v);
                tmem_st_wait();
            }
            fence_async_smem();
            tc_fence_before();
        }
        __syncthreads();  // #4
    }

    if (ok) {
        if (p.odn && tid < D && once) p.odn[(size_t)bh * dqk + qh * D + tid] = sdn[(it & 1) * D + tid];
    } else if (tid == 0) {
        atomicCAS(p.status, 0, 200 + *abort_flag);
    }
    tc_fence_before();
    __syncthreads();
    if (is_ctrl) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// dy_t . ytil_t over all of a head's v columns, for heads split into sub-heads: one warp per (position, head).
template <typename GT>
__global__ void __launch_bounds__(256) mlstm_bw_rowdot(const GT* __restrict__ dy, const bf16* __restrict__ ytil,
                                                       float* __restrict__ dotv, int B, int H, int T, int dhv) {
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // (b*T + t)*H + h
    if (row >= (size_t)B * T * H) return;
    float acc = 0.f;
    for (int c = 4 * lane; c < dhv; c += 128) {
        float d[4];
        if (sizeof(GT) == 4) {
            const float4 t4 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(dy) + row * dhv + c));
            d[0] = t4.x; d[1] = t4.y; d[2] = t4.z; d[3] = t4.w;
        } else {
            const uint2 t2 = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(dy) + row * dhv + c));
            const float2 lo = unpack_bf16(t2.x), hi = unpack_bf16(t2.y);
            d[0] = lo.x; d[1] = lo.y; d[2] = hi.x; d[3] = hi.y;
        }
        const uint2 y2 = __ldg(reinterpret_cast<const uint2*>(ytil + row * dhv + c));
        const float2 y0 = unpack_bf16(y2.x), y1 = unpack_bf16(y2.y);
        acc += d[0] * y0.x + d[1] * y0.y + d[2] * y1.x + d[3] * y1.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        const int h = (int)(row % H);
        const size_t bt = row / H;
        dotv[((size_t)(bt / T) * H + h) * T + bt % T] = acc;
    }
}

// out[i] = sum over `np` planes of part[p][i], four elements per thread (n is a multiple of 4).
template <typename OT>
__global__ void __launch_bounds__(256) sum_planes(const float* __restrict__ part, size_t plane, int np, OT* __restrict__ out,
                                                  size_t n4) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    float4 acc = __ldcs(reinterpret_cast<const float4*>(part) + i);
    for (int q = 1; q < np; ++q) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(part + (size_t)q * plane) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (sizeof(OT) == 4) {
        reinterpret_cast<float4*>(out)[i] = acc;
    } else {
        uint2 pk;
        pk.x = pack_bf16(acc.x, acc.y); pk.y = pack_bf16(acc.z, acc.w);
        reinterpret_cast<uint2*>(out)[i] = pk;
    }
}
// Scalar tail-safe variant for the gate gradients ([B, T, H] need not be a multiple of 4).
__global__ void __launch_bounds__(256) sum_planes_scalar(const float* __restrict__ part, size_t plane, int np,
                                                         float* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float acc = part[i];
    for (int q = 1; q < np; ++q) acc += part[(size_t)q * plane + i];
    out[i] = acc;
}

}  // namespace bw

bool tc_make_map3(CUtensorMap* m, const void* base, int B, int T, int W);
bool tc_make_map2(CUtensorMap* m, const void* base, uint64_t rows, int W, int box_rows);

namespace {
struct BwPlanes {
    size_t qk, v, g, dot, total;  // byte offsets of the dq | dk | dv | dig | dfg | dot regions follow from these sizes
};
BwPlanes bw_planes(int B, int H, int T, int dqk, int dhv) {
    BwPlanes w;
    const int nq = dqk / bw::D, nv = dhv / bw::D;
    w.qk = align_up((size_t)nv * B * T * H * dqk * sizeof(float), 256);
    w.v = align_up((size_t)nq * B * T * H * dhv * sizeof(float), 256);
    w.g = align_up((size_t)nq * nv * B * T * H * sizeof(float), 256);
    w.dot = align_up((size_t)B * H * T * sizeof(float), 256);
    w.total = 2 * w.qk + w.v + 2 * w.g + w.dot;
    return w;
}
}  // namespace

size_t mlstm_tc_bw_workspace_bytes(int B, int H, int T, int dqk, int dhv) {
    if (mlstm_tc_subheads(dqk, dhv) <= 1) return 0;
    return bw_planes(B, H, T, dqk, dhv).total;
}

template <typename GT, typename OT, bool WIDE, bool PACKED = false>
static int bw_launch_kernel(cudaStream_t st, const bw::Params& p, int ctas) {
    using namespace bw;
    // the opt-in to large dynamic shared memory is a per-device function attribute: one flag per device and instantiation
    static std::atomic<bool> attr_set[64];
    const size_t smem = Smem::total + 1024;
    int dev = 0;
    XL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        XL_CUDA(cudaFuncSetAttribute(mlstm_bw_tc<GT, OT, WIDE, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    mlstm_bw_tc<GT, OT, WIDE, PACKED><<<ctas, kThreads, smem, st>>>(p);
    XL_LAUNCH_OK("mlstm_bw_tc");
    return XLSTM_OK;
}

int mlstm_bw_tc_launch(cudaStream_t st, const MlstmBwArgs& a, const void* saved, int gdtype, void* workspace,
                       size_t workspace_bytes) {
    using namespace bw;
    if (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.ytil | (uintptr_t)a.dytil | (uintptr_t)a.dq |
         (uintptr_t)a.dk | (uintptr_t)a.dv | (uintptr_t)saved) & 15) {
        set_error("mlstm_bw (tensor-core path): tensors must be 16-byte aligned");
        return XLSTM_ERR_ARG;
    }
    Params p = {};
    const int BH = a.B * a.H;
    p.nq = a.dqk / D; p.nv = a.dhv / D;
    const int nsub = p.nq * p.nv;
    const bool gbf = gdtype == XLSTM_BF16;
    p.savedC = (const bf16*)saved;
    p.savedn = (const float*)((const char*)saved + mlstm_tc_saved_C_bytes(BH * nsub, a.NC));
    if (!tc_make_map3(&p.tmq, a.q, a.B, a.T, a.H * a.dqk) || !tc_make_map3(&p.tmk, a.k, a.B, a.T, a.H * a.dqk) ||
        !tc_make_map3(&p.tmv, a.v, a.B, a.T, a.H * a.dhv) ||
        !tc_make_map2(&p.tmc, p.savedC, (uint64_t)BH * nsub * (a.NC + 1) * D, D, D)) {
        set_error("mlstm_bw: cuTensorMapEncodeTiled failed");
        return XLSTM_ERR_CUDA;
    }
    p.ig = a.ig; p.fg = a.fg; p.cm = a.cm; p.ytil = (const bf16*)a.ytil; p.msv = a.msv; p.psiv = a.psiv; p.qnv = a.qnv;
    p.dy = a.dytil; p.cdC = a.cdC; p.cdn = a.cdn; p.dq = a.dq; p.dk = a.dk; p.dv = a.dv; p.dig = a.dig; p.dfg = a.dfg;
    p.odC = a.odC; p.odn = a.odn; p.B = a.B; p.H = a.H; p.T = a.T; p.NC = a.NC; p.gbf16 = gbf;
    p.seg = a.seg; p.npack = a.npack;
    if (a.seg && (nsub != 1 || a.NC != 1 || a.T != a.seg * a.npack || a.T > L || a.seg > 32 || a.cm || a.cdC || a.odC)) {
        set_error("mlstm_bw: packed mode takes 128-wide heads, npack * seg <= 64 positions per tile, seg <= 32 and no carries");
        return XLSTM_ERR_ARG;
    }
    p.status = tc_status_ptr();
    if (!p.status) { set_error("mlstm_bw: cannot resolve the device status word"); return XLSTM_ERR_CUDA; }
    if (nsub == 1 && a.seg) return gbf ? bw_launch_kernel<bf16, bf16, false, true>(st, p, BH) : bw_launch_kernel<float, float, false, true>(st, p, BH);
    if (nsub == 1) return gbf ? bw_launch_kernel<bf16, bf16, false>(st, p, BH) : bw_launch_kernel<float, float, false>(st, p, BH);

    // wide heads: fp32 partial planes in the workspace, summed into the caller's buffers afterwards
    const BwPlanes w = bw_planes(a.B, a.H, a.T, a.dqk, a.dhv);
    if (!workspace || workspace_bytes < w.total || ((uintptr_t)workspace & 15)) {
        set_error("mlstm_bw: heads wider than 128 need a 16-byte aligned workspace of %zu B beside the state record (got %zu)",
                  w.total, workspace_bytes);
        return XLSTM_ERR_WORKSPACE;
    }
    char* ws = (char*)workspace;
    float* pdq = (float*)ws; float* pdk = (float*)(ws + w.qk); float* pdv = (float*)(ws + 2 * w.qk);
    float* pdig = (float*)(ws + 2 * w.qk + w.v); float* pdfg = (float*)(ws + 2 * w.qk + w.v + w.g);
    float* dotv = (float*)(ws + 2 * w.qk + w.v + 2 * w.g);
    const size_t rows = (size_t)a.B * a.T * a.H;
    p.dq = pdq; p.dk = pdk; p.dv = pdv; p.dig = pdig; p.dfg = pdfg;
    p.qk_plane = rows * a.dqk; p.v_plane = rows * a.dhv; p.g_plane = rows;
    if (p.nv > 1) {
        if (gbf) mlstm_bw_rowdot<bf16><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)a.dytil, p.ytil, dotv, a.B, a.H, a.T, a.dhv);
        else mlstm_bw_rowdot<float><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const float*)a.dytil, p.ytil, dotv, a.B, a.H, a.T, a.dhv);
        XL_LAUNCH_OK("mlstm_bw_rowdot");
        p.dotv = dotv;
    }
    int rc = gbf ? bw_launch_kernel<bf16, float, true>(st, p, BH * nsub) : bw_launch_kernel<float, float, true>(st, p, BH * nsub);
    if (rc) return rc;
    auto sum_to = [&](const float* part, size_t plane, int np, void* out) {
        const size_t n4 = plane / 4;
        if (gbf) sum_planes<bf16><<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(part, plane, np, (bf16*)out, n4);
        else sum_planes<float><<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(part, plane, np, (float*)out, n4);
        count_launch();
    };
    sum_to(pdq, p.qk_plane, p.nv, a.dq);
    sum_to(pdk, p.qk_plane, p.nv, a.dk);
    sum_to(pdv, p.v_plane, p.nq, a.dv);
    sum_planes_scalar<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(pdig, rows, nsub, a.dig, rows);
    sum_planes_scalar<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(pdfg, rows, nsub, a.dfg, rows);
    XL_LAUNCH_OK("mlstm_bw sum_planes");
    count_launch();
    return XLSTM_OK;
}

}  // namespace xl
