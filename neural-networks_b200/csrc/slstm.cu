// sLSTM recurrent loop, forward and backward, as persistent kernels: thread-block clusters for heads whose
// recurrent slice fits a cluster's shared memory, grid-cooperative kernels (further down) for wider heads.
//
// The T-loop is a chain of dependent small mat-vecs, so it is latency-bound: the design
// keeps everything a step needs on chip. A cluster of CS CTAs owns one (head, batch group);
// each CTA keeps its slice of the recurrent matrix in shared memory for the whole call
// (fp32, so results track the fp32 reference), computes its units' gate pre-activations
// from the head's previous h, applies the pointwise cell, and broadcasts its new h to the
// other CTAs of the cluster through distributed shared memory. One hardware cluster barrier
// per timestep is the only inter-CTA synchronisation; there is no grid-wide barrier and no
// spin-wait. Heads (block-diagonal recurrence) and batch groups are independent clusters.
//
// The backward keeps the columns of Wh that belong to a CTA's own units' gate deltas instead: its
// mat-vec then needs only the deltas the CTA has just computed, yields a partial dh for every unit
// of the head, and the CTAs exchange those partials (see slstm_bw_cluster).
//
// Math: src/nn2/slstm.rs:286-325, 399-423 with the GPU kernels' gate clamps
// (src/gpu/cuda/slstm_fused.cu:132-142). Kernels replaced: src/gpu/cuda/slstm_coop.cu:103-515.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"
#include "slstm_cell.cuh"

namespace cg = cooperative_groups;

namespace xl {

// The two halves of the hardware cluster barrier. A step uses the barrier twice, alternating:
// phase A (arrive right after the mat-vec, wait just before the broadcast) tells every CTA that all
// readers of the exchange buffer are done, so one buffer suffices; phase B (arrive + wait after the
// broadcast) publishes the new contents. Every thread of every CTA executes each call the same
// number of times, so the barrier cannot be left waiting.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

static constexpr int kThreads = 512;
static constexpr int kPF = 2;  // pointwise items per thread whose global operands are prefetched

struct SlstmArgs {
    const float* wh;
    float* g;
    const float* bcat;
    float *c, *n, *m, *h;      // forward state [B,H]
    float* out;
    xlstm_slstm_slabs s;
    const float* dy;
    float *dh, *dc, *dn;       // backward state [B,H]
    int B, H, NH, T, carry;
    int dhd;                   // units per head
    int CS, UPC;               // cluster size, units per CTA
    int KS;                    // k-slices of the mat-vec
    int CPT;                   // output columns per thread in the mat-vec (4 or 2)
    unsigned epoch;            // launch number, part of the tags of the grid kernels' flagged exchange
};

struct SlstmSmem {
    size_t ws, xin, part, stage, state, total;
};

static SlstmSmem smem_layout(int K, int NOUT, int BG, int KS, int UPC, int nstate) {
    SlstmSmem l;
    int NOUTp = (NOUT + 1) & ~1;
    auto a16 = [](size_t x) { return (x + 15) / 16 * 16; };
    l.ws = 0;
    l.xin = l.ws + a16((size_t)K * NOUTp * 4);
    l.part = l.xin + a16((size_t)K * BG * 4);
    l.stage = l.part + a16((size_t)KS * BG * NOUTp * 4);
    l.state = l.stage + a16((size_t)BG * 4 * UPC * 4);
    l.total = l.state + a16((size_t)nstate * BG * UPC * 4);
    return l;
}

// out[b][j] partial sums over a k-slice: part[(ks*BG + b)*NOUTp + j] = sum_{k in slice} xin[k*BG+b] * Ws[k*NOUTp+j].
// CPT = 2: a thread owns a column pair and uses the packed fp32x2 FMA (one instruction per batch element and
// row instead of two); CPT = 4: four columns per thread (one 16-byte weight load per row: the fewest
// shared-memory wavefronts per FMA, for wide outputs).
template <int BG, int CPT>
__device__ __forceinline__ void matvec(const float* __restrict__ Ws, const float* __restrict__ xin,
                                       float* __restrict__ part, int K, int NOUTp, int KS) {
    const int ncols = NOUTp / CPT;
    const int rows_per = (K + KS - 1) / KS;
    for (int item = threadIdx.x; item < ncols * KS; item += kThreads) {
        const int cp = item % ncols, ks = item / ncols;
        const int r0 = ks * rows_per, r1 = min(K, r0 + rows_per);
        const float* wp = Ws + (size_t)r0 * NOUTp + CPT * cp;
        const float* xp = xin + (size_t)r0 * BG;
        if (CPT == 4) {
            float4 acc[BG];
#pragma unroll
            for (int b = 0; b < BG; ++b) acc[b] = make_float4(0.f, 0.f, 0.f, 0.f);
            auto fma4 = [](float x, const float4& w, float4& a) {
                const float2 lo = __ffma2_rn(make_float2(x, x), make_float2(w.x, w.y), make_float2(a.x, a.y));
                const float2 hi = __ffma2_rn(make_float2(x, x), make_float2(w.z, w.w), make_float2(a.z, a.w));
                a = make_float4(lo.x, lo.y, hi.x, hi.y);
            };
#pragma unroll 4
            for (int r = r0; r < r1; ++r) {
                const float4 w = *reinterpret_cast<const float4*>(wp);
                if (BG % 4 == 0) {
#pragma unroll
                    for (int b4 = 0; b4 < BG / 4; ++b4) {
                        const float4 x = *reinterpret_cast<const float4*>(xp + 4 * b4);
                        fma4(x.x, w, acc[4 * b4 + 0]); fma4(x.y, w, acc[4 * b4 + 1]);
                        fma4(x.z, w, acc[4 * b4 + 2]); fma4(x.w, w, acc[4 * b4 + 3]);
                    }
                } else {
#pragma unroll
                    for (int b = 0; b < BG; ++b) fma4(xp[b], w, acc[b]);
                }
                wp += NOUTp;
                xp += BG;
            }
#pragma unroll
            for (int b = 0; b < BG; ++b)
                *reinterpret_cast<float4*>(part + ((size_t)ks * BG + b) * NOUTp + 4 * cp) = acc[b];
        } else if (CPT == 2) {
            float2 acc[BG];
#pragma unroll
            for (int b = 0; b < BG; ++b) acc[b] = make_float2(0.f, 0.f);
#pragma unroll 4
            for (int r = r0; r < r1; ++r) {
                const float2 w = *reinterpret_cast<const float2*>(wp);
                if (BG % 4 == 0) {
#pragma unroll
                    for (int b4 = 0; b4 < BG / 4; ++b4) {
                        const float4 x = *reinterpret_cast<const float4*>(xp + 4 * b4);
                        acc[4 * b4 + 0] = __ffma2_rn(make_float2(x.x, x.x), w, acc[4 * b4 + 0]);
                        acc[4 * b4 + 1] = __ffma2_rn(make_float2(x.y, x.y), w, acc[4 * b4 + 1]);
                        acc[4 * b4 + 2] = __ffma2_rn(make_float2(x.z, x.z), w, acc[4 * b4 + 2]);
                        acc[4 * b4 + 3] = __ffma2_rn(make_float2(x.w, x.w), w, acc[4 * b4 + 3]);
                    }
                } else {
#pragma unroll
                    for (int b = 0; b < BG; ++b) acc[b] = __ffma2_rn(make_float2(xp[b], xp[b]), w, acc[b]);
                }
                wp += NOUTp;
                xp += BG;
            }
#pragma unroll
            for (int b = 0; b < BG; ++b)
                *reinterpret_cast<float2*>(part + ((size_t)ks * BG + b) * NOUTp + 2 * cp) = acc[b];
        }
    }
}

// Copies stage[b][col_local] (ncol local columns per gate block layout given by the caller) into
// every cluster peer's exchange buffer xin_next[(col_global)*BG + b].
template <int BG>
__device__ __forceinline__ void broadcast(cg::cluster_group& cluster, const float* stage, float* xin_next, int CS,
                                          int nloc, int nblocks, int block_stride_loc, int block_stride_glob,
                                          int glob_off) {
    // local column index lc in [0, nblocks*nloc): block = lc / nloc (gate), within = lc % nloc
    const int total = nblocks * nloc * BG;
    for (int e = threadIdx.x; e < total; e += kThreads) {
        const int lc = e / BG, b = e % BG;
        const int blk = lc / nloc, w = lc % nloc;
        const float v = stage[(size_t)b * block_stride_loc * nblocks + blk * block_stride_loc + w];
        const size_t dst = (size_t)(blk * block_stride_glob + glob_off + w) * BG + b;
        for (int p = 0; p < CS; ++p) {
            float* remote = cluster.map_shared_rank(xin_next, p);
            remote[dst] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------------
template <int BG>
__global__ void __launch_bounds__(kThreads) slstm_fw_cluster(SlstmArgs a, SlstmSmem lay) {
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = a.CS, UPC = a.UPC, dhd = a.dhd, H = a.H, T = a.T;
    const int cr = (int)cluster.block_rank();
    const int cid = blockIdx.x / CS;
    const int nbg = (a.B + BG - 1) / BG;
    const int hd = cid / nbg, b0 = (cid % nbg) * BG;
    const int K = dhd, NOUT = 4 * UPC, NOUTp = NOUT;  // 4*UPC is even
    const int tid = threadIdx.x;

    extern __shared__ __align__(16) unsigned char smem[];
    float* Ws = (float*)(smem + lay.ws);
    float* xin = (float*)(smem + lay.xin);      // [K][BG]: h of the whole head
    float* part = (float*)(smem + lay.part);    // [KS][BG][NOUTp]
    float* stage = (float*)(smem + lay.stage);  // [BG][UPC]
    float* st = (float*)(smem + lay.state);     // c,n,m: [3][BG*UPC]
    const int NI = BG * UPC;

    // recurrent slice: Ws[r][gate*UPC + ul] = wh[hd][r][gate*dhd + cr*UPC + ul]
    for (int i = tid; i < K * NOUT; i += kThreads) {
        int r = i / NOUT, col = i % NOUT, gate = col / UPC, ul = col % UPC;
        Ws[(size_t)r * NOUTp + col] = a.wh[((size_t)hd * dhd + r) * 4 * dhd + gate * dhd + cr * UPC + ul];
    }
    // initial h of the whole head, and this CTA's c,n,m
    for (int i = tid; i < K * BG; i += kThreads) {
        int r = i / BG, b = i % BG;
        float v = 0.f;
        if (a.carry && b0 + b < a.B) v = a.h[(size_t)(b0 + b) * H + hd * dhd + r];
        xin[i] = v;
    }
    for (int it = tid; it < NI; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        size_t si = (size_t)(b0 + b) * H + hd * dhd + cr * UPC + ul;
        bool live = a.carry && b0 + b < a.B;
        st[it] = live ? a.c[si] : 0.f;
        st[NI + it] = live ? a.n[si] : 0.f;
        st[2 * NI + it] = live ? a.m[si] : 0.f;
    }
    cluster.sync();  // every CTA's buffers exist before any remote write

    // biases of the items this thread owns in the pointwise phase
    float bias[kPF][4];
#pragma unroll
    for (int p = 0; p < kPF; ++p) {
        const int it = tid + p * kThreads;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            bias[p][q] = (it < NI) ? a.bcat[q * H + hd * dhd + cr * UPC + it % UPC] : 0.f;
    }
    for (int t = 0; t < T; ++t) {
        // issue this step's global reads early; they land while the mat-vec runs
        float gpre[kPF][4];
#pragma unroll
        for (int p = 0; p < kPF; ++p) {
            int it = tid + p * kThreads;
            if (it < NI) {
                int b = it / UPC, ul = it % UPC;
                if (b0 + b < a.B) {
                    const float* gt = a.g + ((size_t)(b0 + b) * T + t) * 4 * H + hd * dhd + cr * UPC + ul;
#pragma unroll
                    for (int q = 0; q < 4; ++q) gpre[p][q] = __ldcs(gt + (size_t)q * H);
                }
            }
        }
        // this CTA's own previous h (a saved record), read before peers may overwrite the buffer
        float hprev[kPF];
#pragma unroll
        for (int p = 0; p < kPF; ++p) {
            const int it = tid + p * kThreads;
            hprev[p] = (it < NI) ? xin[(size_t)(cr * UPC + it % UPC) * BG + it / UPC] : 0.f;
        }
        if (a.CPT == 4) matvec<BG, 4>(Ws, xin, part, K, NOUTp, a.KS);
        else matvec<BG, 2>(Ws, xin, part, K, NOUTp, a.KS);
        if (NI <= kPF * kThreads) cluster_arrive();  // done reading the exchange buffer
        __syncthreads();
        auto cell = [&](int it, const float* gin, const float* bs, float hp) {
            const int b = it / UPC, ul = it % UPC;
            float hh = 0.f;
            if (b0 + b < a.B) {
                const int j = hd * dhd + cr * UPC + ul;
                float gh[4] = {0.f, 0.f, 0.f, 0.f};
                for (int ks = 0; ks < a.KS; ++ks) {
                    const float* pp = part + ((size_t)ks * BG + b) * NOUTp + ul;
#pragma unroll
                    for (int q = 0; q < 4; ++q) gh[q] += pp[q * UPC];
                }
                float* gt = a.g + ((size_t)(b0 + b) * T + t) * 4 * H + j;
                const float z_pre = gin[0] + gh[0] + bs[0];
                const float i_pre = gin[1] + gh[1] + bs[1];
                const float f_pre = gin[2] + gh[2] + bs[2];
                const float o_pre = gin[3] + gh[3] + bs[3];
                const size_t s = ((size_t)(b0 + b) * T + t) * H + j;
                const float cp = st[it], np = st[NI + it], mp = st[2 * NI + it];
                const SlstmFwCell r = slstm_cell_fw(z_pre, i_pre, f_pre, o_pre, cp, np, mp);
                hh = r.h;
                st[it] = r.c; st[NI + it] = r.n; st[2 * NI + it] = r.m;
                __stcs(gt + (size_t)2 * H, f_pre);
                __stcs(a.s.h_prev + s, hp);
                __stcs(a.s.c_prev + s, cp);
                __stcs(a.s.n_prev + s, np);
                __stcs(a.s.zt + s, r.z);
                __stcs(a.s.ot + s, r.o);
                __stcs(a.s.ipr + s, r.ip);
                __stcs(a.s.fpr + s, r.fp);
                __stcs(a.s.c + s, r.c);
                __stcs(a.s.n + s, r.n);
                __stcs(a.out + s, hh);
            }
            stage[(size_t)b * UPC + ul] = hh;
        };
#pragma unroll
        for (int p = 0; p < kPF; ++p) {
            const int it = tid + p * kThreads;
            if (it < NI) cell(it, gpre[p], bias[p], hprev[p]);
        }
        for (int it = tid + kPF * kThreads; it < NI; it += kThreads) {
            const int b = it / UPC, ul = it % UPC;
            float gin[4] = {0.f, 0.f, 0.f, 0.f};
            if (b0 + b < a.B) {
                const float* gt = a.g + ((size_t)(b0 + b) * T + t) * 4 * H + hd * dhd + cr * UPC + ul;
#pragma unroll
                for (int q = 0; q < 4; ++q) gin[q] = gt[(size_t)q * H];
            }
            float bs[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) bs[q] = a.bcat[q * H + hd * dhd + cr * UPC + ul];
            cell(it, gin, bs, xin[(size_t)(cr * UPC + ul) * BG + b]);
        }
        __syncthreads();
        if (NI > kPF * kThreads) cluster_arrive();  // wide CTAs read their previous h inside the cell
        cluster_wait();                               // every CTA is done reading: the buffer may be overwritten
        broadcast<BG>(cluster, stage, xin, CS, UPC, 1, UPC, 0, cr * UPC);
        cluster_arrive();
        cluster_wait();                               // the new h of the whole head is visible
    }
    // final state
    for (int it = tid; it < NI; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        if (b0 + b >= a.B) continue;
        size_t si = (size_t)(b0 + b) * H + hd * dhd + cr * UPC + ul;
        a.c[si] = st[it];
        a.n[si] = st[NI + it];
        a.m[si] = st[2 * NI + it];
        a.h[si] = xin[(size_t)(cr * UPC + ul) * BG + b];
    }
}

// ---------------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------------
// dh_{t-1}[u] = sum_k delta_t[k] Wh[u][k] over the head's 4*dhd gate deltas. A CTA keeps the COLUMNS of Wh that
// belong to its own units' deltas (all dhd rows x its 4*UPC columns), so its mat-vec needs only the deltas it has
// just computed and yields a partial dh for every unit of the head; it then hands each peer the slice of partials
// that peer's units need (distributed shared memory), and a CTA's recurrent dh is the sum of the CS slices it
// received, in rank order. Against broadcasting the deltas to every peer this moves a quarter of the data and
// gives the mat-vec a wide output. The receive buffers alternate by step parity, so one cluster barrier per step
// both publishes the step's partials and fences the reuse of the buffer read two steps earlier.
struct SlstmBwSmem {
    size_t ws, xin, part, recv, state, total;
};

static SlstmBwSmem bw_layout(int K, int NOUTp, int BG, int KS, int UPC, int CS) {
    SlstmBwSmem l;
    auto a16 = [](size_t x) { return (x + 15) / 16 * 16; };
    l.ws = 0;
    l.xin = l.ws + a16((size_t)K * NOUTp * 4);
    l.part = l.xin + a16((size_t)K * BG * 4);
    l.recv = l.part + a16((size_t)KS * BG * NOUTp * 4);
    l.state = l.recv + a16((size_t)2 * CS * BG * UPC * 4);
    l.total = l.state + a16((size_t)2 * BG * UPC * 4);
    return l;
}

template <int BG>
__global__ void __launch_bounds__(kThreads) slstm_bw_cluster(SlstmArgs a, SlstmBwSmem lay) {
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = a.CS, UPC = a.UPC, dhd = a.dhd, H = a.H, T = a.T;
    const int cr = (int)cluster.block_rank();
    const int cid = blockIdx.x / CS;
    const int nbg = (a.B + BG - 1) / BG;
    const int hd = cid / nbg, b0 = (cid % nbg) * BG;
    const int K = 4 * UPC, NOUT = dhd, NOUTp = (NOUT + 1) & ~1;
    const int tid = threadIdx.x;

    extern __shared__ __align__(16) unsigned char smem[];
    float* Ws = (float*)(smem + lay.ws);      // [K = gate*UPC + ul][NOUTp]: Wh[u][gate*dhd + own unit ul] for every unit u
    float* xin = (float*)(smem + lay.xin);    // [K][BG]: this CTA's own gate deltas
    float* part = (float*)(smem + lay.part);  // [KS][BG][NOUTp]: k-slices of the partial dh for the whole head
    float* recv = (float*)(smem + lay.recv);  // [2 parities][CS senders][BG][UPC]: partial dh of the own units
    float* st = (float*)(smem + lay.state);   // dc, dn: [2][BG*UPC]
    const int NI = BG * UPC;

    for (int i = tid; i < K * NOUTp; i += kThreads) {
        const int k = i / NOUTp, u = i % NOUTp, gate = k / UPC, ul = k % UPC;
        Ws[i] = u < NOUT ? a.wh[((size_t)hd * dhd + u) * 4 * dhd + gate * dhd + cr * UPC + ul] : 0.f;
    }
    // the dh carry takes sender 0's place in the buffer the first processed step reads (parity T & 1)
    for (int i = tid; i < 2 * CS * NI; i += kThreads) {
        const int par = i / (CS * NI), sdr = (i / NI) % CS, it = i % NI, b = it / UPC, ul = it % UPC;
        float v = 0.f;
        if (par == (T & 1) && sdr == 0 && a.carry && b0 + b < a.B) v = a.dh[(size_t)(b0 + b) * H + hd * dhd + cr * UPC + ul];
        recv[i] = v;
    }
    for (int it = tid; it < NI; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        size_t si = (size_t)(b0 + b) * H + hd * dhd + cr * UPC + ul;
        bool live = a.carry && b0 + b < a.B;
        st[it] = live ? a.dc[si] : 0.f;
        st[NI + it] = live ? a.dn[si] : 0.f;
    }
    cluster.sync();  // every CTA's buffers exist before any remote write

    // operands of the first processed step
    float pre[kPF][10];
    auto prefetch = [&](int t) {
#pragma unroll
        for (int p = 0; p < kPF; ++p) {
            int it = tid + p * kThreads;
            if (it < NI && t >= 0) {
                int b = it / UPC, ul = it % UPC;
                if (b0 + b < a.B) {
                    const int j = hd * dhd + cr * UPC + ul;
                    const size_t s = ((size_t)(b0 + b) * T + t) * H + j;
                    pre[p][0] = __ldcs(a.dy + s);
                    pre[p][1] = __ldcs(a.s.ot + s);
                    pre[p][2] = __ldcs(a.s.c + s);
                    pre[p][3] = __ldcs(a.s.n + s);
                    pre[p][4] = __ldcs(a.s.fpr + s);
                    pre[p][5] = __ldcs(a.s.ipr + s);
                    pre[p][6] = __ldcs(a.s.zt + s);
                    pre[p][7] = __ldcs(a.s.c_prev + s);
                    pre[p][8] = __ldcs(a.s.n_prev + s);
                    pre[p][9] = __ldcs(a.g + ((size_t)(b0 + b) * T + t) * 4 * H + 2 * H + j);
                }
            }
        }
    };
    prefetch(T - 1);
    for (int t = T - 1; t >= 0; --t) {
        const float* rp = recv + (size_t)((t + 1) & 1) * CS * NI;  // what the peers sent during step t+1 (or the carry)
        auto cell = [&](int it, const float* op) {
            const int b = it / UPC, ul = it % UPC;
            float dz = 0.f, di = 0.f, df = 0.f, dob = 0.f;
            if (b0 + b < a.B) {
                const int j = hd * dhd + cr * UPC + ul;
                float* gt = a.g + ((size_t)(b0 + b) * T + t) * 4 * H + j;
                float dhr = 0.f;
                for (int sdr = 0; sdr < CS; ++sdr) dhr += rp[(size_t)sdr * NI + it];
                const SlstmBwCell r = slstm_cell_bw(op[0] + dhr, op[1], op[2], op[3], op[4], op[5], op[6], op[7], op[8],
                                                    op[9], st[it], st[NI + it]);
                dz = r.dz; di = r.di; df = r.df; dob = r.dob;
                st[it] = r.dc;
                st[NI + it] = r.dn;
                __stcs(gt, dz);
                __stcs(gt + (size_t)H, di);
                __stcs(gt + (size_t)2 * H, df);
                __stcs(gt + (size_t)3 * H, dob);
            }
            xin[(size_t)(0 * UPC + ul) * BG + b] = dz;
            xin[(size_t)(1 * UPC + ul) * BG + b] = di;
            xin[(size_t)(2 * UPC + ul) * BG + b] = df;
            xin[(size_t)(3 * UPC + ul) * BG + b] = dob;
        };
#pragma unroll
        for (int p = 0; p < kPF; ++p) {
            const int it = tid + p * kThreads;
            if (it < NI) cell(it, pre[p]);
        }
        for (int it = tid + kPF * kThreads; it < NI; it += kThreads) {
            const int b = it / UPC, ul = it % UPC;
            float op[10] = {0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (b0 + b < a.B) {
                const int j = hd * dhd + cr * UPC + ul;
                const size_t s = ((size_t)(b0 + b) * T + t) * H + j;
                op[0] = a.dy[s]; op[1] = a.s.ot[s]; op[2] = a.s.c[s]; op[3] = a.s.n[s]; op[4] = a.s.fpr[s];
                op[5] = a.s.ipr[s]; op[6] = a.s.zt[s]; op[7] = a.s.c_prev[s]; op[8] = a.s.n_prev[s];
                op[9] = a.g[((size_t)(b0 + b) * T + t) * 4 * H + 2 * H + j];
            }
            cell(it, op);
        }
        __syncthreads();
        prefetch(t - 1);
        if (a.CPT == 4) matvec<BG, 4>(Ws, xin, part, K, NOUTp, a.KS);
        else matvec<BG, 2>(Ws, xin, part, K, NOUTp, a.KS);
        __syncthreads();
        // sum the k-slices and hand every peer the partials of its units
        float* wbase = recv + (size_t)((t & 1) * CS + cr) * NI;
        for (int e = tid; e < BG * NOUT; e += kThreads) {
            const int b = e / NOUT, u = e % NOUT;
            float v = 0.f;
            for (int ks = 0; ks < a.KS; ++ks) v += part[((size_t)ks * BG + b) * NOUTp + u];
            float* remote = cluster.map_shared_rank(wbase, u / UPC);
            remote[b * UPC + u % UPC] = v;
        }
        cluster_arrive();
        cluster_wait();  // this step's partials are visible everywhere; the other parity's buffer is free again
    }
    const float* rp = recv;  // written during step 0 (parity 0), or the untouched carry when T == 0
    for (int it = tid; it < NI; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        if (b0 + b >= a.B) continue;
        size_t si = (size_t)(b0 + b) * H + hd * dhd + cr * UPC + ul;
        float dhr = 0.f;
        for (int sdr = 0; sdr < CS; ++sdr) dhr += rp[(size_t)sdr * NI + it];
        a.dh[si] = dhr;
        a.dc[si] = st[it];
        a.dn[si] = st[NI + it];
    }
}

// ---------------------------------------------------------------------------------------------
// Grid-cooperative variant for heads too wide for a cluster's shared memory (dense H = 1024,
// block-diagonal heads of 512 units): the G CTAs of a head span up to the whole GPU, launched
// cooperatively so that all are resident. The exchange goes through global memory, and needs no
// buffer of its own: forward peers read h_{t-1} from `out[:, t-1, :]`, backward peers read the gate
// deltas from `g[:, t, :]`, both of which the call has to write anyway. One counter barrier per head
// and step orders the writes before the reads; every wait is bounded and a timeout makes all CTAs
// leave the loop. Batch entries are processed in sub-groups of BG per step so that the staged
// vector fits beside the recurrent slice.
// ---------------------------------------------------------------------------------------------
struct GridSync {
    unsigned int count[64];  // arrivals per head
    unsigned int abort;
    unsigned int pad[63];
};
static __device__ GridSync g_slstm_sync;
static constexpr unsigned kSpinLimit = 1u << 21;  // about a second of polling

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Barrier among the CTAs of head `hd`: returns once `target` arrivals were counted, or false when the
// wait ran out or another CTA gave up.
__device__ __forceinline__ bool group_barrier(GridSync* gs, int hd, unsigned target, int* s_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&gs->count[hd], 1u);
        bool ok = true;
        unsigned spins = 0;
        while (ld_acquire_u32(&gs->count[hd]) < target) {
            ++spins;
            if (spins > kSpinLimit || ((spins & 63u) == 0 && ld_acquire_u32(&gs->abort))) { ok = false; break; }
        }
        if (!ok) atomicExch(&gs->abort, 1u);
        *s_flag = ok ? 1 : 0;
    }
    __syncthreads();
    return *s_flag != 0;
}

// xin[k][0..BG) <- vector k of each live batch entry of a sub-group, read from L2 (the writers are other
// CTAs). A thread takes one k for all entries: consecutive lanes read consecutive addresses of each row
// and write whole [BG] records. `seg` floats are contiguous in a row, segments `sstride` floats apart.
template <int BG>
__device__ __forceinline__ void stage_rows(float* xin, const float* base, size_t bstride, int nlive, int K, int seg,
                                           size_t sstride) {
    for (int k = threadIdx.x; k < K; k += kThreads) {
        const size_t off = (size_t)(k / seg) * sstride + (size_t)(k % seg);
        float v[BG];
#pragma unroll
        for (int b = 0; b < BG; ++b) v[b] = (b < nlive) ? __ldcg(base + (size_t)b * bstride + off) : 0.f;
        float* dst = xin + (size_t)k * BG;
        if (BG % 4 == 0) {
#pragma unroll
            for (int b4 = 0; b4 < BG / 4; ++b4)
                *reinterpret_cast<float4*>(dst + 4 * b4) = make_float4(v[4 * b4], v[4 * b4 + 1], v[4 * b4 + 2], v[4 * b4 + 3]);
        } else {
#pragma unroll
            for (int b = 0; b < BG; ++b) dst[b] = v[b];
        }
    }
}

// Flagged exchange ("value + tag in one 8-byte word"): instead of writing a vector, arriving at a counter and
// having every reader wait for the count, a producer stores each value together with a tag that names the
// launch and the step, and a consumer re-reads a word until its tag is the one it wants. An 8-byte aligned
// store is single-copy atomic, so a matching tag proves the value beside it, with no fence and no barrier:
// a step costs one L2 round trip. Two buffers alternate by step parity; a producer can only reach step t+2
// after every CTA of the head consumed step t, so the buffer it overwrites is no longer being read.
static constexpr size_t kLLWords = (size_t)1 << 18;  // 2 MiB: two buffers of B x H values up to B*H = 131072
static __device__ __align__(16) uint2 g_slstm_ll[kLLWords];

__device__ __forceinline__ unsigned ll_tag(unsigned epoch, int t) { return (epoch << 20) | (unsigned)(t + 1); }
__device__ __forceinline__ void ll_store(uint2* p, float v, unsigned tag) {
    asm volatile("st.relaxed.gpu.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ll_load(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.gpu.global.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// stage_rows over the flagged exchange: every word is polled until it carries `tag`. Returns false when a
// word did not arrive within the polling budget (the caller then raises the abort flag and unwinds).
template <int BG>
__device__ __forceinline__ bool stage_rows_ll(float* xin, const uint2* base, size_t bstride, int nlive, int K, int seg,
                                              size_t sstride, unsigned tag, const unsigned* abort_word) {
    bool ok = true;
    for (int k = threadIdx.x; k < K; k += kThreads) {
        const size_t off = (size_t)(k / seg) * sstride + (size_t)(k % seg);
        uint2 w[BG];
#pragma unroll
        for (int b = 0; b < BG; ++b) w[b] = (b < nlive) ? ll_load(base + (size_t)b * bstride + off) : make_uint2(0u, tag);
        unsigned spins = 0;
        for (;;) {
            bool all = true;
#pragma unroll
            for (int b = 0; b < BG; ++b)
                if (w[b].y != tag) { all = false; w[b] = ll_load(base + (size_t)b * bstride + off); }
            if (all) break;
            if (++spins > kSpinLimit || ((spins & 255u) == 0 && ld_acquire_u32(abort_word))) { ok = false; break; }
        }
        float* dst = xin + (size_t)k * BG;
#pragma unroll
        for (int b = 0; b < BG; ++b) dst[b] = __uint_as_float(w[b].x);
    }
    return ok;
}

struct GridSmem {
    size_t ws, xin, part, state, total;
};

static GridSmem grid_layout(int K, int NOUTp, int BG, int KS, int UPC, int Bp, int nstate) {
    GridSmem l;
    auto a16 = [](size_t x) { return (x + 15) / 16 * 16; };
    l.ws = 0;
    l.xin = l.ws + a16((size_t)K * NOUTp * 4);
    l.part = l.xin + a16((size_t)K * BG * 4);
    l.state = l.part + a16((size_t)KS * BG * NOUTp * 4);
    l.total = l.state + a16((size_t)nstate * Bp * UPC * 4);
    return l;
}

// The same product for the geometry in which every thread owns exactly one (column pair, k-slice of 32 rows) item
// for the whole call: its 64 weights stay in registers across the timesteps, so a step reads only the staged vector
// from shared memory (half the shared-memory wavefronts of the loop above and no weight-load latency in it).
template <int BG>
__device__ __forceinline__ void matvec_reg2(const float2 (&w)[32], const float* __restrict__ xin, float* __restrict__ part,
                                            int NOUTp, int cp, int ks) {
    static_assert(BG % 4 == 0, "register mat-vec takes batch groups of 4, 8, ...");
    float2 acc[BG];
#pragma unroll
    for (int b = 0; b < BG; ++b) acc[b] = make_float2(0.f, 0.f);
    const float* xp = xin + (size_t)ks * 32 * BG;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
#pragma unroll
        for (int b4 = 0; b4 < BG / 4; ++b4) {
            const float4 x = *reinterpret_cast<const float4*>(xp + r * BG + 4 * b4);
            acc[4 * b4 + 0] = __ffma2_rn(make_float2(x.x, x.x), w[r], acc[4 * b4 + 0]);
            acc[4 * b4 + 1] = __ffma2_rn(make_float2(x.y, x.y), w[r], acc[4 * b4 + 1]);
            acc[4 * b4 + 2] = __ffma2_rn(make_float2(x.z, x.z), w[r], acc[4 * b4 + 2]);
            acc[4 * b4 + 3] = __ffma2_rn(make_float2(x.w, x.w), w[r], acc[4 * b4 + 3]);
        }
    }
#pragma unroll
    for (int b = 0; b < BG; ++b) *reinterpret_cast<float2*>(part + ((size_t)ks * BG + b) * NOUTp + 2 * cp) = acc[b];
}

template <int BG, bool LL>
__global__ void __launch_bounds__(kThreads) slstm_fw_grid(SlstmArgs a, GridSmem lay, GridSync* gs, int* status, uint2* ll) {
    const int G = a.CS, UPC = a.UPC, dhd = a.dhd, H = a.H, T = a.T, B = a.B;
    const int hd = blockIdx.x / G, cr = blockIdx.x % G;
    const int K = dhd, NOUT = 4 * UPC;
    const int tid = threadIdx.x;
    const int nsub = (B + BG - 1) / BG, NS = nsub * BG * UPC;

    extern __shared__ __align__(16) unsigned char smem[];
    float* Ws = (float*)(smem + lay.ws);      // [K][4*UPC]
    float* xin = (float*)(smem + lay.xin);    // [K][BG]: h_{t-1} of the head for one batch sub-group
    float* part = (float*)(smem + lay.part);  // [KS][BG][4*UPC]
    float* st = (float*)(smem + lay.state);   // c, n, m, h: [4][nsub*BG*UPC]
    __shared__ int s_flag;

    for (int i = tid; i < K * NOUT; i += kThreads) {
        int r = i / NOUT, col = i % NOUT, gate = col / UPC, ul = col % UPC;
        Ws[i] = a.wh[((size_t)hd * dhd + r) * 4 * dhd + gate * dhd + cr * UPC + ul];
    }
    for (int it = tid; it < NS; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        size_t si = (size_t)b * H + hd * dhd + cr * UPC + ul;
        bool live = a.carry && b < B;
        st[it] = live ? a.c[si] : 0.f;
        st[NS + it] = live ? a.n[si] : 0.f;
        st[2 * NS + it] = live ? a.m[si] : 0.f;
        st[3 * NS + it] = live ? a.h[si] : 0.f;
    }
    __syncthreads();

    // thread `tid` owns item tid = b*UPC + ul (when there is one): its bias stays in registers and its gate
    // pre-activations are fetched at the top of the step, under the staging and the mat-vec
    float bias[4] = {0.f, 0.f, 0.f, 0.f};
    const bool own = tid < B * UPC;
    const int own_j = hd * dhd + cr * UPC + tid % UPC;
    if (own) {
#pragma unroll
        for (int q = 0; q < 4; ++q) bias[q] = a.bcat[q * H + own_j];
    }
    bool ok = true;
    if (tid == 0) s_flag = 1;
    // register-resident weights where the mat-vec's item map is one item of 32 rows per thread (block-diagonal heads of
    // 512 units over 32 CTAs: 64 columns, 16 k-slices)
    const bool wreg_on = BG % 4 == 0 && a.CPT == 2 && (NOUT / 2) * a.KS == kThreads && K == 32 * a.KS;
    const int mv_cp = tid % (NOUT / 2), mv_ks = tid / (NOUT / 2);
    float2 wreg[32];
    if (wreg_on) {
#pragma unroll
        for (int r = 0; r < 32; ++r) wreg[r] = *reinterpret_cast<const float2*>(Ws + (size_t)(mv_ks * 32 + r) * NOUT + 2 * mv_cp);
    }
    __syncthreads();
    for (int t = 0; t < T && ok; ++t) {
        float gpre[4] = {0.f, 0.f, 0.f, 0.f};
        if (own) {
            const float* gt = a.g + ((size_t)(tid / UPC) * T + t) * 4 * H + own_j;
#pragma unroll
            for (int q = 0; q < 4; ++q) gpre[q] = __ldcs(gt + (size_t)q * H);
        }
        for (int sg = 0; sg < nsub; ++sg) {
            const int b0 = sg * BG;
            const int nlive = min(BG, B - b0);
            if (t > 0 && LL) {
                const uint2* src = ll + ((size_t)((t - 1) & 1) * B + b0) * H + hd * dhd;
                if (!stage_rows_ll<BG>(xin, src, (size_t)H, nlive, K, K, 0, ll_tag(a.epoch, t - 1), &gs->abort)) s_flag = 0;
            } else if (t > 0) {
                stage_rows<BG>(xin, a.out + ((size_t)b0 * T + t - 1) * H + hd * dhd, (size_t)T * H, nlive, K, K, 0);
            } else {
                stage_rows<BG>(xin, a.h + (size_t)b0 * H + hd * dhd, (size_t)H, a.carry ? nlive : 0, K, K, 0);
            }
            __syncthreads();
            if (LL && !s_flag) { ok = false; break; }
            if (BG % 4 == 0 && wreg_on) matvec_reg2<(BG % 4 == 0 ? BG : 4)>(wreg, xin, part, NOUT, mv_cp, mv_ks);
            else if (a.CPT == 4) matvec<BG, 4>(Ws, xin, part, K, NOUT, a.KS);
            else matvec<BG, 2>(Ws, xin, part, K, NOUT, a.KS);
            __syncthreads();
            for (int gi = tid; gi < B * UPC; gi += kThreads) {  // global item b*UPC + ul; this sub-group's only
                const int it = gi - b0 * UPC;
                if (it < 0 || it >= BG * UPC) continue;
                const int b = it / UPC, ul = it % UPC;
                const int j = hd * dhd + cr * UPC + ul;
                const int si = gi;
                float gh[4] = {0.f, 0.f, 0.f, 0.f};
                for (int ks = 0; ks < a.KS; ++ks) {
                    const float* pp = part + ((size_t)ks * BG + b) * NOUT + ul;
#pragma unroll
                    for (int q = 0; q < 4; ++q) gh[q] += pp[q * UPC];
                }
                float* gt = a.g + ((size_t)(b0 + b) * T + t) * 4 * H + j;
                float pre[4];
                if (gi == tid) {  // the item whose operands this thread fetched ahead
#pragma unroll
                    for (int q = 0; q < 4; ++q) pre[q] = gpre[q] + gh[q] + bias[q];
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) pre[q] = __ldcs(gt + (size_t)q * H) + gh[q] + __ldg(a.bcat + q * H + j);
                }
                const float cp = st[si], np = st[NS + si], mp = st[2 * NS + si], hp = st[3 * NS + si];
                const SlstmFwCell r = slstm_cell_fw(pre[0], pre[1], pre[2], pre[3], cp, np, mp);
                st[si] = r.c; st[NS + si] = r.n; st[2 * NS + si] = r.m; st[3 * NS + si] = r.h;
                const size_t s = ((size_t)(b0 + b) * T + t) * H + j;
                if (LL) ll_store(ll + ((size_t)(t & 1) * B + b0 + b) * H + j, r.h, ll_tag(a.epoch, t));
                __stcg(a.out + s, r.h);  // the record; without the flagged exchange also what the other CTAs read next step
                __stcs(gt + (size_t)2 * H, pre[2]);
                __stcs(a.s.h_prev + s, hp);
                __stcs(a.s.c_prev + s, cp);
                __stcs(a.s.n_prev + s, np);
                __stcs(a.s.zt + s, r.z);
                __stcs(a.s.ot + s, r.o);
                __stcs(a.s.ipr + s, r.ip);
                __stcs(a.s.fpr + s, r.fp);
                __stcs(a.s.c + s, r.c);
                __stcs(a.s.n + s, r.n);
            }
            __syncthreads();  // the next sub-group reuses xin and part
        }
        // without the flagged exchange: one counter barrier per step (it also orders the last read of the carried
        // h before its update; the flagged form is only launched for T >= 2, where the second step does that)
        if (!LL && ok) ok = group_barrier(gs, hd, (unsigned)(t + 1) * (unsigned)G, &s_flag);
    }
    if (!ok) {
        if (tid == 0) { atomicExch(&gs->abort, 1u); atomicCAS(status, 0, 301); }
        return;
    }
    for (int it = tid; it < NS; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        if (b >= B) continue;
        size_t si = (size_t)b * H + hd * dhd + cr * UPC + ul;
        a.c[si] = st[it];
        a.n[si] = st[NS + it];
        a.m[si] = st[2 * NS + it];
        a.h[si] = st[3 * NS + it];
    }
}

// Backward, grid-cooperative, partial-sum exchange. dh_{t-1}[u] = sum_k delta[k] Wh[u][k] over the head's 4*dhd
// gate deltas. Instead of every CTA gathering all of the head's deltas, a CTA keeps the
// COLUMNS of Wh that belong to its own units' deltas (all dhd rows x its 4*UPC columns, the same 128 KB), so its
// mat-vec needs only the deltas it has just computed (no staging from L2) and yields a partial dh for every unit
// of the head. The partials go to a global exchange buffer; after the head's counter barrier each CTA sums the G
// partials of its own units in a fixed order. Per step a CTA writes B*dhd floats and reads G*B*UPC = B*dhd
// floats, a quarter of what gathering the deltas would read, and the mat-vec has a wide output (four columns per
// thread). Measured against a gather form of the same kernel: 6.9 vs 8.9 us per step at 4 x 512-unit heads,
// 26 vs 75 at dense H = 1024. (The forward keeps the gather form: its partials would be four times wider than h.)
template <int BG>
__global__ void __launch_bounds__(kThreads) slstm_bw_grid_ps(SlstmArgs a, GridSmem lay, GridSync* gs, int* status, float* xch) {
    const int G = a.CS, UPC = a.UPC, dhd = a.dhd, H = a.H, T = a.T, B = a.B, NH = a.NH;
    const int hd = blockIdx.x / G, cr = blockIdx.x % G;
    const int K = 4 * UPC, NOUT = dhd;
    const int tid = threadIdx.x;
    const int nsub = (B + BG - 1) / BG, NS = nsub * BG * UPC;

    extern __shared__ __align__(16) unsigned char smem[];
    float* Ws = (float*)(smem + lay.ws);      // [K = gate*UPC + ul][dhd]: Wh[u][gate*dhd + own unit ul] for every unit u
    float* xin = (float*)(smem + lay.xin);    // [K][BG]: this CTA's own gate deltas for one batch sub-group
    float* part = (float*)(smem + lay.part);  // [KS][BG][dhd]
    float* st = (float*)(smem + lay.state);   // dc, dn, recurrent dh: [3][nsub*BG*UPC]
    __shared__ int s_flag;

    for (int i = tid; i < K * NOUT; i += kThreads) {
        const int k = i / NOUT, u = i % NOUT, gate = k / UPC, ul = k % UPC;
        Ws[i] = a.wh[((size_t)hd * dhd + u) * 4 * dhd + gate * dhd + cr * UPC + ul];
    }
    for (int it = tid; it < NS; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        size_t si = (size_t)b * H + hd * dhd + cr * UPC + ul;
        bool live = a.carry && b < B;
        st[it] = live ? a.dc[si] : 0.f;
        st[NS + it] = live ? a.dn[si] : 0.f;
        st[2 * NS + it] = live ? a.dh[si] : 0.f;
    }
    __syncthreads();

    auto fetch = [&](int it, int t, float* op) {
        const int b = it / UPC, ul = it % UPC;
        const int j = hd * dhd + cr * UPC + ul;
        const size_t s = ((size_t)b * T + t) * H + j;
        op[0] = __ldcs(a.dy + s); op[1] = __ldcs(a.s.ot + s); op[2] = __ldcs(a.s.c + s); op[3] = __ldcs(a.s.n + s);
        op[4] = __ldcs(a.s.fpr + s); op[5] = __ldcs(a.s.ipr + s); op[6] = __ldcs(a.s.zt + s);
        op[7] = __ldcs(a.s.c_prev + s); op[8] = __ldcs(a.s.n_prev + s);
        op[9] = __ldcs(a.g + ((size_t)b * T + t) * 4 * H + 2 * H + j);
    };
    float pre[10];
    const bool own = tid < B * UPC;
    if (own && T > 0) fetch(tid, T - 1, pre);
    const size_t slab = (size_t)B * dhd;  // one CTA's partials for one step
    // One output column per thread where the head's width is the CTA's thread count and the CTA owns 16 units (64 delta
    // rows): the column's 64 weights stay in registers, the thread walks all rows itself and stores its sums straight to
    // the exchange buffer: no k-slice partials in shared memory, no pass that adds them, one block barrier fewer.
    const bool wcol_on = BG % 4 == 0 && NOUT == kThreads && K == 64;
    float wcol[64];
    if (wcol_on) {
#pragma unroll
        for (int k = 0; k < 64; ++k) wcol[k] = Ws[(size_t)k * NOUT + tid];
    }
    bool ok = true;
    for (int t = T - 1; t >= 0 && ok; --t) {
        float* xw = xch + ((size_t)((t & 1) * NH + hd) * G) * slab;  // this step's partials of the head, [G][B][dhd]
        for (int sg = 0; sg < nsub; ++sg) {
            const int b0 = sg * BG;
            // gate deltas of the own units for this sub-group: to g (the record) and to shared memory (the operand)
            if (B % BG != 0) {  // a ragged last sub-group: entries past the batch end stay zero (otherwise all are rewritten)
                for (int e = tid; e < K * BG; e += kThreads) xin[e] = 0.f;
                __syncthreads();
            }
            for (int gi = tid; gi < B * UPC; gi += kThreads) {
                const int it = gi - b0 * UPC;
                if (it < 0 || it >= BG * UPC) continue;
                const int b = it / UPC, ul = it % UPC;
                const int j = hd * dhd + cr * UPC + ul;
                float* gt = a.g + ((size_t)(b0 + b) * T + t) * 4 * H + j;
                float op[10];
                if (gi == tid) {
#pragma unroll
                    for (int q = 0; q < 10; ++q) op[q] = pre[q];
                    if (t > 0) fetch(tid, t - 1, pre);  // lands under the mat-vec and the exchange
                } else {
                    fetch(gi, t, op);
                }
                const SlstmBwCell c = slstm_cell_bw(op[0] + st[2 * NS + gi], op[1], op[2], op[3], op[4], op[5], op[6], op[7],
                                                    op[8], op[9], st[gi], st[NS + gi]);
                st[gi] = c.dc;
                st[NS + gi] = c.dn;
                __stcs(gt, c.dz);
                __stcs(gt + (size_t)H, c.di);
                __stcs(gt + (size_t)2 * H, c.df);
                __stcs(gt + (size_t)3 * H, c.dob);
                xin[(size_t)(0 * UPC + ul) * BG + b] = c.dz;
                xin[(size_t)(1 * UPC + ul) * BG + b] = c.di;
                xin[(size_t)(2 * UPC + ul) * BG + b] = c.df;
                xin[(size_t)(3 * UPC + ul) * BG + b] = c.dob;
            }
            __syncthreads();
            const int nb = min(BG, B - b0);
            if (BG % 4 == 0 && wcol_on) {
                float2 acc2[(BG % 4 == 0 ? BG : 4) / 2];  // batch pairs: the staged row gives them as natural register pairs
#pragma unroll
                for (int i = 0; i < BG / 2; ++i) acc2[i] = make_float2(0.f, 0.f);
#pragma unroll
                for (int k = 0; k < 64; ++k) {
                    const float2 ww = make_float2(wcol[k], wcol[k]);
#pragma unroll
                    for (int b4 = 0; b4 < BG / 4; ++b4) {
                        const float4 x = *reinterpret_cast<const float4*>(xin + (size_t)k * BG + 4 * b4);
                        acc2[2 * b4] = __ffma2_rn(ww, make_float2(x.x, x.y), acc2[2 * b4]);
                        acc2[2 * b4 + 1] = __ffma2_rn(ww, make_float2(x.z, x.w), acc2[2 * b4 + 1]);
                    }
                }
                float* dstc = xw + (size_t)cr * slab + (size_t)b0 * dhd + tid;
#pragma unroll
                for (int i = 0; i < BG / 2; ++i) {
                    if (2 * i < nb) __stcg(dstc + (size_t)(2 * i) * dhd, acc2[i].x);
                    if (2 * i + 1 < nb) __stcg(dstc + (size_t)(2 * i + 1) * dhd, acc2[i].y);
                }
                __syncthreads();
                continue;
            }
            matvec<BG, 4>(Ws, xin, part, K, NOUT, a.KS);
            __syncthreads();
            // sum the k-slices and publish this CTA's partial dh for every unit of the head
            for (int e = tid; e < nb * (NOUT / 4); e += kThreads) {
                const int b = e / (NOUT / 4), u4 = e % (NOUT / 4);
                float4 acc = *reinterpret_cast<const float4*>(part + (size_t)b * NOUT + 4 * u4);
                for (int ks = 1; ks < a.KS; ++ks) {
                    const float4 v = *reinterpret_cast<const float4*>(part + ((size_t)ks * BG + b) * NOUT + 4 * u4);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                __stcg(reinterpret_cast<float4*>(xw + (size_t)cr * slab + (size_t)(b0 + b) * dhd) + u4, acc);
            }
            __syncthreads();
        }
        ok = group_barrier(gs, hd, (unsigned)(T - t) * (unsigned)G, &s_flag);
        if (!ok) break;
        // dh_{t-1} of the own units: the G partials, summed in CTA order
        // four lanes per item: lane q sums the partials of CTAs q, q+4, ... in order, then the four sums are combined
        for (int base = 0; base < B * UPC; base += kThreads / 4) {
            const int it = base + tid / 4, q = tid & 3;
            float acc = 0.f;
            if (it < B * UPC) {
                const int b = it / UPC, ul = it % UPC;
                const float* src = xw + (size_t)b * dhd + cr * UPC + ul;
#pragma unroll 8
                for (int s2 = q; s2 < G; s2 += 4) acc += __ldcg(src + (size_t)s2 * slab);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (it < B * UPC && q == 0) st[2 * NS + it] = acc;
        }
        __syncthreads();
    }
    if (!ok) {
        if (tid == 0) { atomicExch(&gs->abort, 1u); atomicCAS(status, 0, 303); }
        return;
    }
    for (int it = tid; it < NS; it += kThreads) {
        int b = it / UPC, ul = it % UPC;
        if (b >= B) continue;
        size_t si = (size_t)b * H + hd * dhd + cr * UPC + ul;
        a.dc[si] = st[it];
        a.dn[si] = st[NS + it];
        a.dh[si] = st[2 * NS + it];
    }
}

// ---------------------------------------------------------------------------------------------
// Host side: geometry and launch
// ---------------------------------------------------------------------------------------------
struct Geo {
    int BG, CS, UPC, KS, CPT;
    SlstmSmem lay;      // forward
    SlstmBwSmem blay;   // backward
    size_t total;       // dynamic shared memory of the kernel this geometry is for
};

static const size_t kSmemCap = 220 * 1024;

static bool fits(int BG, int CS, int dhd, bool bwd, Geo* out) {
    if (dhd % CS) return false;
    int UPC = dhd / CS;
    // forward: K = dhd inputs (the head's h), 4*UPC outputs; backward: K = 4*UPC own deltas, dhd outputs
    int K = bwd ? 4 * UPC : dhd, NOUT = bwd ? dhd : 4 * UPC;
    int NOUTp = (NOUT + 1) & ~1;
    // wide outputs: four columns per thread (fewest shared-memory wavefronts per FMA) on as many k-slices as the
    // partial buffer affords, even though that leaves threads idle in the mat-vec (6.09 vs 6.44 us per backward
    // step at 4 x 256-unit heads); narrow outputs: column pairs
    int CPT = 2;
    if (NOUTp % 4 == 0 && NOUTp >= 128) CPT = 4;  // forward 4.77 vs 5.09, backward 6.09 vs 6.44 us per step at 4 x 256-unit heads
    int ncols = NOUTp / CPT;
    int KS = kThreads / ncols;
    if (KS < 1) KS = 1;
    if (KS > 16) KS = 16;
    if (KS > K) KS = K;
    if (CPT == 4 && bwd && KS > 4) KS = 4;
    if (CPT == 4 && !bwd && KS > 8) KS = 8;
    out->BG = BG; out->CS = CS; out->UPC = UPC; out->KS = KS; out->CPT = CPT;
    if (bwd) {
        out->blay = bw_layout(K, NOUTp, BG, KS, UPC, CS);
        out->total = out->blay.total;
    } else {
        out->lay = smem_layout(K, NOUT, BG, KS, UPC, 3);
        out->total = out->lay.total;
    }
    return out->total <= kSmemCap;
}

// Cluster size for a fixed batch group: the widest (<= 8, the portable limit) that keeps >= 8 units
// per CTA and the whole grid within the SM count; failing that, the narrowest whose slice fits.
static bool geometry_for(int BG, int B, int NH, int dhd, bool bwd, Geo* out) {
    int nbg = (B + BG - 1) / BG;
    for (int CS = 8; CS >= 1; CS /= 2)
        if ((dhd / CS >= 8 || CS == 1) && NH * nbg * CS <= sm_count() && fits(BG, CS, dhd, bwd, out)) return true;
    for (int CS = 1; CS <= 8; CS *= 2)
        if (fits(BG, CS, dhd, bwd, out)) return true;
    return false;
}

// Clusters of this geometry that can be resident at once (GPC fragmentation makes this less than
// SMs / CS). The attribute call and the occupancy query cost milliseconds on the host, so the
// answer is cached per (kernel, device, cluster size, shared-memory size).
template <int BG>
static int coresident(bool bwd, const Geo& g, int* out) {
    const void* kern = bwd ? (const void*)slstm_bw_cluster<BG> : (const void*)slstm_fw_cluster<BG>;
    static std::atomic<unsigned long long> key_of[2][64];
    static std::atomic<int> val_of[2][64];
    int dev = 0;
    XL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    const unsigned long long key = ((unsigned long long)g.total << 8) | (unsigned)g.CS;
    if (key_of[bwd][dev].load() == key) { *out = val_of[bwd][dev].load(); return XLSTM_OK; }
    XL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.total));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g.CS);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = g.total;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    XL_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (getenv("XLSTM_DEBUG"))
        fprintf(stderr, "[xlstm] slstm %s: BG=%d CS=%d UPC=%d KS=%d CPT=%d smem=%zu clusters co-resident=%d\n", bwd ? "bw" : "fw",
                BG, g.CS, g.UPC, g.KS, g.CPT, g.total, n);
    val_of[bwd][dev].store(n);
    key_of[bwd][dev].store(key);
    *out = n;
    return XLSTM_OK;
}

template <int BG>
static int launch(cudaStream_t st, bool bwd, const SlstmArgs& a, const Geo& g) {
    int nbg = (a.B + BG - 1) / BG;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.NH * nbg * g.CS));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = g.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (bwd) XL_CUDA(cudaLaunchKernelEx(&cfg, slstm_bw_cluster<BG>, a, g.blay));
    else XL_CUDA(cudaLaunchKernelEx(&cfg, slstm_fw_cluster<BG>, a, g.lay));
    count_launch();
    return XLSTM_OK;
}

static int coresident_any(int BG, bool bwd, const Geo& g, int* out) {
    switch (BG) {
        case 16: return coresident<16>(bwd, g, out);
        case 12: return coresident<12>(bwd, g, out);
        case 8: return coresident<8>(bwd, g, out);
        case 4: return coresident<4>(bwd, g, out);
        case 2: return coresident<2>(bwd, g, out);
        default: return coresident<1>(bwd, g, out);
    }
}

int* tc_status_ptr();

// Launch counter of the flagged exchange, one per device and shared by every instantiation of the grid kernels
// (they all tag words in the one exchange array). Twelve bits of it go into the tags; when they wrap, the array
// is cleared first, so a word left by an earlier launch can never carry the tag a later launch polls for.
static unsigned g_ll_epoch[64];

struct GridGeo {
    int BG, G, UPC, KS, CPT;
    GridSmem lay;
};

// Widest split of a head over CTAs (all heads together within the SM count) whose slice fits, then the
// largest batch sub-group that fits beside it.
static bool grid_geometry(int B, int NH, int dhd, bool bwd, GridGeo* out) {
    if (NH > 64) return false;
    int gmax = sm_count() / NH;
    if (gmax > dhd) gmax = dhd;
    for (int G = gmax; G >= 1; --G) {
        if (dhd % G) continue;
        const int UPC = dhd / G;
        const int K = bwd ? 4 * dhd : dhd, NOUT = bwd ? UPC : 4 * UPC, NOUTp = (NOUT + 1) & ~1;
        const int CPT = 2;
        const int ncols = NOUTp / CPT;
        int KS = kThreads / ncols;
        if (KS < 1) KS = 1;
        if (KS > 32) KS = 32;
        if (KS > K) KS = K;
        for (int BG = 8; BG >= 1; BG /= 2) {
            if (BG > 1 && BG / 2 >= B) continue;
            const int nsub = (B + BG - 1) / BG;
            GridSmem l = grid_layout(K, NOUTp, BG, KS, UPC, nsub * BG, bwd ? 3 : 4);
            if (l.total > kSmemCap) continue;
            out->BG = BG; out->G = G; out->UPC = UPC; out->KS = KS; out->CPT = CPT; out->lay = l;
            return true;
        }
    }
    return false;
}

template <int BG, bool LL>
static int launch_grid(cudaStream_t st, bool bwd, SlstmArgs a, const GridGeo& g) {
    const void* kern = (const void*)slstm_fw_grid<BG, LL>;
    // per device: barrier words' address, and whether the whole grid can be resident at once
    static std::atomic<unsigned long long> key_of[2][64];
    static GridSync* sync_of[64];
    static uint2* ll_of[64];
    int dev = 0;
    XL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    const int grid = a.NH * g.G;
    const unsigned long long key = ((unsigned long long)g.lay.total << 16) | (unsigned)grid;
    if (key_of[bwd][dev].load() != key) {
        XL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.lay.total));
        int per_sm = 0;
        XL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, g.lay.total));
        if (per_sm * sm_count() < grid) {
            set_error("slstm: %d CTAs of %zu bytes cannot be resident together", grid, g.lay.total);
            return XLSTM_DECLINED;
        }
        void* p = nullptr;
        XL_CUDA(cudaGetSymbolAddress(&p, g_slstm_sync));
        sync_of[dev] = (GridSync*)p;
        XL_CUDA(cudaGetSymbolAddress(&p, g_slstm_ll));
        ll_of[dev] = (uint2*)p;
        if (getenv("XLSTM_DEBUG"))
            fprintf(stderr, "[xlstm] slstm %s grid: G=%d UPC=%d BG=%d KS=%d CPT=%d smem=%zu CTAs=%d\n", bwd ? "bw" : "fw", g.G,
                    g.UPC, g.BG, g.KS, g.CPT, g.lay.total, grid);
        key_of[bwd][dev].store(key);
    }
    GridSync* gs = sync_of[dev];
    XL_CUDA(cudaMemsetAsync(gs, 0, sizeof(GridSync), st));
    a.CS = g.G; a.UPC = g.UPC; a.KS = g.KS; a.CPT = g.CPT;
    GridSmem lay = g.lay;
    int* status = tc_status_ptr();
    if (!status) return XLSTM_ERR_CUDA;
    uint2* ll = ll_of[dev];
    unsigned epoch = ++g_ll_epoch[dev];
    if ((epoch & 0xfffu) == 0) {
        XL_CUDA(cudaMemsetAsync(ll, 0, sizeof(g_slstm_ll), st));
        epoch = ++g_ll_epoch[dev];
    }
    a.epoch = epoch & 0xfffu;
    void* args[5] = {&a, &lay, &gs, &status, &ll};
    XL_CUDA(cudaLaunchCooperativeKernel(kern, dim3((unsigned)grid), dim3(kThreads), args, g.lay.total, st));
    count_launch();
    return XLSTM_OK;
}

// Geometry of the partial-sum backward: the same split of a head over CTAs, K = 4*UPC own deltas, output dhd wide.
static bool grid_geometry_ps(int B, int NH, int dhd, GridGeo* out) {
    if (NH > 64 || dhd % 4) return false;
    int gmax = sm_count() / NH;
    if (gmax > dhd) gmax = dhd;
    for (int G = gmax; G >= 1; --G) {
        if (dhd % G) continue;
        const int UPC = dhd / G, K = 4 * UPC, ncols = dhd / 4;
        int KS = kThreads / ncols;
        if (KS < 1) KS = 1;
        if (KS > K) KS = K;
        for (int BG = 8; BG >= 1; BG /= 2) {
            if (BG > 1 && BG / 2 >= B) continue;
            const int nsub = (B + BG - 1) / BG;
            GridSmem l = grid_layout(K, dhd, BG, KS, UPC, nsub * BG, 3);
            if (l.total > kSmemCap) continue;
            out->BG = BG; out->G = G; out->UPC = UPC; out->KS = KS; out->CPT = 4; out->lay = l;
            return true;
        }
    }
    return false;
}

template <int BG>
static int launch_grid_ps(cudaStream_t st, SlstmArgs a, const GridGeo& g) {
    const void* kern = (const void*)slstm_bw_grid_ps<BG>;
    static std::atomic<unsigned long long> key_of[64];
    static GridSync* sync_of[64];
    static float* xch_of[64];
    static size_t xch_bytes[64];
    int dev = 0;
    XL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    const int grid = a.NH * g.G;
    const unsigned long long key = ((unsigned long long)g.lay.total << 16) | (unsigned)grid;
    if (key_of[dev].load() != key) {
        XL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.lay.total));
        int per_sm = 0;
        XL_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, g.lay.total));
        if (per_sm * sm_count() < grid) {
            set_error("slstm: %d CTAs of %zu bytes cannot be resident together", grid, g.lay.total);
            return XLSTM_DECLINED;
        }
        void* p = nullptr;
        XL_CUDA(cudaGetSymbolAddress(&p, g_slstm_sync));
        sync_of[dev] = (GridSync*)p;
        if (getenv("XLSTM_DEBUG"))
            fprintf(stderr, "[xlstm] slstm bw grid (partial sums): G=%d UPC=%d BG=%d KS=%d smem=%zu CTAs=%d\n", g.G, g.UPC, g.BG,
                    g.KS, g.lay.total, grid);
        key_of[dev].store(key);
    }
    // exchange buffer: two step parities x every CTA's [B, dhd] partials; transient scratch the library keeps
    // (grow-only, one per device; the reference's ops keep such scratch per stream, src/gpu/ops.rs:463-474)
    const size_t need = (size_t)2 * grid * a.B * a.dhd * sizeof(float);
    if (xch_bytes[dev] < need) {
        if (xch_of[dev]) XL_CUDA(cudaFree(xch_of[dev]));
        xch_of[dev] = nullptr; xch_bytes[dev] = 0;
        void* p = nullptr;
        XL_CUDA(cudaMalloc(&p, need));
        xch_of[dev] = (float*)p; xch_bytes[dev] = need;
    }
    GridSync* gs = sync_of[dev];
    XL_CUDA(cudaMemsetAsync(gs, 0, sizeof(GridSync), st));
    a.CS = g.G; a.UPC = g.UPC; a.KS = g.KS; a.CPT = g.CPT;
    GridSmem lay = g.lay;
    int* status = tc_status_ptr();
    if (!status) return XLSTM_ERR_CUDA;
    float* xch = xch_of[dev];
    void* args[5] = {&a, &lay, &gs, &status, &xch};
    XL_CUDA(cudaLaunchCooperativeKernel(kern, dim3((unsigned)grid), dim3(kThreads), args, g.lay.total, st));
    count_launch();
    return XLSTM_OK;
}

static int run_grid(cudaStream_t st, bool bwd, const SlstmArgs& a) {
    if (bwd) {
        GridGeo gp;
        if (!grid_geometry_ps(a.B, a.NH, a.dhd, &gp)) {
            set_error("slstm_bw: recurrent slice for %d units per head over %d heads does not fit the GPU's shared memory", a.dhd, a.NH);
            return XLSTM_DECLINED;
        }
        switch (gp.BG) {
            case 8: return launch_grid_ps<8>(st, a, gp);
            case 4: return launch_grid_ps<4>(st, a, gp);
            case 2: return launch_grid_ps<2>(st, a, gp);
            default: return launch_grid_ps<1>(st, a, gp);
        }
    }
    GridGeo g;
    if (!grid_geometry(a.B, a.NH, a.dhd, bwd, &g)) {
        set_error("slstm: recurrent slice for %d units per head over %d heads does not fit the GPU's shared memory", a.dhd, a.NH);
        return XLSTM_DECLINED;
    }
    // Flagged exchange: forward only, and only where it measured faster than the counter barrier, which is when
    // the whole batch is one sub-group (512-unit heads at B = 8: 4.3 vs 5.1 us per step; with several
    // sub-groups per step the polling costs more than the one barrier it saves). Its two buffers must fit the
    // built-in array, the tags need T < 2^20, and the second step is what orders the carried h (see the kernel).
    const bool ll = !bwd && a.B <= g.BG && (size_t)2 * a.B * a.H <= kLLWords && a.T >= 2 && a.T < (1 << 20);
    switch (g.BG) {
        case 8: return ll ? launch_grid<8, true>(st, bwd, a, g) : launch_grid<8, false>(st, bwd, a, g);
        case 4: return ll ? launch_grid<4, true>(st, bwd, a, g) : launch_grid<4, false>(st, bwd, a, g);
        case 2: return ll ? launch_grid<2, true>(st, bwd, a, g) : launch_grid<2, false>(st, bwd, a, g);
        default: return ll ? launch_grid<1, true>(st, bwd, a, g) : launch_grid<1, false>(st, bwd, a, g);
    }
}

// Batch group: start from the largest of 8/4/2/1 that does not pad the batch by 2x or more, and grow
// it (12, 16) while the clusters it needs exceed what can be resident at once: a second wave of
// clusters doubles the time of a latency-bound loop, a wider batch group costs far less.
static int run(cudaStream_t st, bool bwd, SlstmArgs a) {
    const int cand[6] = {1, 2, 4, 8, 12, 16};
    int first = 0;
    for (int i = 3; i >= 0; --i)
        if (cand[i] == 1 || cand[i] / 2 < a.B) { first = i; break; }
    Geo chosen;
    int chosen_bg = 0;
    for (int i = first; i < 6; ++i) {
        const int BG = cand[i];
        if (i > first && BG / 2 >= a.B) break;
        Geo g;
        if (!geometry_for(BG, a.B, a.NH, a.dhd, bwd, &g)) continue;
        int maxc = 0;
        int rc = coresident_any(BG, bwd, g, &maxc);
        if (rc) return rc;
        if (maxc < 1) continue;
        if (chosen_bg == 0) { chosen = g; chosen_bg = BG; }  // fallback: runs in waves
        if (a.NH * ((a.B + BG - 1) / BG) <= maxc) { chosen = g; chosen_bg = BG; break; }
    }
    if (chosen_bg == 0) return run_grid(st, bwd, a);  // too wide for a cluster: split the head over the whole GPU
    const Geo& g = chosen;
    a.CS = g.CS; a.UPC = g.UPC; a.KS = g.KS; a.CPT = g.CPT;
    switch (chosen_bg) {
        case 16: return launch<16>(st, bwd, a, g);
        case 12: return launch<12>(st, bwd, a, g);
        case 8: return launch<8>(st, bwd, a, g);
        case 4: return launch<4>(st, bwd, a, g);
        case 2: return launch<2>(st, bwd, a, g);
        default: return launch<1>(st, bwd, a, g);
    }
}

}  // namespace xl

using namespace xl;

static int check_common(const char* who, const float* wh, const float* g, const xlstm_slstm_slabs* s, int B, int H,
                        int NH, int T) {
    XL_CHECK_ARG(wh && g && s, "%s: null pointer", who);
    XL_CHECK_ARG(B > 0 && H > 0 && NH > 0 && T >= 0 && H % NH == 0, "%s: bad shape B=%d H=%d NH=%d T=%d", who, B, H, NH, T);
    XL_CHECK_ARG(s->c_prev && s->n_prev && s->ipr && s->fpr && s->c && s->n && s->zt && s->ot && s->h_prev,
                 "%s: null slab pointer", who);
    return XLSTM_OK;
}

extern "C" int xlstm_slstm_fw(void* stream, const float* wh, float* g, const float* bcat, float* c, float* n,
                              float* m, float* h, float* out, const xlstm_slstm_slabs* slabs, int B, int H, int NH,
                              int T, int carry, unsigned flags) {
    (void)flags;
    int rc = check_common("slstm_fw", wh, g, slabs, B, H, NH, T);
    if (rc) return rc;
    XL_CHECK_ARG(bcat && c && n && m && h && out, "slstm_fw: null pointer");
    SlstmArgs a = {};
    a.wh = wh; a.g = g; a.bcat = bcat; a.c = c; a.n = n; a.m = m; a.h = h; a.out = out; a.s = *slabs;
    a.B = B; a.H = H; a.NH = NH; a.T = T; a.carry = carry; a.dhd = H / NH;
    return run((cudaStream_t)stream, false, a);
}

extern "C" int xlstm_slstm_bw(void* stream, const float* wh, const float* dy, float* g, float* dh, float* dc,
                              float* dn, const xlstm_slstm_slabs* slabs, int B, int H, int NH, int T, int carry,
                              unsigned flags) {
    (void)flags;
    int rc = check_common("slstm_bw", wh, g, slabs, B, H, NH, T);
    if (rc) return rc;
    XL_CHECK_ARG(dy && dh && dc && dn, "slstm_bw: null pointer");
    SlstmArgs a = {};
    a.wh = wh; a.g = g; a.dy = dy; a.dh = dh; a.dc = dc; a.dn = dn; a.s = *slabs;
    a.B = B; a.H = H; a.NH = NH; a.T = T; a.carry = carry; a.dhd = H / NH;
    return run((cudaStream_t)stream, true, a);
}
