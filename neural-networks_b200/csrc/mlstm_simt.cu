// Chunkwise mLSTM core on CUDA cores (fp32 arithmetic throughout).
//
// This is the engine's exact-arithmetic path: it serves fp32 storage (where results must
// track the reference to 1e-4) and every shape the tensor-core kernels do not cover. One
// CTA owns one (batch, head) pair and walks its chunks in order with the matrix memory C
// (forward) or its gradient dC (backward) resident in shared memory, so chunk states
// never round-trip through HBM inside a call.
//
// Math: the chunkwise form of src/gpu/cuda/mlstm_fused.cu:12-19 (forward) and the
// reference kernels' backward (mlstm_fused.cu:256-293, 830-858, 1036-1050, 1132-1190,
// 1272-1333), with the stabiliser m held constant in the backward.
#include "common.cuh"
#include "mlstm.cuh"

namespace xl {

static constexpr int kThreads = 256;
static constexpr int kWarps = kThreads / 32;

template <typename T>
__device__ __forceinline__ int row_pad() { return sizeof(T) == 4 ? 1 : 2; }

// Shared-memory carve-up helper.
struct Carver {
    unsigned char* p;
    __device__ Carver(void* base) : p((unsigned char*)base) {}
    template <typename U>
    __device__ U* take(size_t n) {
        U* r = (U*)p;
        p += (n * sizeof(U) + 15) / 16 * 16;
        return r;
    }
};

template <typename T>
size_t fw_smem_bytes(int L, int dqk, int dhv) {
    int pad = sizeof(T) == 4 ? 1 : 2;
    auto a16 = [](size_t x) { return (x + 15) / 16 * 16; };
    size_t s = 0;
    s += 2 * a16((size_t)L * (dqk + pad) * sizeof(T));  // Q, K
    s += a16((size_t)L * (dhv + pad) * sizeof(T));      // V
    s += a16((size_t)dhv * (dqk + 1) * 4);              // C
    s += a16((size_t)dqk * 4);                          // n
    s += a16((size_t)L * (L + 1) * 4);                  // S
    s += 8 * a16((size_t)L * 4) + 256;                  // vectors + scalars
    return s;
}

template <typename T>
size_t bw_smem_bytes(int L, int dqk, int dhv) {
    int pad = sizeof(T) == 4 ? 1 : 2;
    auto a16 = [](size_t x) { return (x + 15) / 16 * 16; };
    size_t s = 0;
    s += 2 * a16((size_t)L * (dqk + pad) * sizeof(T));  // Q, K
    s += a16((size_t)L * (dhv + pad) * sizeof(T));      // V
    s += a16((size_t)L * (dhv + 1) * 4);                // dN
    s += a16((size_t)dhv * (dqk + 1) * 4);              // dC
    s += a16((size_t)dqk * 4);                          // dn
    s += 3 * a16((size_t)L * (L + 1) * 4);              // DS, dS, P
    s += 14 * a16((size_t)L * 4) + 256;                 // vectors + scalars
    return s;
}

// ---------------------------------------------------------------------------------------
// Forward. grid = B*H, block = 256.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) mlstm_fw_simt(MlstmFwArgs a) {
    const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = a.L, dqk = a.dqk, dhv = a.dhv, T_ = a.T, H = a.H;
    const int pq = dqk + row_pad<T>(), pv = dhv + row_pad<T>(), pc = dqk + 1, ps = L + 1;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    Carver cv(smem_raw);
    T* sQ = cv.take<T>((size_t)L * pq);
    T* sK = cv.take<T>((size_t)L * pq);
    T* sV = cv.take<T>((size_t)L * pv);
    float* sC = cv.take<float>((size_t)dhv * pc);
    float* sn = cv.take<float>(dqk);
    float* sS = cv.take<float>((size_t)L * ps);
    float* sfc = cv.take<float>(L);
    float* sig = cv.take<float>(L);
    float* slf = cv.take<float>(L);
    float* sm = cv.take<float>(L);
    float* sb = cv.take<float>(L);
    float* sa = cv.take<float>(L);
    float* sipsi = cv.take<float>(L);
    float* sscal = cv.take<float>(8);  // [0]=m_prev, [1]=g

    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    T* ytil = (T*)a.ytil;

    // initial state
    for (int i = tid; i < dhv * dqk; i += kThreads) {
        int vv = i / dqk, c = i % dqk;
        sC[vv * pc + c] = a.cC ? a.cC[(size_t)bh * dhv * dqk + i] : 0.f;
    }
    for (int c = tid; c < dqk; c += kThreads) sn[c] = a.cn ? a.cn[(size_t)bh * dqk + c] : 0.f;
    if (tid == 0) sscal[0] = a.cm ? a.cm[bh] : 0.f;
    __syncthreads();

    for (int ch = 0; ch < a.NC; ++ch) {
        const int t0 = ch * L, Lc = min(L, T_ - t0);
        // record the state entering this chunk
        if (a.savedC) {
            float* dst = a.savedC + ((size_t)bh * a.NC + ch) * dhv * dqk;
            for (int i = tid; i < dhv * dqk; i += kThreads) dst[i] = sC[(i / dqk) * pc + (i % dqk)];
            float* dn_ = a.savedn + ((size_t)bh * a.NC + ch) * dqk;
            for (int c = tid; c < dqk; c += kThreads) dn_[c] = sn[c];
        }
        // tiles
        for (int i = tid; i < Lc * dqk; i += kThreads) {
            int t = i / dqk, c = i % dqk;
            size_t gidx = (((size_t)b * T_ + t0 + t) * H + h) * dqk + c;
            sQ[t * pq + c] = q[gidx];
            sK[t * pq + c] = k[gidx];
        }
        for (int i = tid; i < Lc * dhv; i += kThreads) {
            int t = i / dhv, c = i % dhv;
            sV[t * pv + c] = v[(((size_t)b * T_ + t0 + t) * H + h) * dhv + c];
        }
        if (tid < Lc) {
            size_t gi = ((size_t)b * T_ + t0 + tid) * H + h;
            slf[tid] = log_sigmoid(a.fg[gi]);
            sig[tid] = a.ig[gi];
        }
        __syncthreads();
        // gate scans: fc = cumsum(lf); m_t = fc_t + max(m_prev, max_{j<=t}(i_j - fc_j))
        if (tid == 0) {
            float mprev = sscal[0], run = 0.f, u = -INFINITY;
            for (int t = 0; t < Lc; ++t) {
                run += slf[t];
                sfc[t] = run;
                u = fmaxf(u, sig[t] - run);
                float mt = run + fmaxf(mprev, u);
                sm[t] = mt;
                sb[t] = expf(run + mprev - mt);
            }
            float mL = sm[Lc - 1], fL = sfc[Lc - 1];
            for (int j = 0; j < Lc; ++j) sa[j] = expf(fL - sfc[j] + sig[j] - mL);
            sscal[1] = expf(fL + mprev - mL);
            sscal[2] = mL;
        }
        __syncthreads();
        if (!a.states_only) {
            // S_tj = (q_t·k_j) * exp(fc_t - fc_j + i_j - m_t), j <= t
            for (int i = tid; i < Lc * Lc; i += kThreads) {
                int t = i / Lc, j = i % Lc;
                float s = 0.f;
                if (j <= t) {
                    const T* qr = sQ + t * pq;
                    const T* kr = sK + j * pq;
                    for (int c = 0; c < dqk; ++c) s += (float)qr[c] * (float)kr[c];
                    s *= expf(sfc[t] - sfc[j] + sig[j] - sm[t]);
                }
                sS[t * ps + j] = s;
            }
            __syncthreads();
            // qn_t = rowsum(S) + b_t (q_t·n);  psi_t = max(|qn_t|, exp(-m_t))
            for (int t = warp; t < Lc; t += kWarps) {
                float acc = 0.f;
                for (int j = lane; j <= t; j += 32) acc += sS[t * ps + j];
                float qn_ = 0.f;
                for (int c = lane; c < dqk; c += 32) qn_ += (float)sQ[t * pq + c] * sn[c];
                acc = warp_sum(acc);
                qn_ = warp_sum(qn_);
                if (lane == 0) {
                    float qn = acc + sb[t] * qn_;
                    float psi = fmaxf(fabsf(qn), expf(-sm[t]));
                    sipsi[t] = 1.f / psi;
                    size_t o = (size_t)bh * T_ + t0 + t;
                    a.msv[o] = sm[t];
                    a.psiv[o] = psi;
                    a.qnv[o] = qn;
                }
            }
            __syncthreads();
            // ytil_tv = (sum_j S_tj v_jv + b_t sum_c q_tc C_vc) / psi_t
            for (int t = warp; t < Lc; t += kWarps) {
                for (int vv = lane; vv < dhv; vv += 32) {
                    float acc = 0.f;
                    for (int j = 0; j <= t; ++j) acc += sS[t * ps + j] * (float)sV[j * pv + vv];
                    float inter = 0.f;
                    const float* cr = sC + vv * pc;
                    const T* qr = sQ + t * pq;
                    for (int c = 0; c < dqk; ++c) inter += (float)qr[c] * cr[c];
                    float y = (acc + sb[t] * inter) * sipsi[t];
                    stf(ytil, (((size_t)b * T_ + t0 + t) * H + h) * dhv + vv, y);
                }
            }
            __syncthreads();
        }
        // state: C_vc = g C_vc + sum_j a_j v_jv k_jc ; n_c = g n_c + sum_j a_j k_jc
        {
            float g = sscal[1];
            for (int i = tid; i < dhv * dqk; i += kThreads) {
                int vv = i / dqk, c = i % dqk;
                float acc = 0.f;
                for (int j = 0; j < Lc; ++j) acc += sa[j] * (float)sV[j * pv + vv] * (float)sK[j * pq + c];
                sC[vv * pc + c] = g * sC[vv * pc + c] + acc;
            }
            for (int c = tid; c < dqk; c += kThreads) {
                float acc = 0.f;
                for (int j = 0; j < Lc; ++j) acc += sa[j] * (float)sK[j * pq + c];
                sn[c] = g * sn[c] + acc;
            }
            __syncthreads();
            if (tid == 0) sscal[0] = sscal[2];
            __syncthreads();
        }
    }
    if (a.oC)
        for (int i = tid; i < dhv * dqk; i += kThreads)
            a.oC[(size_t)bh * dhv * dqk + i] = sC[(i / dqk) * pc + (i % dqk)];
    if (a.on)
        for (int c = tid; c < dqk; c += kThreads) a.on[(size_t)bh * dqk + c] = sn[c];
    if (a.om && tid == 0) a.om[bh] = sscal[0];
}

// ---------------------------------------------------------------------------------------
// Backward. grid = B*H, block = 256. Chunks are walked right to left with dC, dn resident
// in shared memory; the state that ENTERED each chunk is read from the record the forward
// (or the recompute pass) wrote.
// ---------------------------------------------------------------------------------------
template <typename T, typename G>
__global__ void __launch_bounds__(kThreads) mlstm_bw_simt(MlstmBwArgs a) {
    const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = a.L, dqk = a.dqk, dhv = a.dhv, T_ = a.T, H = a.H;
    const int pq = dqk + row_pad<T>(), pv = dhv + row_pad<T>(), pc = dqk + 1, ps = L + 1, pn = dhv + 1;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    Carver cv(smem_raw);
    T* sQ = cv.take<T>((size_t)L * pq);
    T* sK = cv.take<T>((size_t)L * pq);
    T* sV = cv.take<T>((size_t)L * pv);
    float* sdN = cv.take<float>((size_t)L * pn);
    float* sdC = cv.take<float>((size_t)dhv * pc);
    float* sdn = cv.take<float>(dqk);
    float* sDS = cv.take<float>((size_t)L * ps);
    float* sdS = cv.take<float>((size_t)L * ps);
    float* sP = cv.take<float>((size_t)L * ps);
    float* sfc = cv.take<float>(L);
    float* sig = cv.take<float>(L);
    float* sfg = cv.take<float>(L);
    float* sm = cv.take<float>(L);
    float* sb = cv.take<float>(L);
    float* sa = cv.take<float>(L);
    float* sdqn = cv.take<float>(L);
    float* sda = cv.take<float>(L);
    float* sdb = cv.take<float>(L);
    float* srow = cv.take<float>(L);
    float* scol = cv.take<float>(L);
    float* sred = cv.take<float>(32);
    float* sscal = cv.take<float>(8);  // [0]=g, [1]=dg

    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    const T* ytil = (const T*)a.ytil;
    const G* dy = (const G*)a.dytil;
    G* dq = (G*)a.dq;
    G* dk = (G*)a.dk;
    G* dv = (G*)a.dv;

    for (int i = tid; i < dhv * dqk; i += kThreads)
        sdC[(i / dqk) * pc + (i % dqk)] = a.cdC ? a.cdC[(size_t)bh * dhv * dqk + i] : 0.f;
    for (int c = tid; c < dqk; c += kThreads) sdn[c] = a.cdn ? a.cdn[(size_t)bh * dqk + c] : 0.f;
    __syncthreads();

    for (int ch = a.NC - 1; ch >= 0; --ch) {
        const int t0 = ch * L, Lc = min(L, T_ - t0);
        const float* Ck = a.savedC + ((size_t)bh * a.NC + ch) * dhv * dqk;
        const float* nk = a.savedn + ((size_t)bh * a.NC + ch) * dqk;
        for (int i = tid; i < Lc * dqk; i += kThreads) {
            int t = i / dqk, c = i % dqk;
            size_t gidx = (((size_t)b * T_ + t0 + t) * H + h) * dqk + c;
            sQ[t * pq + c] = q[gidx];
            sK[t * pq + c] = k[gidx];
        }
        for (int i = tid; i < Lc * dhv; i += kThreads) {
            int t = i / dhv, c = i % dhv;
            sV[t * pv + c] = v[(((size_t)b * T_ + t0 + t) * H + h) * dhv + c];
        }
        if (tid < Lc) {
            size_t gi = ((size_t)b * T_ + t0 + tid) * H + h;
            sfg[tid] = a.fg[gi];
            sig[tid] = a.ig[gi];
            sm[tid] = a.msv[(size_t)bh * T_ + t0 + tid];
        }
        __syncthreads();
        if (tid == 0) {
            float mprev = (ch == 0) ? (a.cm ? a.cm[bh] : 0.f) : a.msv[(size_t)bh * T_ + t0 - 1];
            float run = 0.f;
            for (int t = 0; t < Lc; ++t) {
                run += log_sigmoid(sfg[t]);
                sfc[t] = run;
                sb[t] = expf(run + mprev - sm[t]);
            }
            float mL = sm[Lc - 1], fL = sfc[Lc - 1];
            for (int j = 0; j < Lc; ++j) sa[j] = expf(fL - sfc[j] + sig[j] - mL);
            sscal[0] = expf(fL + mprev - mL);
        }
        // dN_t = dy_t / psi_t ; dqn_t = sign(qn)(-sum_v dy ytil / psi) where |qn| > exp(-m)
        for (int t = warp; t < Lc; t += kWarps) {
            size_t o = (size_t)bh * T_ + t0 + t;
            float ipsi = 1.f / a.psiv[o];
            float acc = 0.f;
            size_t base = (((size_t)b * T_ + t0 + t) * H + h) * dhv;
            for (int vv = lane; vv < dhv; vv += 32) {
                float d = ldf(dy, base + vv);
                acc += d * ldf(ytil, base + vv);
                sdN[t * pn + vv] = d * ipsi;
            }
            acc = warp_sum(acc);
            if (lane == 0) {
                float qn = a.qnv[o];
                float r = 0.f;
                if (fabsf(qn) > expf(-a.msv[o])) r = (qn > 0.f ? 1.f : -1.f) * (-acc * ipsi);
                sdqn[t] = r;
            }
        }
        __syncthreads();
        // S, Dbar, DS, dds, dS, P
        for (int i = tid; i < Lc * Lc; i += kThreads) {
            int t = i / Lc, j = i % Lc;
            float DS = 0.f, dS = 0.f, P = 0.f;
            if (j <= t) {
                const T* qr = sQ + t * pq;
                const T* kr = sK + j * pq;
                float s = 0.f;
                for (int c = 0; c < dqk; ++c) s += (float)qr[c] * (float)kr[c];
                float D = expf(sfc[t] - sfc[j] + sig[j] - sm[t]);
                float dds = sdqn[t];
                const float* nr = sdN + t * pn;
                const T* vr = sV + j * pv;
                for (int c = 0; c < dhv; ++c) dds += nr[c] * (float)vr[c];
                DS = D * s;
                dS = dds * D;
                P = dds * DS;
            }
            sDS[t * ps + j] = DS;
            sdS[t * ps + j] = dS;
            sP[t * ps + j] = P;
        }
        __syncthreads();
        if (tid < Lc) {
            float r = 0.f, c_ = 0.f;
            for (int j = 0; j <= tid; ++j) r += sP[tid * ps + j];
            for (int t = tid; t < Lc; ++t) c_ += sP[t * ps + tid];
            srow[tid] = r;
            scol[tid] = c_;
        }
        // dg = <dC, C_k> + dn·n_k
        {
            float acc = 0.f;
            for (int i = tid; i < dhv * dqk; i += kThreads) acc += sdC[(i / dqk) * pc + (i % dqk)] * Ck[i];
            for (int c = tid; c < dqk; c += kThreads) acc += sdn[c] * nk[c];
            acc = block_sum(acc, sred);
            if (tid == 0) sscal[1] = acc;
        }
        // dV_jv = sum_{t>=j} DS_tj dN_tv + a_j sum_c k_jc dC_vc
        for (int j = warp; j < Lc; j += kWarps) {
            for (int vv = lane; vv < dhv; vv += 32) {
                float acc = 0.f;
                for (int t = j; t < Lc; ++t) acc += sDS[t * ps + j] * sdN[t * pn + vv];
                float inter = 0.f;
                const T* kr = sK + j * pq;
                const float* dcr = sdC + vv * pc;
                for (int c = 0; c < dqk; ++c) inter += (float)kr[c] * dcr[c];
                stf(dv, (((size_t)b * T_ + t0 + j) * H + h) * dhv + vv, acc + sa[j] * inter);
            }
        }
        // dQ_tc = sum_{j<=t} dS_tj k_jc + b_t (sum_v dN_tv C_vc + dqn_t n_c);  db_t = inter_t · q_t
        for (int t = warp; t < Lc; t += kWarps) {
            float dbacc = 0.f;
            for (int c = lane; c < dqk; c += 32) {
                float acc = 0.f;
                for (int j = 0; j <= t; ++j) acc += sdS[t * ps + j] * (float)sK[j * pq + c];
                float inter = sdqn[t] * nk[c];
                const float* nr = sdN + t * pn;
                for (int vv = 0; vv < dhv; ++vv) inter += nr[vv] * Ck[(size_t)vv * dqk + c];
                stf(dq, (((size_t)b * T_ + t0 + t) * H + h) * dqk + c, acc + sb[t] * inter);
                dbacc += inter * (float)sQ[t * pq + c];
            }
            dbacc = warp_sum(dbacc);
            if (lane == 0) sdb[t] = dbacc;
        }
        // dK_jc = sum_{t>=j} dS_tj q_tc + a_j (sum_v v_jv dC_vc + dn_c);  da_j = inter_j · k_j
        for (int j = warp; j < Lc; j += kWarps) {
            float daacc = 0.f;
            for (int c = lane; c < dqk; c += 32) {
                float acc = 0.f;
                for (int t = j; t < Lc; ++t) acc += sdS[t * ps + j] * (float)sQ[t * pq + c];
                float inter = sdn[c];
                const T* vr = sV + j * pv;
                for (int vv = 0; vv < dhv; ++vv) inter += (float)vr[vv] * sdC[vv * pc + c];
                stf(dk, (((size_t)b * T_ + t0 + j) * H + h) * dqk + c, acc + sa[j] * inter);
                daacc += inter * (float)sK[j * pq + c];
            }
            daacc = warp_sum(daacc);
            if (lane == 0) sda[j] = daacc;
        }
        __syncthreads();
        // gate gradients (fixed serial order)
        if (tid == 0) {
            float g = sscal[0], dg = sscal[1];
            float tail = 0.f;
            for (int j = 0; j < Lc; ++j) tail += sda[j] * sa[j];
            tail += dg * g;
            float run = 0.f;
            for (int r = Lc - 1; r >= 0; --r) {
                float dfc = srow[r] - scol[r] + sdb[r] * sb[r] - sda[r] * sa[r];
                if (r == Lc - 1) dfc += tail;
                run += dfc;
                size_t gi = ((size_t)b * T_ + t0 + r) * H + h;
                a.dfg[gi] = run * (1.f - stable_sigmoid(sfg[r]));
                a.dig[gi] = scol[r] + sda[r] * sa[r];
            }
        }
        // dC_vc = g dC_vc + sum_t b_t dN_tv q_tc ; dn_c = g dn_c + sum_t b_t dqn_t q_tc
        {
            float g = sscal[0];
            for (int i = tid; i < dhv * dqk; i += kThreads) {
                int vv = i / dqk, c = i % dqk;
                float acc = 0.f;
                for (int t = 0; t < Lc; ++t) acc += sb[t] * sdN[t * pn + vv] * (float)sQ[t * pq + c];
                sdC[vv * pc + c] = g * sdC[vv * pc + c] + acc;
            }
            for (int c = tid; c < dqk; c += kThreads) {
                float acc = 0.f;
                for (int t = 0; t < Lc; ++t) acc += sb[t] * sdqn[t] * (float)sQ[t * pq + c];
                sdn[c] = g * sdn[c] + acc;
            }
        }
        __syncthreads();
    }
    if (a.odC)
        for (int i = tid; i < dhv * dqk; i += kThreads)
            a.odC[(size_t)bh * dhv * dqk + i] = sdC[(i / dqk) * pc + (i % dqk)];
    if (a.odn)
        for (int c = tid; c < dqk; c += kThreads) a.odn[(size_t)bh * dqk + c] = sdn[c];
}

// ---------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------
static const size_t kMaxSmem = 227 * 1024;

template <typename T>
static int launch_fw(cudaStream_t st, const MlstmFwArgs& a) {
    size_t smem = fw_smem_bytes<T>(a.L, a.dqk, a.dhv);
    if (smem > kMaxSmem) {
        set_error("mlstm_fw (CUDA-core path): L=%d dqk=%d dhv=%d needs %zu B shared memory", a.L, a.dqk, a.dhv, smem);
        return XLSTM_DECLINED;
    }
    XL_CUDA(cudaFuncSetAttribute(mlstm_fw_simt<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mlstm_fw_simt<T><<<a.B * a.H, kThreads, smem, st>>>(a);
    XL_LAUNCH_OK("mlstm_fw_simt");
    return XLSTM_OK;
}

int mlstm_fw_simt_launch(cudaStream_t st, const MlstmFwArgs& a, int dtype) {
    return dtype == XLSTM_BF16 ? launch_fw<bf16>(st, a) : launch_fw<float>(st, a);
}

bool mlstm_simt_supported(int L, int dqk, int dhv, int dtype) {
    size_t f = dtype == XLSTM_BF16 ? fw_smem_bytes<bf16>(L, dqk, dhv) : fw_smem_bytes<float>(L, dqk, dhv);
    size_t b = dtype == XLSTM_BF16 ? bw_smem_bytes<bf16>(L, dqk, dhv) : bw_smem_bytes<float>(L, dqk, dhv);
    return f <= kMaxSmem && b <= kMaxSmem;
}

template <typename T, typename G>
static int launch_bw(cudaStream_t st, const MlstmBwArgs& a) {
    size_t smem = bw_smem_bytes<T>(a.L, a.dqk, a.dhv);
    if (smem > kMaxSmem) {
        set_error("mlstm_bw (CUDA-core path): L=%d dqk=%d dhv=%d needs %zu B shared memory", a.L, a.dqk, a.dhv, smem);
        return XLSTM_DECLINED;
    }
    XL_CUDA(cudaFuncSetAttribute(mlstm_bw_simt<T, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mlstm_bw_simt<T, G><<<a.B * a.H, kThreads, smem, st>>>(a);
    XL_LAUNCH_OK("mlstm_bw_simt");
    return XLSTM_OK;
}

int mlstm_bw_simt_launch(cudaStream_t st, const MlstmBwArgs& a, int dtype, int gdtype) {
    if (dtype == XLSTM_BF16)
        return gdtype == XLSTM_BF16 ? launch_bw<bf16, bf16>(st, a) : launch_bw<bf16, float>(st, a);
    return gdtype == XLSTM_BF16 ? launch_bw<float, bf16>(st, a) : launch_bw<float, float>(st, a);
}

}  // namespace xl
