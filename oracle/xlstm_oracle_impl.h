/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's xLSTM layer math.
 *
 * This file is the body of the oracle, included twice by xlstm_oracle.c: once with
 * REAL=float (suffix _f32: the faithful twin of the reference's fp32 CPU path, also the
 * thing timed as the CPU baseline) and once with REAL=double (suffix _f64: the same
 * algorithm carried in double, used as the low-noise comparison target).
 *
 * Parity status: PARITY UNPINNED at the bit level. The reference (a Rust crate) cannot
 * be built in this environment and its tests hold no golden vectors or known answers
 * for these layers; the restatement is validated instead by the reference's own
 * property tests restated in tests/ (directional finite differences, chunk-length
 * invariance, carry == whole sequence) and by an independent autograd cross-check.
 *
 * Only tests, the smoke check and the benchmark's cpu_baseline leg may link or call
 * this code. The product never does.
 *
 * Every function cites the reference file:line it follows (paths inside the reference
 * project).
 */

/* ---- scalar helpers ---------------------------------------------------------------- */

/* src/nn2/mlstm.rs:31-38 (same body at src/nn2/slstm.rs:20-27) */
static inline REAL FN(sigmoid)(REAL x) {
    if (x >= (REAL)0) return (REAL)1 / ((REAL)1 + R_EXP(-x));
    REAL e = R_EXP(x);
    return e / ((REAL)1 + e);
}

/* src/nn2/mlstm.rs:41-47 */
static inline REAL FN(log_sigmoid)(REAL x) {
    if (x >= (REAL)0) return -R_LOG((REAL)1 + R_EXP(-x));
    return x - R_LOG((REAL)1 + R_EXP(x));
}

static inline REAL FN(dot)(const REAL* a, const REAL* b, int n) {
    REAL s = 0;
    for (int i = 0; i < n; ++i) s += a[i] * b[i];
    return s;
}

/* ---- GEMM: C[m,n] = beta*C + A·B in the three forms the layers use ------------------ */
/* src/tensor/gemm.rs:40-182 — row-major, MR=4 row blocking over the output; the
 * summation order along k is the plain ascending one, as there. */

void FN(gemm_nn)(int m, int k, int n, const REAL* a, const REAL* b, REAL* c, REAL beta) {
    for (int i0 = 0; i0 < m; i0 += 4) {
        int mr = m - i0 < 4 ? m - i0 : 4;
        for (int r = 0; r < mr; ++r) {
            REAL* cr = c + (size_t)(i0 + r) * n;
            if (beta == (REAL)0) for (int j = 0; j < n; ++j) cr[j] = 0;
            else if (beta != (REAL)1) for (int j = 0; j < n; ++j) cr[j] *= beta;
        }
        for (int p = 0; p < k; ++p) {
            const REAL* br = b + (size_t)p * n;
            for (int r = 0; r < mr; ++r) {
                REAL av = a[(size_t)(i0 + r) * k + p];
                REAL* cr = c + (size_t)(i0 + r) * n;
                for (int j = 0; j < n; ++j) cr[j] += av * br[j];
            }
        }
    }
}

/* C[m,n] = beta*C + Aᵀ·B with A stored [k,m], B stored [k,n] (src/tensor/gemm.rs gemm_tn) */
void FN(gemm_tn)(int m, int k, int n, const REAL* a, const REAL* b, REAL* c, REAL beta) {
    for (int i = 0; i < m; ++i) {
        REAL* cr = c + (size_t)i * n;
        if (beta == (REAL)0) for (int j = 0; j < n; ++j) cr[j] = 0;
        else if (beta != (REAL)1) for (int j = 0; j < n; ++j) cr[j] *= beta;
    }
    for (int p = 0; p < k; ++p) {
        const REAL* ar = a + (size_t)p * m;
        const REAL* br = b + (size_t)p * n;
        for (int i = 0; i < m; ++i) {
            REAL av = ar[i];
            REAL* cr = c + (size_t)i * n;
            for (int j = 0; j < n; ++j) cr[j] += av * br[j];
        }
    }
}

/* C[m,n] = beta*C + A·Bᵀ with A [m,k], B stored [n,k] (src/tensor/gemm.rs gemm_nt) */
void FN(gemm_nt)(int m, int k, int n, const REAL* a, const REAL* b, REAL* c, REAL beta) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            REAL s = FN(dot)(a + (size_t)i * k, b + (size_t)j * k, k);
            REAL* o = c + (size_t)i * n + j;
            *o = (beta == (REAL)0 ? (REAL)0 : beta * *o) + s;
        }
}

/* ---- mLSTM core, recurrent form -------------------------------------------------------
 *
 * The part of src/nn2/mlstm.rs:483-541 between the projections and the head norm, in
 * the layout of the GPU op it is the oracle for (src/gpu/ops.rs:4380-4395): q,k
 * [B*T, H*dqk], v [B*T, H*dhv], gate logits [B*T, H], element (b,h,t,c) at
 * ((b*T+t)*H+h)*W+c; k arrives already scaled by 1/sqrt(dqk). Per-(b,h) scalars are
 * [B*H, T]. C0/n0/m0 (each may be NULL = zero) is the state the call continues from
 * (src/gpu/mlstm.rs:598-623); C_end/n_end/m_end (each may be NULL) receive the state
 * after the last step.
 */
static void FN(mlstm_fw_one)(const REAL* q, const REAL* k, const REAL* v, const REAL* ig,
                             const REAL* fg, const REAL* C0, const REAL* n0, const REAL* m0,
                             int b, int h, int H, int T, int dqk, int dhv, REAL* ytil,
                             REAL* m_out, REAL* psi_out, REAL* nq_out, REAL* C_end,
                             REAL* n_end, REAL* m_end) {
    int bh = b * H + h;
    size_t cn = (size_t)dhv * dqk;
    REAL* C = (REAL*)calloc(cn, sizeof(REAL));
    REAL* n = (REAL*)calloc(dqk, sizeof(REAL));
    REAL m = 0;
    if (C0) memcpy(C, C0 + (size_t)bh * cn, cn * sizeof(REAL));
    if (n0) memcpy(n, n0 + (size_t)bh * dqk, dqk * sizeof(REAL));
    if (m0) m = m0[bh];
    for (int t = 0; t < T; ++t) {
        size_t pos = (size_t)b * T + t;
        const REAL* qh = q + (pos * H + h) * dqk;
        const REAL* kh = k + (pos * H + h) * dqk;
        const REAL* vh = v + (pos * H + h) * dhv;
        REAL lf = FN(log_sigmoid)(fg[pos * H + h]);
        REAL ii = ig[pos * H + h];
        REAL mh = lf + m > ii ? lf + m : ii;          /* mlstm.rs:488 */
        REAL ip = R_EXP(ii - mh);                      /* :489 */
        REAL fp = R_EXP(lf + m - mh);                  /* :490 */
        m = mh;
        for (int j = 0; j < dqk; ++j) n[j] = fp * n[j] + ip * kh[j];   /* :507 */
        REAL nq = FN(dot)(n, qh, dqk);                 /* :510 */
        REAL flo = R_EXP(-mh);                         /* :523 */
        REAL psi = R_FABS(nq) > flo ? R_FABS(nq) : flo;
        REAL inv_psi = (REAL)1 / psi;
        REAL* yt = ytil + (pos * H + h) * dhv;
        for (int i = 0; i < dhv; ++i) {
            REAL ivi = ip * vh[i];
            REAL* cr = C + (size_t)i * dqk;
            for (int j = 0; j < dqk; ++j) cr[j] = fp * cr[j] + ivi * kh[j];   /* :536 */
            yt[i] = FN(dot)(cr, qh, dqk) * inv_psi;                            /* :538-540 */
        }
        if (m_out) m_out[(size_t)bh * T + t] = mh;
        if (psi_out) psi_out[(size_t)bh * T + t] = psi;
        if (nq_out) nq_out[(size_t)bh * T + t] = nq;
    }
    if (C_end) memcpy(C_end + (size_t)bh * cn, C, cn * sizeof(REAL));
    if (n_end) memcpy(n_end + (size_t)bh * dqk, n, dqk * sizeof(REAL));
    if (m_end) m_end[bh] = m;
    free(C); free(n);
}

void FN(mlstm_core_fw)(const REAL* q, const REAL* k, const REAL* v, const REAL* ig,
                       const REAL* fg, const REAL* C0, const REAL* n0, const REAL* m0,
                       int B, int H, int T, int dqk, int dhv, REAL* ytil, REAL* m_out,
                       REAL* psi_out, REAL* nq_out, REAL* C_end, REAL* n_end, REAL* m_end) {
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * H; ++bh)
        FN(mlstm_fw_one)(q, k, v, ig, fg, C0, n0, m0, bh / H, bh % H, H, T, dqk, dhv, ytil,
                         m_out, psi_out, nq_out, C_end, n_end, m_end);
}

/* Backward of the core: src/nn2/mlstm.rs:731-806, with the stabiliser m held constant
 * and dk taken with respect to the pre-scaled k (the reference CPU cell multiplies dk by
 * 1/sqrt(dqk) afterwards, :809-811, because its k is scaled inside the cell; the GPU op
 * receives pre-scaled k, src/gpu/mlstm.rs:241-252). dC_in/dn_in (may be NULL = zero) is
 * the BPTT state arriving from the call to the right, dC_out/dn_out (may be NULL) the
 * one handed to the call on the left (src/gpu/ops.rs:4228-4233). The forward is re-run
 * per (b,h) to rebuild the per-step records. */
void FN(mlstm_core_bw)(const REAL* q, const REAL* k, const REAL* v, const REAL* ig,
                       const REAL* fg, const REAL* C0, const REAL* n0, const REAL* m0,
                       const REAL* dytil, const REAL* dC_in, const REAL* dn_in, int B, int H,
                       int T, int dqk, int dhv, REAL* dq, REAL* dk, REAL* dv, REAL* dig,
                       REAL* dfg, REAL* dC_out, REAL* dn_out) {
    size_t cn = (size_t)dhv * dqk;
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * H; ++bh) {
        int b = bh / H, h = bh % H;
        REAL* Cs = (REAL*)malloc((size_t)(T + 1) * cn * sizeof(REAL));
        REAL* ns = (REAL*)malloc((size_t)(T + 1) * dqk * sizeof(REAL));
        REAL* ips = (REAL*)malloc((size_t)T * sizeof(REAL));
        REAL* fps = (REAL*)malloc((size_t)T * sizeof(REAL));
        REAL* ytil = (REAL*)malloc((size_t)T * dhv * sizeof(REAL));
        REAL* msv = (REAL*)malloc((size_t)T * sizeof(REAL));
        REAL* psv = (REAL*)malloc((size_t)T * sizeof(REAL));
        REAL* nqv = (REAL*)malloc((size_t)T * sizeof(REAL));
        REAL* dC = (REAL*)calloc(cn, sizeof(REAL));
        REAL* dn = (REAL*)calloc(dqk, sizeof(REAL));
        REAL* tmp = (REAL*)malloc((size_t)dqk * sizeof(REAL));
        /* re-run the forward of this (b,h) into private per-step records */
        {
            REAL* C = (REAL*)calloc(cn, sizeof(REAL));
            REAL* n = (REAL*)calloc(dqk, sizeof(REAL));
            REAL m = 0;
            if (C0) memcpy(C, C0 + (size_t)bh * cn, cn * sizeof(REAL));
            if (n0) memcpy(n, n0 + (size_t)bh * dqk, dqk * sizeof(REAL));
            if (m0) m = m0[bh];
            memcpy(Cs, C, cn * sizeof(REAL)); memcpy(ns, n, dqk * sizeof(REAL));
            for (int t = 0; t < T; ++t) {
                size_t pos = (size_t)b * T + t;
                const REAL* qh = q + (pos * H + h) * dqk;
                const REAL* kh = k + (pos * H + h) * dqk;
                const REAL* vh = v + (pos * H + h) * dhv;
                REAL lf = FN(log_sigmoid)(fg[pos * H + h]);
                REAL ii = ig[pos * H + h];
                REAL mh = lf + m > ii ? lf + m : ii;
                REAL ip = R_EXP(ii - mh), fp = R_EXP(lf + m - mh);
                m = mh;
                for (int j = 0; j < dqk; ++j) n[j] = fp * n[j] + ip * kh[j];
                REAL nq = FN(dot)(n, qh, dqk);
                REAL flo = R_EXP(-mh);
                REAL psi = R_FABS(nq) > flo ? R_FABS(nq) : flo;
                for (int i = 0; i < dhv; ++i) {
                    REAL ivi = ip * vh[i];
                    REAL* cr = C + (size_t)i * dqk;
                    for (int j = 0; j < dqk; ++j) cr[j] = fp * cr[j] + ivi * kh[j];
                    ytil[(size_t)t * dhv + i] = FN(dot)(cr, qh, dqk);   /* C·q, unnormalised (mlstm.rs:539 `cq`) */
                }
                msv[t] = mh; psv[t] = psi; nqv[t] = nq; ips[t] = ip; fps[t] = fp;
                memcpy(Cs + (size_t)(t + 1) * cn, C, cn * sizeof(REAL));
                memcpy(ns + (size_t)(t + 1) * dqk, n, dqk * sizeof(REAL));
            }
            free(C); free(n);
        }
        if (dC_in) memcpy(dC, dC_in + (size_t)bh * cn, cn * sizeof(REAL));
        if (dn_in) memcpy(dn, dn_in + (size_t)bh * dqk, dqk * sizeof(REAL));
        for (int t = T - 1; t >= 0; --t) {
            size_t pos = (size_t)b * T + t;
            const REAL* qh = q + (pos * H + h) * dqk;
            const REAL* kh = k + (pos * H + h) * dqk;
            const REAL* vh = v + (pos * H + h) * dhv;
            const REAL* dht = dytil + (pos * H + h) * dhv;
            const REAL* cq = ytil + (size_t)t * dhv;
            REAL* dqh = dq + (pos * H + h) * dqk;
            REAL* dkh = dk + (pos * H + h) * dqk;
            REAL* dvh = dv + (pos * H + h) * dhv;
            const REAL* Cprev = Cs + (size_t)t * cn;
            const REAL* Ccur = Cs + (size_t)(t + 1) * cn;
            const REAL* nprev = ns + (size_t)t * dqk;
            const REAL* ncur = ns + (size_t)(t + 1) * dqk;
            REAL inv_psi = (REAL)1 / psv[t];
            REAL dpsi = -(inv_psi * inv_psi) * FN(dot)(dht, cq, dhv);    /* :743 */
            REAL flo = R_EXP(-msv[t]);
            REAL dnq = 0;                                                  /* :746-750 */
            if (R_FABS(nqv[t]) > flo) dnq = (nqv[t] > 0 ? (REAL)1 : (nqv[t] < 0 ? (REAL)-1 : (REAL)0)) * dpsi;
            /* Rust's f32::signum returns +1 for +0.0; |nq| > floor > 0 rules zero out here */
            REAL ip = ips[t], fp = fps[t];
            REAL dfp = 0, dip = 0;
            for (int j = 0; j < dqk; ++j) {                                /* :763-767 */
                dqh[j] = dnq * ncur[j];
                dkh[j] = 0;
                dn[j] += dnq * qh[j];
            }
            for (int i = 0; i < dhv; ++i) {                                /* :771-790 */
                REAL dop = dht[i] * inv_psi;
                REAL* dcb = dC + (size_t)i * dqk;
                for (int j = 0; j < dqk; ++j) tmp[j] = dop * qh[j] + dcb[j];
                REAL row_df = FN(dot)(tmp, Cprev + (size_t)i * dqk, dqk);
                REAL row_dv = FN(dot)(tmp, kh, dqk);
                const REAL* crow = Ccur + (size_t)i * dqk;
                for (int j = 0; j < dqk; ++j) {
                    dcb[j] = tmp[j] * fp;
                    dqh[j] += dop * crow[j];
                    dkh[j] += tmp[j] * vh[i];
                }
                dfp += row_df;
                dip += vh[i] * row_dv;
                dvh[i] = ip * row_dv;
            }
            dfp += FN(dot)(dn, nprev, dqk);                                /* :795-800 */
            dip += FN(dot)(dn, kh, dqk);
            for (int j = 0; j < dqk; ++j) {
                dkh[j] = ip * (dkh[j] + dn[j]);
                dn[j] *= fp;
            }
            dig[pos * H + h] = dip * ip;                                   /* :803 */
            REAL sigf = FN(sigmoid)(fg[pos * H + h]);                      /* :804 exp(log σ) == σ */
            dfg[pos * H + h] = dfp * fp * ((REAL)1 - sigf);               /* :805 */
        }
        if (dC_out) memcpy(dC_out + (size_t)bh * cn, dC, cn * sizeof(REAL));
        if (dn_out) memcpy(dn_out + (size_t)bh * dqk, dn, dqk * sizeof(REAL));
        free(Cs); free(ns); free(ips); free(fps); free(ytil); free(msv); free(psv);
        free(nqv); free(dC); free(dn); free(tmp);
    }
}

/* ---- sLSTM recurrent loop -------------------------------------------------------------
 *
 * src/nn2/slstm.rs:286-325 (forward) and :399-423 (backward), in the shape of the GPU op
 * it is the oracle for (src/gpu/cuda/slstm_fused.cu:96-158,184-229; src/gpu/ops.rs
 * 2787-2880): g [B,T,4H] holds the hoisted input contribution x·Wx with gate blocks
 * z,i,f,o; wh is the recurrent matrix; bcat [4H] the biases. The two gate values are
 * clamped to <= 1 as the GPU kernels do (slstm_fused.cu:139-140).
 *
 * NH > 1 selects block-diagonal recurrence: wh is [NH, dh, 4*dh] with dh = H/NH, row =
 * source unit inside the head, column = gate*dh + unit inside the head — equal to the
 * reference's dense [H,4H] matrix with every off-block entry zero. NH == 1 is the dense
 * reference layout [H, 4H].
 *
 * State c,n,m,h [B,H] is read if `carry` (else zero) and always written back. Saved
 * slabs (each [B,T,H]): c_prev,n_prev,ipr,fpr,c,n,zt,ot,h_prev. The f block of g is
 * overwritten with the biased pre-activation (slstm_fused.cu:122).
 */
void FN(slstm_fw)(const REAL* wh, REAL* g, const REAL* bcat, REAL* cst, REAL* nst, REAL* mst,
                  REAL* hst, int carry, int B, int H, int NH, int T, REAL* out, REAL* c_prev,
                  REAL* n_prev, REAL* ipr, REAL* fpr, REAL* c_out, REAL* n_out, REAL* zt,
                  REAL* ot, REAL* h_prev) {
    int dh = H / NH;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b) {
        REAL* hp = (REAL*)calloc(H, sizeof(REAL));
        REAL* c = (REAL*)calloc(H, sizeof(REAL));
        REAL* n = (REAL*)calloc(H, sizeof(REAL));
        REAL* m = (REAL*)calloc(H, sizeof(REAL));
        REAL* gh = (REAL*)malloc((size_t)4 * H * sizeof(REAL));
        if (carry) {
            memcpy(hp, hst + (size_t)b * H, H * sizeof(REAL));
            memcpy(c, cst + (size_t)b * H, H * sizeof(REAL));
            memcpy(n, nst + (size_t)b * H, H * sizeof(REAL));
            memcpy(m, mst + (size_t)b * H, H * sizeof(REAL));
        }
        for (int t = 0; t < T; ++t) {
            REAL* gt = g + ((size_t)b * T + t) * 4 * H;
            size_t s0 = ((size_t)b * T + t) * H;
            /* gh = h_{t-1} · Wh */
            for (int x = 0; x < 4 * H; ++x) gh[x] = 0;
            for (int hd = 0; hd < NH; ++hd)
                for (int r = 0; r < dh; ++r) {
                    REAL hv = hp[hd * dh + r];
                    const REAL* wr = wh + ((size_t)hd * dh + r) * 4 * dh;
                    for (int gt_ = 0; gt_ < 4; ++gt_)
                        for (int u = 0; u < dh; ++u)
                            gh[gt_ * H + hd * dh + u] += hv * wr[gt_ * dh + u];
                }
            for (int j = 0; j < H; ++j) {
                REAL zp = gt[j] + gh[j] + bcat[j];
                REAL ipre = gt[H + j] + gh[H + j] + bcat[H + j];
                REAL fpre = gt[2 * H + j] + gh[2 * H + j] + bcat[2 * H + j];
                REAL opre = gt[3 * H + j] + gh[3 * H + j] + bcat[3 * H + j];
                gt[2 * H + j] = fpre;
                h_prev[s0 + j] = hp[j];
                REAL z = R_TANH(zp);
                REAL o = FN(sigmoid)(opre);
                REAL fm = FN(log_sigmoid)(fpre) + m[j];
                REAL np = n[j], cp = c[j];
                REAL mm = (np == (REAL)0) ? ipre : (fm > ipre ? fm : ipre);   /* slstm.rs:296-300 */
                REAL ip = R_EXP(ipre - mm), fp = R_EXP(fm - mm);
                if (ip > (REAL)1) ip = 1;
                if (fp > (REAL)1) fp = 1;
                REAL cc = fp * cp + ip * z, nn = fp * np + ip;
                c_prev[s0 + j] = cp; n_prev[s0 + j] = np;
                zt[s0 + j] = z; ot[s0 + j] = o; ipr[s0 + j] = ip; fpr[s0 + j] = fp;
                c_out[s0 + j] = cc; n_out[s0 + j] = nn;
                c[j] = cc; n[j] = nn; m[j] = mm;
                out[s0 + j] = o * cc / nn;                                    /* :319 */
            }
            for (int j = 0; j < H; ++j) hp[j] = out[s0 + j];
        }
        memcpy(hst + (size_t)b * H, hp, H * sizeof(REAL));
        memcpy(cst + (size_t)b * H, c, H * sizeof(REAL));
        memcpy(nst + (size_t)b * H, n, H * sizeof(REAL));
        memcpy(mst + (size_t)b * H, m, H * sizeof(REAL));
        free(hp); free(c); free(n); free(m); free(gh);
    }
}

/* Reverse loop. g enters holding the biased f pre-activation in its f block and leaves
 * holding the four gate deltas (slstm_fused.cu:197,221-224). dh,dc,dn [B,H] carry the BPTT
 * state: read if `carry` (else zero), always written back (what flows to the call on the
 * left). Weight gradients are NOT formed here: the reference defers dWh = Σ h_prevᵀ·dg,
 * dWx and dx to GEMMs after the loop (src/gpu/slstm.rs:903-940). */
void FN(slstm_bw)(const REAL* wh, const REAL* dy, REAL* g, REAL* dhs, REAL* dcs, REAL* dns,
                  int carry, int B, int H, int NH, int T, const REAL* c_prev,
                  const REAL* n_prev, const REAL* ipr, const REAL* fpr, const REAL* c_out,
                  const REAL* n_out, const REAL* zt, const REAL* ot) {
    int dh = H / NH;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b) {
        REAL* dhb = (REAL*)calloc(H, sizeof(REAL));
        REAL* dcb = (REAL*)calloc(H, sizeof(REAL));
        REAL* dnb = (REAL*)calloc(H, sizeof(REAL));
        if (carry) {
            memcpy(dhb, dhs + (size_t)b * H, H * sizeof(REAL));
            memcpy(dcb, dcs + (size_t)b * H, H * sizeof(REAL));
            memcpy(dnb, dns + (size_t)b * H, H * sizeof(REAL));
        }
        for (int t = T - 1; t >= 0; --t) {
            REAL* gt = g + ((size_t)b * T + t) * 4 * H;
            size_t s0 = ((size_t)b * T + t) * H;
            for (int j = 0; j < H; ++j) {
                REAL fpre = gt[2 * H + j];
                REAL d = dy[s0 + j] + dhb[j];
                REAL o = ot[s0 + j], c = c_out[s0 + j], n = n_out[s0 + j];
                REAL dop = d * (c / n) * o * ((REAL)1 - o);
                REAL dc = d * o / n + dcb[j];
                REAL dn = d * o * (-c) / (n * n) + dnb[j];
                REAL f = fpr[s0 + j], i = ipr[s0 + j], z = zt[s0 + j];
                REAL dfg_ = dc * c_prev[s0 + j] + dn * n_prev[s0 + j];
                REAL dig_ = dc * z + dn;
                REAL dzp = dc * i * ((REAL)1 - z * z);
                gt[j] = dzp;
                gt[H + j] = dig_ * i;
                gt[2 * H + j] = dfg_ * f * ((REAL)1 - FN(sigmoid)(fpre));
                gt[3 * H + j] = dop;
                dcb[j] = dc * f; dnb[j] = dn * f;
            }
            /* dh_{t-1} = dg · Whᵀ */
            for (int hd = 0; hd < NH; ++hd)
                for (int r = 0; r < dh; ++r) {
                    const REAL* wr = wh + ((size_t)hd * dh + r) * 4 * dh;
                    REAL s = 0;
                    for (int gt_ = 0; gt_ < 4; ++gt_)
                        for (int u = 0; u < dh; ++u)
                            s += gt[gt_ * H + hd * dh + u] * wr[gt_ * dh + u];
                    dhb[hd * dh + r] = s;
                }
        }
        memcpy(dhs + (size_t)b * H, dhb, H * sizeof(REAL));
        memcpy(dcs + (size_t)b * H, dcb, H * sizeof(REAL));
        memcpy(dns + (size_t)b * H, dnb, H * sizeof(REAL));
        free(dhb); free(dcb); free(dnb);
    }
}

/* ---- grouped RMSNorm: src/nn2/ops.rs:110-185, eps from src/nn2/rms_norm.rs:18 ---------- */
void FN(rmsnorm_fw)(const REAL* x, const REAL* gamma, int rows, int F, int group, REAL eps,
                    REAL* y, REAL* x_hat, REAL* inv_rms) {
    int gpr = F / group;
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < gpr; ++g) {
            size_t off = (size_t)r * F + (size_t)g * group;
            REAL ss = 0;
            for (int i = 0; i < group; ++i) ss += x[off + i] * x[off + i];
            REAL inv = (REAL)1 / R_SQRT(ss / (REAL)group + eps);
            if (inv_rms) inv_rms[(size_t)r * gpr + g] = inv;
            for (int i = 0; i < group; ++i) {
                REAL xh = x[off + i] * inv;
                if (x_hat) x_hat[off + i] = xh;
                y[off + i] = gamma[g * group + i] * xh;
            }
        }
}

void FN(rmsnorm_bw)(const REAL* dy, const REAL* x_hat, const REAL* inv_rms, const REAL* gamma,
                    int rows, int F, int group, REAL* dx, REAL* dgamma /* accumulated */) {
    int gpr = F / group;
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < gpr; ++g) {
            size_t off = (size_t)r * F + (size_t)g * group;
            REAL inv = inv_rms[(size_t)r * gpr + g];
            REAL s = 0;
            for (int i = 0; i < group; ++i) {
                REAL dyxh = dy[off + i] * x_hat[off + i];
                dgamma[g * group + i] += dyxh;
                s += gamma[g * group + i] * dyxh;
            }
            REAL sg = s / (REAL)group;
            for (int i = 0; i < group; ++i)
                dx[off + i] = inv * (gamma[g * group + i] * dy[off + i] - x_hat[off + i] * sg);
        }
}

/* ---- softmax cross-entropy: src/nn2/loss.rs:10-53; the masked / scaled form follows
 * src/gpu/cuda/mlstm_ops.cu:332-370 (rows whose mask is 0 contribute nothing and get a
 * zero gradient; `inv` replaces 1/rows) ------------------------------------------------ */
REAL FN(softmax_ce)(const REAL* logits, const unsigned* targets, const unsigned* mask, int rows,
                    int C, REAL inv, REAL* dlogits) {
    REAL loss = 0;
    for (int r = 0; r < rows; ++r) {
        const REAL* z = logits + (size_t)r * C;
        REAL* d = dlogits + (size_t)r * C;
        if (mask && !mask[r]) { for (int j = 0; j < C; ++j) d[j] = 0; continue; }
        REAL mx = z[0];
        for (int j = 1; j < C; ++j) if (z[j] > mx) mx = z[j];
        REAL sum = 0;
        for (int j = 0; j < C; ++j) { d[j] = R_EXP(z[j] - mx); sum += d[j]; }
        REAL is = (REAL)1 / sum;
        for (int j = 0; j < C; ++j) d[j] *= is;
        REAL pt = d[targets[r]];
        loss -= R_LOG(pt > (REAL)1e-30 ? pt : (REAL)1e-30);
        d[targets[r]] -= (REAL)1;
        for (int j = 0; j < C; ++j) d[j] *= inv;
    }
    return loss * inv;
}

/* ---- AdamW: src/nn2/optim.rs:49-71 ------------------------------------------------------ */
void FN(adamw)(REAL* p, const REAL* g, REAL* m, REAL* v, size_t n, REAL lr, REAL b1, REAL b2,
               REAL eps, REAL wd, int t) {
    REAL bc1 = (REAL)1 - R_POW(b1, (REAL)t);
    REAL bc2 = (REAL)1 - R_POW(b2, (REAL)t);
    for (size_t k = 0; k < n; ++k) {
        REAL gk = g[k];
        m[k] = b1 * m[k] + ((REAL)1 - b1) * gk;
        v[k] = b2 * v[k] + ((REAL)1 - b2) * gk * gk;
        REAL mh = m[k] / bc1, vh = v[k] / bc2;
        REAL pk = p[k];
        pk -= lr * wd * pk;
        pk -= lr * mh / (R_SQRT(vh) + eps);
        p[k] = pk;
    }
}

/* ---- SoftCap: src/nn2/ops.rs:25-42 ------------------------------------------------------ */
void FN(softcap_fw)(const REAL* x, size_t n, REAL cap, REAL* y) {
    for (size_t i = 0; i < n; ++i) y[i] = cap * R_TANH(x[i] / cap);
}
void FN(softcap_bw)(const REAL* dy, const REAL* y, size_t n, REAL cap, REAL* dx) {
    for (size_t i = 0; i < n; ++i) { REAL t = y[i] / cap; dx[i] = dy[i] * ((REAL)1 - t * t); }
}
