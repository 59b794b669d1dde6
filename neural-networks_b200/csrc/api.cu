// C-ABI layer: argument checking, workspace carving and dispatch for the mLSTM entry points,
// plus the library-wide helpers (error text, launch counter, device properties).
#include <stdarg.h>
#include <string.h>

#include "common.cuh"
#include "mlstm.cuh"

namespace xl {

static thread_local char g_err[512] = "";
std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static int check_shape(const char* who, const xlstm_mlstm_shape* s) {
    XL_CHECK_ARG(s, "%s: null shape", who);
    XL_CHECK_ARG(s->B > 0 && s->H > 0 && s->T > 0 && s->dqk > 0 && s->dhv > 0 && s->L > 0,
                 "%s: bad shape B=%d H=%d T=%d dqk=%d dhv=%d L=%d", who, s->B, s->H, s->T, s->dqk, s->dhv, s->L);
    XL_CHECK_ARG((s->dtype == XLSTM_F32 || s->dtype == XLSTM_BF16) && (s->gdtype == XLSTM_F32 || s->gdtype == XLSTM_BF16),
                 "%s: unknown storage type", who);
    return XLSTM_OK;
}

static inline int eff_L(const xlstm_mlstm_shape* s) { return s->L < s->T ? s->L : s->T; }
static inline int num_chunks(const xlstm_mlstm_shape* s) { int L = eff_L(s); return (s->T + L - 1) / L; }

// The tensor-core kernels work on 64-row chunk tiles whatever T is: a sequence shorter than a chunk is one ragged
// chunk (rows past T are zero-filled by the tensor map and never stored), so the requested L decides, not min(L, T).
static inline bool use_tc(const xlstm_mlstm_shape* s) {
    return !(s->flags & XLSTM_FORCE_SIMT) && mlstm_tc_supported(s->L, s->dqk, s->dhv, s->dtype) && s->T >= 1;
}

// Chunk-state record of the CUDA-core path: C then n, each the state ENTERING a chunk, f32.
static size_t saved_C_bytes(const xlstm_mlstm_shape* s) {
    return align_up((size_t)s->B * s->H * num_chunks(s) * s->dhv * s->dqk * sizeof(float), 256);
}
static size_t saved_n_bytes(const xlstm_mlstm_shape* s) {
    return align_up((size_t)s->B * s->H * num_chunks(s) * s->dqk * sizeof(float), 256);
}

}  // namespace xl

using namespace xl;

extern "C" int xlstm_version(void) { return 1; }
extern "C" const char* xlstm_last_error(void) { return g_err; }
extern "C" uint64_t xlstm_launch_count(void) { return g_launches.load(); }
extern "C" int xlstm_device_status(void) {
    int v = 0;
    int rc = tc_status_read_and_clear(&v);
    if (rc) return rc;
    if (v != 0) {
        set_error("a device-side wait ran out of its budget (code %d); the kernel unwound without completing", v);
        return XLSTM_ERR_TIMEOUT;
    }
    return XLSTM_OK;
}

// Chunk-state record of the tensor-core path: one bf16 C and fp32 n per 128 x 128 sub-head and chunk boundary.
static size_t tc_record_bytes(const xlstm_mlstm_shape* s) {
    const int bhs = s->B * s->H * mlstm_tc_subheads(s->dqk, s->dhv);
    return mlstm_tc_saved_C_bytes(bhs, num_chunks(s)) + mlstm_tc_saved_n_bytes(bhs, num_chunks(s));
}

// Packed mode of the tensor-core path (XLSTM_PACK_SHORT): sequences of at most 32 positions with no carry, 64 / T of
// them to a 64-row chunk tile. Returns the sequences per tile, 0 when the call runs unpacked (flag absent, or a shape the
// packed kernels do not cover), -1 when the flag is set on a call that cannot be packed by its arguments. The first
// (B / n) * n sequences run packed; the rest, fewer than n, run unpacked on the tail of every tensor.
static int tc_pack_count(const xlstm_mlstm_shape* s, bool any_carry_or_state) {
    if (!(s->flags & XLSTM_PACK_SHORT) || !use_tc(s) || s->dqk != 128 || s->dhv != 128) return 0;
    if (any_carry_or_state || s->T > 32) {
        set_error("mlstm: XLSTM_PACK_SHORT takes sequences of at most 32 positions without carries or state outputs");
        return -1;
    }
    const int n = 64 / s->T;
    return s->B >= n ? n : 0;
}
static size_t tc_record_bytes_bh(int bh, int nc) { return mlstm_tc_saved_C_bytes(bh, nc) + mlstm_tc_saved_n_bytes(bh, nc); }
template <typename T>
static T* off(T* p, size_t bytes) { return p ? (T*)((char*)p + bytes) : p; }
template <typename T>
static const T* off(const T* p, size_t bytes) { return p ? (const T*)((const char*)p + bytes) : p; }

// The forward arguments of sequences [b0, b0 + nb) of a call (tensor-core path: bf16 q, k, v, ytil).
static MlstmFwArgs fw_slice(MlstmFwArgs a, int b0, int nb) {
    const size_t rows = (size_t)b0 * a.T;
    a.q = off(a.q, rows * a.H * a.dqk * 2); a.k = off(a.k, rows * a.H * a.dqk * 2); a.v = off(a.v, rows * a.H * a.dhv * 2);
    a.ig = off(a.ig, rows * a.H * 4); a.fg = off(a.fg, rows * a.H * 4);
    a.ytil = off(a.ytil, rows * a.H * a.dhv * 2);
    a.msv = off(a.msv, rows * a.H * 4); a.psiv = off(a.psiv, rows * a.H * 4); a.qnv = off(a.qnv, rows * a.H * 4);
    a.B = nb;
    return a;
}
// ... and turned into the packed launch: nb / n tiles of n sequences each.
static MlstmFwArgs fw_packed(MlstmFwArgs a, int n) {
    a.seg = a.T; a.npack = n; a.B /= n; a.T *= n; a.NC = 1;
    return a;
}
static int tc_fw_maybe_packed(cudaStream_t st, int n, const MlstmFwArgs& a, void* saved, void* workspace,
                              size_t workspace_bytes) {
    if (!n) return mlstm_fw_tc_launch(st, a, saved, workspace, workspace_bytes);
    const int full = a.B / n * n, tail = a.B - full;
    int rc = mlstm_fw_tc_launch(st, fw_packed(fw_slice(a, 0, full), n), saved, workspace, workspace_bytes);
    if (rc || !tail) return rc;
    return mlstm_fw_tc_launch(st, fw_slice(a, full, tail), off(saved, tc_record_bytes_bh(full / n * a.H, 1)), workspace,
                              workspace_bytes);
}

extern "C" size_t xlstm_mlstm_saved_bytes(const xlstm_mlstm_shape* s) {
    if (!s || s->B <= 0 || s->H <= 0 || s->T <= 0 || s->dqk <= 0 || s->dhv <= 0 || s->L <= 0) return 0;
    if (use_tc(s)) return tc_record_bytes(s);
    return saved_C_bytes(s) + saved_n_bytes(s);
}
extern "C" size_t xlstm_mlstm_fw_workspace_bytes(const xlstm_mlstm_shape* s) {
    if (!s || s->B <= 0 || s->H <= 0 || s->T <= 0 || s->dqk <= 0 || s->dhv <= 0 || s->L <= 0) return 0;
    if (use_tc(s)) return mlstm_tc_fw_workspace_bytes(s->B, s->H, s->T, s->dqk, s->dhv);
    return 0;
}
extern "C" size_t xlstm_mlstm_bw_workspace_bytes(const xlstm_mlstm_shape* s, int have_saved) {
    if (!s || s->B <= 0 || s->H <= 0 || s->T <= 0 || s->dqk <= 0 || s->dhv <= 0 || s->L <= 0) return 0;
    if (use_tc(s)) return (have_saved ? 0 : tc_record_bytes(s)) + mlstm_tc_bw_workspace_bytes(s->B, s->H, s->T, s->dqk, s->dhv);
    if (have_saved) return 0;
    return saved_C_bytes(s) + saved_n_bytes(s);
}

extern "C" int xlstm_mlstm_fw(void* stream, const xlstm_mlstm_shape* s, const void* q, const void* k, const void* v,
                              const float* ig, const float* fg, const float* carry_C, const float* carry_n,
                              const float* carry_m, void* ytil, float* msv, float* psiv, float* qnv, void* saved,
                              float* out_C, float* out_n, float* out_m, void* workspace, size_t workspace_bytes) {
    int rc = check_shape("mlstm_fw", s);
    if (rc) return rc;
    XL_CHECK_ARG(q && k && v && ig && fg && ytil && msv && psiv && qnv, "mlstm_fw: null pointer");
    XL_CHECK_ARG((carry_C != nullptr) == (carry_n != nullptr) && (carry_C != nullptr) == (carry_m != nullptr),
                 "mlstm_fw: carry C, n, m must be given together");
    MlstmFwArgs a = {};
    a.q = q; a.k = k; a.v = v; a.ig = ig; a.fg = fg; a.cC = carry_C; a.cn = carry_n; a.cm = carry_m;
    a.ytil = ytil; a.msv = msv; a.psiv = psiv; a.qnv = qnv;
    if (saved) { a.savedC = (float*)saved; a.savedn = (float*)((char*)saved + saved_C_bytes(s)); }
    a.oC = out_C; a.on = out_n; a.om = out_m;
    a.B = s->B; a.H = s->H; a.T = s->T; a.dqk = s->dqk; a.dhv = s->dhv; a.L = eff_L(s); a.NC = num_chunks(s);
    a.states_only = 0;
    if (use_tc(s)) {
        const int npk = tc_pack_count(s, a.cC || a.oC);
        if (npk < 0) return XLSTM_ERR_ARG;
        return tc_fw_maybe_packed((cudaStream_t)stream, npk, a, saved, workspace, workspace_bytes);
    }
    return mlstm_fw_simt_launch((cudaStream_t)stream, a, s->dtype);
}

extern "C" int xlstm_mlstm_final_state(void* stream, const xlstm_mlstm_shape* s, const void* q, const void* k, const void* v,
                                       const float* ig, const float* fg, const float* carry_C, const float* carry_n,
                                       const float* carry_m, float* out_C, float* out_n, float* out_m) {
    int rc = check_shape("mlstm_final_state", s);
    if (rc) return rc;
    XL_CHECK_ARG(q && k && v && ig && fg && out_C && out_n && out_m, "mlstm_final_state: null pointer");
    XL_CHECK_ARG((carry_C != nullptr) == (carry_n != nullptr) && (carry_C != nullptr) == (carry_m != nullptr),
                 "mlstm_final_state: carry C, n, m must be given together");
    MlstmFwArgs a = {};
    a.q = q; a.k = k; a.v = v; a.ig = ig; a.fg = fg; a.cC = carry_C; a.cn = carry_n; a.cm = carry_m;
    a.oC = out_C; a.on = out_n; a.om = out_m;
    a.B = s->B; a.H = s->H; a.T = s->T; a.dqk = s->dqk; a.dhv = s->dhv; a.L = eff_L(s); a.NC = num_chunks(s);
    a.states_only = 1;
    if (use_tc(s)) return mlstm_fw_tc_launch((cudaStream_t)stream, a, nullptr, nullptr, 0);
    return mlstm_fw_simt_launch((cudaStream_t)stream, a, s->dtype);
}

extern "C" int xlstm_mlstm_bw(void* stream, const xlstm_mlstm_shape* s, const void* q, const void* k, const void* v,
                              const float* ig, const float* fg, const float* carry_C, const float* carry_n,
                              const float* carry_m, const void* ytil, const float* msv, const float* psiv,
                              const float* qnv, const void* saved, const void* d_ytil, const float* carry_dC,
                              const float* carry_dn, void* dq, void* dk, void* dv, float* dig, float* dfg,
                              float* out_dC, float* out_dn, void* workspace, size_t workspace_bytes) {
    int rc = check_shape("mlstm_bw", s);
    if (rc) return rc;
    XL_CHECK_ARG(q && k && v && ig && fg && ytil && msv && psiv && qnv && d_ytil && dq && dk && dv && dig && dfg,
                 "mlstm_bw: null pointer");
    XL_CHECK_ARG((carry_C != nullptr) == (carry_n != nullptr) && (carry_C != nullptr) == (carry_m != nullptr),
                 "mlstm_bw: carry C, n, m must be given together");
    XL_CHECK_ARG((carry_dC != nullptr) == (carry_dn != nullptr), "mlstm_bw: carry dC, dn must be given together");
    cudaStream_t st = (cudaStream_t)stream;
    if (use_tc(s)) {
        char* ws = (char*)workspace;
        size_t ws_left = workspace ? workspace_bytes : 0;
        const int npk = tc_pack_count(s, carry_C || carry_dC || out_dC);
        if (npk < 0) return XLSTM_ERR_ARG;
        const int full = npk ? s->B / npk * npk : 0, tail = s->B - full;
        if (!saved) {
            // recompute the chunk-boundary states (bf16 record) into the workspace with the forward's state-only pass
            size_t need = xlstm_mlstm_bw_workspace_bytes(s, 0);
            if (!workspace || workspace_bytes < need) {
                set_error("mlstm_bw: workspace of %zu B is smaller than the %zu B needed to recompute chunk states",
                          workspace_bytes, need);
                return XLSTM_ERR_WORKSPACE;
            }
            MlstmFwArgs f = {};
            f.q = q; f.k = k; f.v = v; f.ig = ig; f.fg = fg; f.cC = carry_C; f.cn = carry_n; f.cm = carry_m;
            f.B = s->B; f.H = s->H; f.T = s->T; f.dqk = s->dqk; f.dhv = s->dhv; f.L = eff_L(s); f.NC = num_chunks(s);
            f.states_only = 1;
            rc = tc_fw_maybe_packed(st, npk, f, workspace, nullptr, 0);
            if (rc) return rc;
            saved = workspace;
            ws += tc_record_bytes(s);
            ws_left -= tc_record_bytes(s);
        }
        MlstmBwArgs a = {};
        a.q = q; a.k = k; a.v = v; a.ig = ig; a.fg = fg; a.cm = carry_m; a.ytil = ytil; a.msv = msv; a.psiv = psiv;
        a.qnv = qnv; a.dytil = d_ytil; a.cdC = carry_dC; a.cdn = carry_dn;
        a.dq = dq; a.dk = dk; a.dv = dv; a.dig = dig; a.dfg = dfg; a.odC = out_dC; a.odn = out_dn;
        a.B = s->B; a.H = s->H; a.T = s->T; a.dqk = s->dqk; a.dhv = s->dhv; a.L = eff_L(s); a.NC = num_chunks(s);
        if (!npk) return mlstm_bw_tc_launch(st, a, saved, s->gdtype, ws, ws_left);
        // packed: the first `full` sequences npk to a tile, then the few that are left as they are
        const size_t gw = s->gdtype == XLSTM_BF16 ? 2 : 4;
        auto slice = [&](int b0, int nb) {
            MlstmBwArgs x = a;
            const size_t rows = (size_t)b0 * a.T, hq = (size_t)a.H * a.dqk, hv = (size_t)a.H * a.dhv;
            x.q = off(a.q, rows * hq * 2); x.k = off(a.k, rows * hq * 2); x.v = off(a.v, rows * hv * 2);
            x.ig = off(a.ig, rows * a.H * 4); x.fg = off(a.fg, rows * a.H * 4);
            x.ytil = off(a.ytil, rows * hv * 2); x.dytil = off(a.dytil, rows * hv * gw);
            x.msv = off(a.msv, rows * a.H * 4); x.psiv = off(a.psiv, rows * a.H * 4); x.qnv = off(a.qnv, rows * a.H * 4);
            x.dq = off(a.dq, rows * hq * gw); x.dk = off(a.dk, rows * hq * gw); x.dv = off(a.dv, rows * hv * gw);
            x.dig = off(a.dig, rows * a.H * 4); x.dfg = off(a.dfg, rows * a.H * 4);
            x.B = nb;
            return x;
        };
        MlstmBwArgs pk = slice(0, full);
        pk.seg = a.T; pk.npack = npk; pk.B = full / npk; pk.T = a.T * npk; pk.NC = 1;
        rc = mlstm_bw_tc_launch(st, pk, saved, s->gdtype, ws, ws_left);
        if (rc || !tail) return rc;
        return mlstm_bw_tc_launch(st, slice(full, tail), off(saved, tc_record_bytes_bh(full / npk * a.H, 1)), s->gdtype, ws, ws_left);
    }
    const float *sC, *sn;
    if (saved) {
        sC = (const float*)saved;
        sn = (const float*)((const char*)saved + saved_C_bytes(s));
    } else {
        // recompute the chunk-boundary states into the workspace
        size_t need = xlstm_mlstm_bw_workspace_bytes(s, 0);
        if (!workspace || workspace_bytes < need) {
            set_error("mlstm_bw: workspace of %zu B is smaller than the %zu B needed to recompute chunk states",
                      workspace_bytes, need);
            return XLSTM_ERR_WORKSPACE;
        }
        MlstmFwArgs f = {};
        f.q = q; f.k = k; f.v = v; f.ig = ig; f.fg = fg; f.cC = carry_C; f.cn = carry_n; f.cm = carry_m;
        f.savedC = (float*)workspace; f.savedn = (float*)((char*)workspace + saved_C_bytes(s));
        f.B = s->B; f.H = s->H; f.T = s->T; f.dqk = s->dqk; f.dhv = s->dhv; f.L = eff_L(s); f.NC = num_chunks(s);
        f.states_only = 1;
        rc = mlstm_fw_simt_launch(st, f, s->dtype);
        if (rc) return rc;
        sC = f.savedC; sn = f.savedn;
    }
    MlstmBwArgs a = {};
    a.q = q; a.k = k; a.v = v; a.ig = ig; a.fg = fg; a.cm = carry_m; a.ytil = ytil; a.msv = msv; a.psiv = psiv;
    a.qnv = qnv; a.savedC = sC; a.savedn = sn; a.dytil = d_ytil; a.cdC = carry_dC; a.cdn = carry_dn;
    a.dq = dq; a.dk = dk; a.dv = dv; a.dig = dig; a.dfg = dfg; a.odC = out_dC; a.odn = out_dn;
    a.B = s->B; a.H = s->H; a.T = s->T; a.dqk = s->dqk; a.dhv = s->dhv; a.L = eff_L(s); a.NC = num_chunks(s);
    return mlstm_bw_simt_launch(st, a, s->dtype, s->gdtype);
}
