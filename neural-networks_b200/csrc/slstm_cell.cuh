// Pointwise sLSTM cell, forward and backward, shared by the cluster and the grid-cooperative
// recurrent kernels. Math: src/nn2/slstm.rs:286-325 (forward), 399-423 (backward), with the gate
// clamps i', f' <= 1 of the GPU kernels (src/gpu/cuda/slstm_fused.cu:132-142).
#pragma once
#include "common.cuh"

namespace xl {

struct SlstmFwCell {
    float z, o, ip, fp, c, n, m, h;
};

// exp/log go through the hardware approximations (relative error ~1e-6, inside the 1e-4 budget).
__device__ __forceinline__ SlstmFwCell slstm_cell_fw(float z_pre, float i_pre, float f_pre, float o_pre, float cp,
                                                      float np, float mp) {
    SlstmFwCell r;
    r.z = 1.f - __fdividef(2.f, 1.f + __expf(2.f * z_pre));
    r.o = __fdividef(1.f, 1.f + __expf(-o_pre));
    const float fm = fminf(f_pre, 0.f) - __logf(1.f + __expf(-fabsf(f_pre))) + mp;  // log sigmoid(f) + m_prev
    r.m = (np == 0.f) ? i_pre : fmaxf(fm, i_pre);
    r.ip = fminf(1.f, __expf(i_pre - r.m));
    r.fp = fminf(1.f, __expf(fm - r.m));
    r.c = r.fp * cp + r.ip * r.z;
    r.n = r.fp * np + r.ip;
    r.h = __fdividef(r.o * r.c, r.n);
    return r;
}

struct SlstmBwCell {
    float dz, di, df, dob;  // gate deltas (pre-activation gradients)
    float dc, dn;           // state gradients handed to step t-1
};

// d_h: upstream dy_t plus the recurrent term; (dc_in, dn_in): state gradients arriving from step t+1.
__device__ __forceinline__ SlstmBwCell slstm_cell_bw(float d_h, float o, float c, float n, float f, float i, float z,
                                                      float c_prev, float n_prev, float f_pre, float dc_in,
                                                      float dn_in) {
    // One reciprocal of n serves the three quotients, and the quotients and the sigmoid go through the hardware
    // approximations like the forward cell's (relative error ~1e-6): with IEEE divisions and the library exponential
    // this chain was 1.7 k of a 12.6 k-cycle step of the grid kernel.
    SlstmBwCell r;
    const float rn = __fdividef(1.f, n);
    const float hn = c * rn;  // c / n
    const float dho = d_h * o;
    r.dob = dho * hn * (1.f - o);
    const float d_c = dho * rn + dc_in;
    const float d_n = dn_in - dho * hn * rn;
    const float d_f_gate = d_c * c_prev + d_n * n_prev;
    const float d_i_gate = d_c * z + d_n;
    r.dz = d_c * i * (1.f - z * z);
    r.di = d_i_gate * i;
    const float e = __expf(-fabsf(f_pre));          // 1 - sigmoid(f_pre) = sigmoid(-f_pre), branch-free
    const float rs = __fdividef(1.f, 1.f + e);
    r.df = d_f_gate * f * (f_pre >= 0.f ? e * rs : rs);
    r.dc = d_c * f;
    r.dn = d_n * f;
    return r;
}

}  // namespace xl
