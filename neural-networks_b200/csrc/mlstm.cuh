// Argument blocks shared by the mLSTM kernels and the C-ABI layer.
#pragma once
#include <cuda_runtime.h>

namespace xl {

struct MlstmFwArgs {
    const void *q, *k, *v;
    const float *ig, *fg;
    const float *cC, *cn, *cm;  // carry in (may be null)
    void* ytil;
    float *msv, *psiv, *qnv;
    float *savedC, *savedn;     // [BH, NC, dhv*dqk], [BH, NC, dqk]: state entering each chunk (may be null)
    float *oC, *on, *om;        // state after the last position (may be null)
    int B, H, T, dqk, dhv, L, NC;
    int states_only;            // 1: walk the state recurrence only (recompute pass of the backward)
    // tensor-core path, packed mode (0 = off): T = npack * seg positions hold npack independent sequences of seg
    // positions each (seg <= 32, one chunk, no carry, no state out); msv / psiv / qnv stay [sequence][head][seg]
    int seg, npack;
};

struct MlstmBwArgs {
    const void *q, *k, *v;
    const float *ig, *fg;
    const float* cm;            // m the forward call entered with (may be null = 0)
    const void* ytil;
    const float *msv, *psiv, *qnv;
    const float *savedC, *savedn;
    const void* dytil;
    const float *cdC, *cdn;     // BPTT carry in (may be null)
    void *dq, *dk, *dv;
    float *dig, *dfg;
    float *odC, *odn;
    int B, H, T, dqk, dhv, L, NC;
    int seg, npack;             // packed mode of the tensor-core path, as in MlstmFwArgs
};

int mlstm_fw_simt_launch(cudaStream_t st, const MlstmFwArgs& a, int dtype);
int mlstm_bw_simt_launch(cudaStream_t st, const MlstmBwArgs& a, int dtype, int gdtype);
bool mlstm_simt_supported(int L, int dqk, int dhv, int dtype);

// Tensor-core (tcgen05) path
bool mlstm_tc_supported(int L, int dqk, int dhv, int dtype);
size_t mlstm_tc_saved_C_bytes(int BH, int NC);
size_t mlstm_tc_saved_n_bytes(int BH, int NC);
// Heads wider than 128 (multiples of 128) run as 128 x 128 sub-heads; `saved` then holds one record per sub-head.
int mlstm_tc_subheads(int dqk, int dhv);
size_t mlstm_tc_fw_workspace_bytes(int B, int H, int T, int dqk, int dhv);
size_t mlstm_tc_bw_workspace_bytes(int B, int H, int T, int dqk, int dhv);  // excluding a recomputed state record
int mlstm_fw_tc_launch(cudaStream_t st, const MlstmFwArgs& a, void* saved, void* workspace, size_t workspace_bytes);
int mlstm_bw_tc_launch(cudaStream_t st, const MlstmBwArgs& a, const void* saved, int gdtype, void* workspace,
                       size_t workspace_bytes);
int tc_status_read_and_clear(int* out);

}  // namespace xl
