/*
 * xlstm_b200 — C ABI of the B200 (sm_100a) engine for the xLSTM training hot path.
 *
 * Every entry point is an op-level replacement for one function of the reference's
 * `gpu::ops` seam (Rust, paths below are inside the reference project): the body of the
 * Rust function calls the C function instead of launching its NVRTC kernels.
 *
 * Conventions (the reference's own, src/gpu/buf.rs:24-30, src/gpu/mod.rs:128-148):
 *   - all data pointers are DEVICE pointers; the caller allocates every input, output,
 *     saved buffer and workspace; the callee writes every element of its outputs;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) in program order; no
 *     call synchronises the stream or the device;
 *   - tensors are contiguous row-major; q/k/v and gate logits are position-major
 *     [B*T, H*W]: element (b,h,t,c) at ((b*T+t)*H+h)*W+c (src/gpu/ops.rs:4357-4366);
 *   - a NULL carry means "zero state", materialised by the kernel, not by a memset
 *     (src/gpu/cuda/mlstm_fused.cu:455-465);
 *   - the storage width of the narrow ("slab") tensors is explicit in every call
 *     (XLSTM_F32 / XLSTM_BF16) instead of a process-wide switch (src/gpu/kernels.rs:208-215);
 *   - there is no CPU fallback: without a CUDA device every compute call returns
 *     XLSTM_ERR_CUDA.
 *
 * Return value: XLSTM_OK, XLSTM_DECLINED (shape not supported by this engine — nothing
 * was launched; mirrors the reference's `bool` "declined" fast paths, src/gpu/ops.rs:
 * 2712-2777), or a negative error. xlstm_last_error() gives the text of the last failure
 * on the calling thread.
 */
#ifndef XLSTM_B200_H
#define XLSTM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XLSTM_OK 0
#define XLSTM_DECLINED 1
#define XLSTM_ERR_ARG (-1)
#define XLSTM_ERR_CUDA (-2)
#define XLSTM_ERR_TIMEOUT (-3)
#define XLSTM_ERR_WORKSPACE (-4)

#define XLSTM_F32 0
#define XLSTM_BF16 1

/* flags */
#define XLSTM_FORCE_SIMT 1u /* use the CUDA-core kernels even where a tensor-core kernel exists */
/* Sequences of at most 32 positions that neither take nor leave a state (the hierarchical model's word rectangles:
 * thousands of 9-position sequences per call; no reference counterpart, its kernels take one sequence per block):
 * the tensor-core kernels put 64 / T of them into each 64-row chunk tile, with gate scans that restart at every
 * sequence and a block-diagonal decay mask, instead of one ragged tile per sequence. Set it on the forward call and on
 * its backward call alike (the state record is laid out tile by tile); a call with the flag that passes a carry, asks
 * for a state or a state gradient, or has T > 32 is refused. Ignored where the tensor-core path does not apply or the
 * heads are not 128 x 128 (the call then runs as without the flag). Results are those of the unpacked call. */
#define XLSTM_PACK_SHORT 2u

int xlstm_version(void);
const char* xlstm_last_error(void);
/* Number of kernels this library has launched from the calling process so far. */
uint64_t xlstm_launch_count(void);
/* Synchronising health check: XLSTM_OK, or XLSTM_ERR_TIMEOUT if a kernel launched earlier gave up
 * on a bounded device-side wait (it then unwound cleanly and its outputs are invalid). Clears the
 * flag. Copies one word from the device, so it waits for work already enqueued. */
int xlstm_device_status(void);

/* ---- chunkwise mLSTM core -------------------------------------------------------------
 * Replaces ops::mlstm_fused_fw / ops::mlstm_fused_bw (src/gpu/ops.rs:4380-4537,
 * 4546-4707) and their kernels (src/gpu/cuda/mlstm_fused.cu:136,224,271,415,514,747,859).
 */
typedef struct {
    int B, H, T, dqk, dhv;
    int L;          /* chunk length (blocking only: results do not depend on it). L = 64 with bf16 storage and
                       dqk, dhv multiples of 128 up to 512 selects the tensor-core kernels, for every T >= 1: a
                       sequence shorter than a chunk is one ragged chunk. Everything else runs on the CUDA-core
                       kernels with min(L, T) as the chunk. */
    int dtype;      /* storage of q, k, v, ytil                (MlstmShape + SlabBuf width) */
    int gdtype;     /* storage of d_ytil, dq, dk, dv            (reference: always f32) */
    unsigned flags;
} xlstm_mlstm_shape;

/* Bytes of the opaque chunk-state record the forward can leave for the backward
 * (the reference's cst/nst arrays, src/gpu/ops.rs:3955-3967). Passing saved=NULL to
 * both calls makes the backward recompute the chunk-boundary states instead. */
size_t xlstm_mlstm_saved_bytes(const xlstm_mlstm_shape* s);
size_t xlstm_mlstm_fw_workspace_bytes(const xlstm_mlstm_shape* s);
size_t xlstm_mlstm_bw_workspace_bytes(const xlstm_mlstm_shape* s, int have_saved);

/* q,k [B*T,H*dqk] (k pre-scaled by 1/sqrt(dqk), src/gpu/mlstm.rs:241-252), v [B*T,H*dhv]
 * at `dtype`; ig,fg [B*T,H] f32 gate logits; carry_* the state the call continues from
 * (C [BH,dhv,dqk], n [BH,dqk], m [BH], f32; all three NULL = start at zero).
 * Outputs: ytil [B*T,H*dhv] at `dtype`; msv (stabiliser m_t), psiv (normaliser psi_t),
 * qnv (q·n before the floor), each [BH,T] f32; saved (optional); out_* the state after
 * the last position (optional, f32). */
int xlstm_mlstm_fw(void* stream, const xlstm_mlstm_shape* s, const void* q, const void* k,
                   const void* v, const float* ig, const float* fg, const float* carry_C,
                   const float* carry_n, const float* carry_m, void* ytil, float* msv,
                   float* psiv, float* qnv, void* saved, float* out_C, float* out_n,
                   float* out_m, void* workspace, size_t workspace_bytes);

/* The state a call would end in, without its outputs: the recurrence over (C, n, m) alone, about half a
 * forward's time. New (the reference has no such entry): context parallelism summarises a segment with it
 * before the carry from the ranks to its left is known. Arguments as in xlstm_mlstm_fw; out_* required. */
int xlstm_mlstm_final_state(void* stream, const xlstm_mlstm_shape* s, const void* q, const void* k,
                            const void* v, const float* ig, const float* fg, const float* carry_C,
                            const float* carry_n, const float* carry_m, float* out_C, float* out_n,
                            float* out_m);

/* Backward with the stabiliser held constant. d_ytil [B*T,H*dhv] at `gdtype`;
 * carry_dC [BH,dhv,dqk], carry_dn [BH,dqk] f32: gradient w.r.t. the state this call left
 * (NULL = zero), out_dC/out_dn: gradient w.r.t. the state it entered with (optional).
 * dq,dk [B*T,H*dqk], dv [B*T,H*dhv] at `gdtype`; dig,dfg [B*T,H] f32. */
int xlstm_mlstm_bw(void* stream, const xlstm_mlstm_shape* s, const void* q, const void* k,
                   const void* v, const float* ig, const float* fg, const float* carry_C,
                   const float* carry_n, const float* carry_m, const void* ytil,
                   const float* msv, const float* psiv, const float* qnv, const void* saved,
                   const void* d_ytil, const float* carry_dC, const float* carry_dn, void* dq,
                   void* dk, void* dv, float* dig, float* dfg, float* out_dC, float* out_dn,
                   void* workspace, size_t workspace_bytes);

/* ---- sLSTM recurrent loop ---------------------------------------------------------------
 * Replaces ops::slstm_fused_time / slstm_fused_time_bwd (src/gpu/ops.rs:2787-2880,
 * src/gpu/cuda/slstm_coop.cu:103,374). All tensors f32.
 *   wh: NH==1: dense [H,4H] (gate blocks z,i,f,o);  NH>1: block-diagonal [NH,dh,4*dh],
 *       dh=H/NH, row = source unit inside the head, column = gate*dh + unit in the head.
 *   g [B,T,4H]: x·Wx on entry; forward overwrites its f block with the biased
 *       pre-activation, backward overwrites all of it with the four gate deltas.
 *   state c,n,m,h [B,H]: read when carry!=0 (else zero), always written.
 *   slabs: nine [B,T,H] records in this order:
 *       c_prev, n_prev, i', f', c, n, z, o, h_prev   (src/gpu/ops.rs:2206-2256).
 * Heads of up to 256 units run on thread-block clusters. Wider heads (dense H up to 1024, block-diagonal
 * heads up to 512 units) run as ONE cooperative launch spanning the GPU, whose CTAs wait on one another
 * with bounded polls (a timeout shows in xlstm_device_status); that path uses barrier words, a 2 MiB
 * exchange array and (backward) a grow-only exchange buffer held by the library per device, so keep
 * those calls on one stream per device, as the reference keeps all its calls. Anything wider returns 1.
 */
typedef struct {
    float *c_prev, *n_prev, *ipr, *fpr, *c, *n, *zt, *ot, *h_prev;
} xlstm_slstm_slabs;

int xlstm_slstm_fw(void* stream, const float* wh, float* g, const float* bcat, float* c,
                   float* n, float* m, float* h, float* out, const xlstm_slstm_slabs* slabs,
                   int B, int H, int NH, int T, int carry, unsigned flags);
/* dh,dc,dn [B,H]: BPTT state, read when carry!=0 (else zero), always written. */
int xlstm_slstm_bw(void* stream, const float* wh, const float* dy, float* g, float* dh,
                   float* dc, float* dn, const xlstm_slstm_slabs* slabs, int B, int H, int NH,
                   int T, int carry, unsigned flags);

/* ---- grouped RMSNorm -----------------------------------------------------------------------
 * Replaces ops::rms_norm_forward_into / rms_norm_backward_into (src/gpu/ops.rs:1601-1685).
 * x,y [rows,F]; gamma [F] f32; inv_rms [rows*F/group] f32. x_hat (f32) may be NULL (the backward
 * rebuilds it from x and inv_rms). x may be stored as bf16 (the mLSTM core's output feeding the
 * head-wise norm) and y may be written as bf16 where only GEMMs consume it: the casts the reference
 * launches around the norm (src/gpu/cuda/bf16_cast.cu:22-60) happen inside it. */
int xlstm_rmsnorm_fw(void* stream, const void* x, int x_dtype, const float* gamma, void* y, int y_dtype,
                     float* inv_rms, float* x_hat, int rows, int F, int group, float eps);
size_t xlstm_rmsnorm_bw_workspace_bytes(int rows, int F);
/* dgamma [F] is ACCUMULATED into (+=), by a fixed-order two-stage column sum. dy f32; x at x_dtype;
 * dx at dx_dtype. residual (f32 [rows,F], or NULL) is added to dx: the gradient that reaches the same
 * tensor through the block's skip connection (the reference adds it with a pass of its own,
 * src/gpu/block.rs:856-909). */
int xlstm_rmsnorm_bw(void* stream, const float* dy, const void* x, int x_dtype, const float* inv_rms,
                     const float* gamma, const float* residual, void* dx, int dx_dtype, float* dgamma,
                     int rows, int F, int group, void* workspace, size_t workspace_bytes);

/* ---- softmax cross-entropy, forward + backward in one pass ---------------------------------
 * Replaces ops::softmax_cross_entropy and masked_softmax_ce_u32_into (src/gpu/ops.rs:
 * 1689-1714, 3567-3618). logits [rows,C] f32; targets u32 [rows]; mask u32 [rows] or NULL;
 * dlogits = (p - onehot)*inv (may alias logits); *loss_accum += inv * sum of row losses,
 * added on the device (no host read-back). */
size_t xlstm_ce_workspace_bytes(int rows);
int xlstm_ce_fw_bw(void* stream, const float* logits, const uint32_t* targets,
                   const uint32_t* mask, float* dlogits, float* loss_accum, int rows, int C,
                   float inv, void* workspace, size_t workspace_bytes);

/* The same loss with the flat LM's soft-cap folded in (reference: softcap_forward/backward,
 * src/gpu/cuda/common.cu:4-12, applied by gpu::Lm between the head and the loss, src/gpu/lm.rs:84-163):
 * pre_logits are the head's outputs x, the loss is taken on cap*tanh(x/cap), and d_pre (may alias
 * pre_logits) is the gradient with respect to x. Saves the capped logits' round trips through HBM. */
int xlstm_softcap_ce_fw_bw(void* stream, const float* pre_logits, const uint32_t* targets,
                           const uint32_t* mask, float* d_pre, float* loss_accum, int rows, int C,
                           float inv, float cap, void* workspace, size_t workspace_bytes);

/* The same op for hosts that cannot allocate device memory (a runtime whose buffer pool already
 * owns all of it, or a step loop that must stay clear of the CUDA allocator): the per-row scratch
 * is a fixed array inside the library instead of a caller workspace. It has no counterpart in the
 * reference. At most XLSTM_CE_NOALLOC_MAX_ROWS rows per call, larger calls are refused with
 * XLSTM_ERR_ARG. All calls on one device share the array: calls that may overlap on the GPU race,
 * so keep them on one stream. The first call on a device resolves the array's address and should
 * be made before any stream capture begins. */
#define XLSTM_CE_NOALLOC_MAX_ROWS 65536
int xlstm_ce_fw_bw_noalloc(void* stream, const float* logits, const uint32_t* targets,
                           const uint32_t* mask, float* dlogits, float* loss_accum, int rows,
                           int C, float inv);

/* ---- element-wise glue, one pass each (replace swiglu_forward/backward, src/gpu/cuda/block.cu:6-29, and
 * ogate_fwd/ogate_bwd, src/gpu/cuda/mlstm_ops.cu:147-153, 400-407, with the bf16 narrowing of outputs
 * that feed a GEMM folded in, src/gpu/cuda/bf16_cast.cu:22-60). Flat arrays of n elements; out_dtype is
 * XLSTM_F32 or XLSTM_BF16 and applies to the outputs typed void*. */
/* out = SiLU(gate_pre + bias_gate) * (value + bias_value). The biases ([cols] each, or both NULL) are the
 * gate/value projections' biases, folded in here so that those GEMMs need no bias pass (the reference seeds
 * the GEMM output with broadcast_row, src/gpu/cuda/common.cu:20-48); element i is in column i % cols. */
int xlstm_swiglu_fw(void* stream, const void* gate_pre, const void* value, int in_dtype, const float* bias_gate,
                    const float* bias_value, int cols, void* out, int out_dtype, size_t n);
/* with g = gate_pre + bias_gate, v = value + bias_value: d_gate = d_mixed * v * SiLU'(g); d_value = d_mixed * SiLU(g).
 * in_dtype is the width of gate_pre / value (a bf16 layer takes them narrow straight from its GEMMs' epilogues),
 * d_dtype that of d_mixed; bf16 inputs need bf16 outputs. */
int xlstm_swiglu_bw(void* stream, const void* d_mixed, int d_dtype, const void* gate_pre, const void* value,
                    int in_dtype, const float* bias_gate, const float* bias_value, int cols, void* d_gate,
                    void* d_value, int out_dtype, size_t n);
/* o <- sigmoid(o + bias) in place; hc = o * yhat. bias ([cols], or NULL) is the output-gate projection's
 * bias, folded in here like the SwiGLU biases above. */
int xlstm_ogate_fw(void* stream, float* o, const float* yhat, const float* bias, int cols, void* hc, int out_dtype,
                   size_t n);
/* do_pre = d_hc * yhat * o * (1 - o) with o the activated gate; d_yhat = d_hc * o (fp32) */
int xlstm_ogate_bw(void* stream, const float* d_hc, const float* o, const float* yhat, void* do_pre,
                   int out_dtype, float* d_yhat, size_t n);
/* x = hi + mid + lo as three bf16 arrays (hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid)): the
 * operands of an fp32-accurate product run as six bf16 tensor-core GEMMs (the fp32 head of gpu::Lm,
 * src/gpu/lm.rs:84-163, which the reference runs as a cublasSgemm). No reference counterpart. */
int xlstm_split3_bf16(void* stream, const float* x, void* hi, void* mid, void* lo, size_t n);

/* Bias gradient of a projection, with the narrowing of the same tensor for the two weight-side GEMMs folded in
 * (replaces add_col_sum, src/gpu/cuda/common.cu:49-124, and a cast, src/gpu/cuda/bf16_cast.cu:22-60):
 * acc[c] += scale * sum_r x[r][c] (fixed summation order, no float atomics); if out_bf16 is not NULL,
 * out_bf16[r][c] = bf16(scale * x[r][c]). x [rows, cols] at x_dtype. */
size_t xlstm_colsum_workspace_bytes(int rows, int cols);
int xlstm_colsum_narrow(void* stream, const void* x, int x_dtype, int rows, int cols, float scale, void* out_bf16,
                        float* acc, void* workspace, size_t workspace_bytes);
/* out[r][c] = bias[c] (+ residual[r][c] when given): the seed a projection's GEMM accumulates into with beta = 1
 * (broadcast_row / broadcast_row_resid, src/gpu/cuda/common.cu:20-48). f32, [rows, cols]. */
int xlstm_bias_rows(void* stream, const float* residual, const float* bias, float* out, int rows, int cols);

/* Embedding backward without float atomics (replaces embedding_scatter_add / embedding_scatter_merge,
 * src/gpu/cuda/common.cu:127-168): table_g[id] += sum of the rows d[pos] with ids[pos] == id, in ascending
 * position order. The caller passes the ids sorted stably (`sorted_ids`) and the positions in that order
 * (`order`), both int32 [n]; d is [n, dm] fp32, table_g [vocab, dm] fp32. */
int xlstm_embedding_scatter_add(void* stream, const float* d, const int* sorted_ids, const int* order,
                                float* table_g, int n, int dm);


/* ---- AdamW over many tensors ----------------------------------------------------------------
 * Replaces ops::adamw and AdamwQueue::flush (src/gpu/ops.rs:1775-1933, src/gpu/cuda/
 * common.cu:323-361). `descs` is a HOST array. bc1 = 1-beta1^t, bc2 = 1-beta2^t are
 * computed by the caller as the reference does. p_bf16 (optional) receives the bf16 copy
 * of the updated parameter in the same pass; zero_grad!=0 clears g after use. */
typedef struct {
    float* p;
    float* g;
    float* m;
    float* v;
    void* p_bf16;
    uint64_t len;
    float wd; /* this tensor's decoupled weight decay (0 for biases and norm scales) */
    float _pad;
} xlstm_adamw_desc;

int xlstm_adamw_multi(void* stream, const xlstm_adamw_desc* descs, int n, float lr,
                      float beta1, float beta2, float eps, float bc1, float bc2, int zero_grad);

/* ---- data-parallel gradient buckets over NCCL --------------------------------------------------
 * No counterpart in the reference, which trains on one GPU (src/gpu/mod.rs:134); this is what a host
 * that runs one replica per GPU calls around its backward pass and in front of AdamwQueue::flush
 * (src/gpu/hierarchical.rs:1696-1746). Gradients live in flat fp32 buckets the caller owns. NCCL is
 * bound at run time (libnccl.so.2; a copy the process already holds is reused). State is per device:
 * make the device current first, and keep the calls for one device on one host thread.
 *   xlstm_dp_unique_id:  rank 0 obtains the 128-byte id and hands it to every rank (any host channel).
 *   xlstm_dp_init:       collective over the ranks; creates the communicator for the current device.
 *   xlstm_dp_init_comm:  adopt a communicator (ncclComm_t) the host already has; never destroyed here.
 *   xlstm_dp_bucket_register: returns the bucket's index (>= 0) or a negative error.
 *   xlstm_dp_bucket_start: call when everything enqueued on producer_stream so far has written the
 *       bucket; a SUM all-reduce (in place, fp32) is ordered behind that point on a library-owned
 *       high-priority stream and runs while producer_stream carries on with the layers below.
 *   xlstm_dp_wait:       `stream` waits for every reduction started since the last wait.
 * With the loss scaled by 1 / (rows * ranks) on every rank the summed gradient is the gradient of the
 * global mean loss. Plain NCCL collectives only. */
int xlstm_dp_unique_id(void* out128);
int xlstm_dp_init(int nranks, int rank, const void* unique_id128);
int xlstm_dp_init_comm(void* nccl_comm);
int xlstm_dp_world(void); /* ranks of the current device's communicator, 0 if none */
int xlstm_dp_bucket_register(float* grads, size_t n);
int xlstm_dp_bucket_start(int index, void* producer_stream);
int xlstm_dp_wait(void* stream);
int xlstm_dp_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif
