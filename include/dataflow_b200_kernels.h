/*
 * dataflow_b200_kernels.h -- the C-ABI between host C code and the sm_100a kernels.
 *
 * Plain pointers and sizes only. Every function enqueues work on `stream` (a CUstream /
 * cudaStream_t passed as void *, NULL = the legacy default stream) of the CURRENT device and
 * returns without synchronising. Datatypes are DataflowDatatype values (dataflow_abi.h).
 * Return value: DFB200_OK, or a negative DFB200_ERR_* code; dfb200_last_error() gives the
 * message of the last failure on the calling thread. Nothing here falls back to the CPU.
 *
 * Each entry point replaces one family of `<op>_<dtype>_kernel` symbols of the reference's
 * cubin together with its `<op>_set_launch_config` host function; the argument order after
 * the datatypes is the reference kernel's parameter order.
 *
 * Alignment contract (checked, DFB200_ERR_ARG otherwise): tensor base pointers are 16-byte
 * aligned and row lengths are multiples of 8 elements, so that every 8-element packet of a
 * row (128 bits for 16-bit types, 2 x 128 for fp32, 64 for fp8) is naturally aligned.
 */
#ifndef DATAFLOW_B200_KERNELS_H
#define DATAFLOW_B200_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFB200_OK             0
#define DFB200_ERR_ARG       -1   /* NULL / misaligned pointer, bad size */
#define DFB200_ERR_DTYPE     -2   /* datatype combination the op does not have */
#define DFB200_ERR_CUDA      -3   /* launch or runtime error (message holds cudaGetErrorString) */
#define DFB200_ERR_WORKSPACE -4   /* workspace missing or too small */

const char * dfb200_last_error(void);

/* Synchronises `stream` and returns the kernels' status: 0 when every bounded device-side wait
 * (for an asynchronous copy) completed, otherwise a positive code naming the wait that gave up
 * (also copied per kernel family into status_words[0..n_words) when non-NULL); negative on a
 * CUDA error. The status words are cleared when non-zero. */
int dfb200_read_kernel_status(void * stream, unsigned int * status_words, int n_words);

/* Self-test of the bounded waits: a kernel waits (about two seconds, the limit) on a barrier nothing completes, gives up, records code
 * 0x7e57 in status word `slot` and ends normally. Returns 1 when the wait gave up as designed. Allocates a 4-byte flag for the call. */
int dfb200_selftest_bounded_wait(int slot, void * stream);

/* Library build info: "sm_100a", and the SM count of the current device (0 if no device). */
const char * dfb200_target_arch(void);
int dfb200_sm_count(void);

/* ---- RMSNorm ----------------------------------------------------------------------------
 * Replaces rms_norm_<dt>_kernel (src/ops/nvidia/norm/rms_norm.cu:4,143,280,415,539) and
 * rms_norm_set_launch_config / rms_norm_set_attribute_config (src/ops/nvidia/norm/rms_norm_config.c:3-79).
 * out[r,i] = T( (f32(X[r,i]) * rms[r]) * f32(w[i]) ),  rms[r] = rsqrt(mean_i X[r,i]^2 + eps);
 * weighted_sums[r] = sum_i w[i]*X[r,i] and rms_vals[r] = rms[r] are written when non-NULL. */
int dfb200_rms_norm(int fwd_dt, int n_rows, int n_cols, float eps,
                    const void * rms_weight, const void * X, void * out,
                    float * weighted_sums, float * rms_vals, void * stream);

/* Replaces rms_norm_bwd_x_<fwd>_<bwd>_kernel (src/ops/nvidia/norm/rms_norm_bwd_x.cu:4-590) and
 * rms_norm_bwd_x_set_launch_config (src/ops/nvidia/norm/rms_norm_config.c:81-151).
 * dX[r,i] += dY[r,i] * B( w[i]*rms[r] - (X[r,i]*rms[r]^3 / n_cols) * weighted_sums[r] )
 * with the multiply-add done as one fused operation in the bwd datatype B, as the reference
 * binary does (the reference's formula, which accumulates into dX). */
int dfb200_rms_norm_bwd_x(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps,
                          const float * fwd_weighted_sums, const float * fwd_rms_vals,
                          const void * rms_weight, const void * X_inp,
                          const void * upstream_dX, void * dX, void * stream);

/* Replaces rms_norm_bwd_w_<fwd>_<bwd>_kernel (src/ops/nvidia/norm/rms_norm_bwd_w.cu:4-700) and
 * rms_norm_bwd_w_set_launch_config (src/ops/nvidia/norm/rms_norm_config.c:154-222).
 * dW[c] = B( f32(dW[c]) + sum_r f32(dY[r,c]) * f32(X[r,c]) * rms[r] ), reduced in fp32 in a
 * fixed order (two launches, no atomics). Needs dfb200_rms_norm_bwd_w_workspace_bytes() bytes
 * of 16-byte aligned device scratch; its contents on entry do not matter. */
uint64_t dfb200_rms_norm_bwd_w_workspace_bytes(int n_rows, int n_cols);
int dfb200_rms_norm_bwd_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps,
                          const float * fwd_rms_vals, const void * X_inp,
                          const void * upstream_dX, void * dW,
                          void * workspace, uint64_t workspace_bytes, void * stream);

/* No counterpart in the reference (its kernel accumulates into dW with atomics in the gradient's own type): the same reduction with
 * the column sums WRITTEN as fp32 -- column_sums[c] = sum_r f32(dY[r,c]) * f32(X[r,c]) * rms[r], overwritten, nothing read -- which is
 * what a token-sharded caller all-reduces: column_sums can be a slot of the packed fp32 exchange buffer (dataflow_b200_exchange.h),
 * so nothing has to be packed or unpacked around the collective. Same workspace as dfb200_rms_norm_bwd_w. */
int dfb200_rms_norm_bwd_w_sums(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps,
                               const float * fwd_rms_vals, const void * X_inp,
                               const void * upstream_dX, float * column_sums,
                               void * workspace, uint64_t workspace_bytes, void * stream);

/* No counterpart in the reference, which launches rms_norm_bwd_x and rms_norm_bwd_w one after the other, each reading X and dY
 * (src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c: the backward of every norm): both in ONE pass over X and
 * dY -- 4 * n_cols elements of traffic per row instead of 6. dX is what dfb200_rms_norm_bwd_x writes, bit for bit; dW (the
 * accumulating form) or column_sums (the fp32 form of dfb200_rms_norm_bwd_w_sums) differ from the separate op's only by the order
 * of the fp32 additions over the rows. Same workspace as dfb200_rms_norm_bwd_w. Row lengths or alignments the 16-byte packet
 * kernels cannot take run as the two separate general-shape passes. */
int dfb200_rms_norm_bwd_x_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps,
                            const float * fwd_weighted_sums, const float * fwd_rms_vals,
                            const void * rms_weight, const void * X_inp, const void * upstream_dX,
                            void * dX, void * dW, void * workspace, uint64_t workspace_bytes, void * stream);
int dfb200_rms_norm_bwd_x_w_sums(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps,
                                 const float * fwd_weighted_sums, const float * fwd_rms_vals,
                                 const void * rms_weight, const void * X_inp, const void * upstream_dX,
                                 void * dX, float * column_sums, void * workspace, uint64_t workspace_bytes, void * stream);

/* No counterpart in the reference. rms_norm_bwd_w for callers that cannot allocate device memory or pass a
 * workspace: a program whose own arena already owns the whole device (one bulk alloc_mem at start-up), or a step
 * loop that must not hit cudaMalloc's device-wide synchronisation. Same results as dfb200_rms_norm_bwd_w; the
 * partial sums go to a 5 MiB array built into the library (held by every GPU that loads it until exit), so
 * n_SM * n_cols must be <= 1,310,720 (n_cols <= 8192 on a 148-SM B200) or the call fails with
 * DFB200_ERR_WORKSPACE. The first call on a device resolves the array's address: issue it before any stream
 * capture. Calls share the array: calls that overlap on the GPU race, so keep them ordered. */
int dfb200_rms_norm_bwd_w_static(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps,
                                 const float * fwd_rms_vals, const void * X_inp,
                                 const void * upstream_dX, void * dW, void * stream);

/* ---- RoPE -------------------------------------------------------------------------------
 * Replaces rope_<dt>_kernel (src/ops/nvidia/attention/rope.cu:3,60,123,183,243), rope_bwd_x_<dt>_kernel
 * (src/ops/nvidia/attention/rope_bwd_x.cu:3,62,120) and their launch configs
 * (src/ops/nvidia/attention/attn_misc_config.c:3-53). N = tokens * model_dim. In place on
 * X_q [tokens, model_dim] and X_k [tokens, num_kv_heads*head_dim]; interleaved pairs (2j, 2j+1)
 * of each head are rotated by angle pos * theta^(-2j/head_dim); bwd applies the transpose. */
int dfb200_rope(int fwd_dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                const int * seq_positions, void * X_q, void * X_k, void * stream);
int dfb200_rope_bwd_x(int bwd_dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                      const int * seq_positions, void * dX_q, void * dX_k, void * stream);

/* ---- SwiGLU -----------------------------------------------------------------------------
 * Replaces swiglu_<dt>_kernel (src/ops/nvidia/activations/swiglu.cu:4-112), swiglu_bwd_x_<f>_<b>_kernel
 * (src/ops/nvidia/activations/swiglu_bwd_x.cu:4-185) and src/ops/nvidia/activations/swiglu_config.c:4-50.
 * out = silu(x_w1) * x_w3;  dX_w3 = dY*silu(x_w1);  dX_w1 = dY * x_w3 * dsilu(x_w1). */
int dfb200_swiglu(int fwd_dt, int num_rows, int num_cols,
                  const void * x_w1, const void * x_w3, void * out, void * stream);
int dfb200_swiglu_bwd_x(int fwd_dt, int bwd_dt, int num_rows, int num_cols,
                        const void * x_w1, const void * x_w3, const void * upstream_dX,
                        void * dX_w1, void * dX_w3, void * stream);

/* ---- softmax / cross entropy ------------------------------------------------------------
 * dfb200_softmax replaces softmax_<f>_<b>_kernel (src/ops/nvidia/loss/softmax.cu:3-960) and
 * softmax_set_launch_config (src/ops/nvidia/loss/loss_misc_config.c:3-26): row softmax with the
 * reference's rounding points (max and x-max in the input type, 32 interleaved partial sums
 * and the row total rounded to the input type). One HBM read and one write per element.
 * dfb200_cross_entropy_loss replaces cross_entropy_loss_<dt>_kernel
 * (src/ops/nvidia/loss/cross_entropy.cu:5,19,33) with its intended semantics:
 * pred[r, labels[r]] -= 1 for every row r; rows whose label is >= n_cols are left untouched. */
int dfb200_softmax(int fwd_dt, int bwd_dt, int n_rows, int n_cols,
                   const void * X, void * out, void * stream);
int dfb200_cross_entropy_loss(int bwd_dt, int n_rows, int n_cols,
                              void * pred_logits, const uint32_t * labels, void * stream);

/* Fused softmax + cross entropy, forward and backward in one pass over the logits (no
 * counterpart in the reference, which runs the two kernels above back to back and never
 * computes the loss value). dlogits = softmax(logits) - onehot(labels), bit-identical to
 * dfb200_softmax followed by dfb200_cross_entropy_loss; row_loss[r] = log(sum_r) - (x[r,label]-max_r)
 * in fp32 (optional); loss_sum[0] = sum_r row_loss[r] accumulated in fp64 in a fixed order and
 * stored as fp32, loss_sum[1] = number of rows with a valid label (both optional, 2 floats).
 * workspace: dfb200_softmax_cross_entropy_workspace_bytes() bytes of device scratch. */
uint64_t dfb200_softmax_cross_entropy_workspace_bytes(int n_rows, int n_cols);
int dfb200_softmax_cross_entropy(int fwd_dt, int bwd_dt, int n_rows, int n_cols,
                                 const void * logits, const uint32_t * labels, void * dlogits,
                                 float * row_loss, float * loss_sum,
                                 void * workspace, uint64_t workspace_bytes, void * stream);

/* ---- FP8-weight SwiGLU FFN, forward and input-gradient backward ---------------------------------
 * No counterpart in the reference (its only GEMM is the external cuBLASLt call, without scales:
 * src/ops/nvidia/external/matmul_helper/src/matmul_helper.c:577-657). tcgen05 tensor-core GEMMs with fp32
 * accumulation in tensor memory. Weights: e4m3, stored [out_features, in_features] row-major, one fp32 scale per
 * output channel (w = code * scale). Activations: bf16, quantised inside to e4m3 with one scale per row.
 *   dfb200_quantize_rows_e4m3    v = X[r,c] * col_factors[c] (factors optional); Q = e4m3(v * 448 / amax_r); row_scales[r] = amax_r / 448
 *   dfb200_gemm_e4m3             out[m,n] = bf16( (sum_k A[m,k] W[n,k]) * a_row_scales[m] * w_scales[n] + residual[m,n] )
 *                                (w_scales and residual may be NULL; residual bf16 [M,N], may alias out)
 *   dfb200_gemm_e4m3_swiglu      H[m,n] = bf16( silu(g) * u ), g / u = the same with the gate / up weights; g and u are also stored
 *                                (bf16 [M,N]) when gate_save / up_save are given
 *   dfb200_gemm_e4m3_swiglu_bwd  dh = (sum_k dOut[m,k] WdownT[n,k]) * row_scale[m]; [dG | dU][m, n and N+n] from dh and the saved g, u
 *   dfb200_swiglu_ffn_fp8        out = down(swiglu(gate(A), up(A))) + residual (optional);  dfb200_swiglu_ffn_fp8_bwd: dA from dOut and the saved g, u
 *   dfb200_ffn_fp8_prepare_bwd_weights  WgateupT [d, 2f] = [Wgate^T | Wup^T], WdownT [f, d] = Wdown^T (codes only)
 * Both FFN calls take dfb200_swiglu_ffn_fp8_workspace_bytes() bytes of scratch from the caller; weight gradients: dfb200_swiglu_ffn_fp8_wgrad.
 * Shapes: reduction lengths multiples of 16, N a multiple of 8, 16-byte aligned tensors, row length of a quantised matrix <= 32768. */
int dfb200_quantize_rows_e4m3(int n_rows, int n_cols, const void * X_bf16, const float * col_factors, void * Q_e4m3, float * row_scales, void * stream);
int dfb200_transpose_bytes(int rows, int cols, const void * in, int ld_in, void * out, int ld_out, void * stream);
int dfb200_gemm_e4m3(int M, int N, int K, const void * A_e4m3, const float * a_row_scales, const void * W_e4m3, const float * w_scales,
                     const void * residual_bf16, void * out_bf16, void * stream);
int dfb200_gemm_e4m3_swiglu(int M, int N, int K, const void * A_e4m3, const float * a_row_scales, const void * Wgate_e4m3,
                            const float * gate_scales, const void * Wup_e4m3, const float * up_scales, void * H_bf16,
                            void * gate_save_bf16, void * up_save_bf16, void * stream);
/* Row quantisation fused with the elementwise op that makes the row (the bf16 intermediate is never stored):
 *   dfb200_swiglu_quantize_rows_e4m3      codes [n_rows, f]  of h = bf16(silu(gate) * up)                      (arithmetic of dfb200_swiglu)
 *   dfb200_swiglu_bwd_quantize_rows_e4m3  codes [n_rows, 2f] of [dgate | dup] = swiglu_bwd_x(gate, up, dH) in bf16, times col_factors[2f]
 *                                         (arithmetic of dfb200_swiglu_bwd_x; col_factors may be NULL, else 16-byte aligned) */
int dfb200_swiglu_quantize_rows_e4m3(int n_rows, int f, const void * gate_bf16, const void * up_bf16, void * Q_e4m3, float * row_scales, void * stream);
int dfb200_swiglu_bwd_quantize_rows_e4m3(int n_rows, int f, const void * gate_bf16, const void * up_bf16, const void * dH_bf16,
                                         const float * col_factors, void * Q_e4m3, float * row_scales, void * dgate_dup_bf16 /* [n_rows, 2f] or NULL */,
                                         void * stream);
/* Operands of the weight-gradient GEMMs (reduction over the rows): the transpose, quantised with one scale per row of the transpose.
 *   dfb200_col_amax_bf16            col_amax[c] = max_r |X[r, c]|
 *   dfb200_transpose_quantize_e4m3  Qt[c, r] = e4m3( X[r, c] * 448 / col_amax[c] ), col_scales[c] = col_amax[c] / 448 (1 for an all-zero column);
 *                                   n_rows a multiple of 16, n_cols of 8 */
int dfb200_col_amax_bf16(int n_rows, int n_cols, const void * X_bf16, float * col_amax, void * stream);
int dfb200_transpose_quantize_e4m3(int n_rows, int n_cols, const void * X_bf16, const float * col_amax, void * Qt_e4m3, float * col_scales, void * stream);
int dfb200_gemm_e4m3_swiglu_bwd(int M, int N, int K, const void * dOut_e4m3, const float * dout_row_scales, const void * WdownT_e4m3,
                                const void * gate_saved_bf16, const void * up_saved_bf16, void * dgate_dup_bf16, void * stream);
uint64_t dfb200_swiglu_ffn_fp8_workspace_bytes(int T, int d, int f);
int dfb200_swiglu_ffn_fp8(int T, int d, int f, const void * A_bf16, const void * Wgate, const float * gate_scales, const void * Wup,
                          const float * up_scales, const void * Wdown, const float * down_scales, const void * residual_bf16, void * out_bf16,
                          void * gate_save_bf16, void * up_save_bf16, void * workspace, uint64_t workspace_bytes, void * stream);
int dfb200_ffn_fp8_prepare_bwd_weights(int d, int f, const void * Wgate, const void * Wup, const void * Wdown, void * WgateupT, void * WdownT,
                                       void * stream);
int dfb200_swiglu_ffn_fp8_bwd(int T, int d, int f, const void * dOut_bf16, const void * gate_saved_bf16, const void * up_saved_bf16,
                              const void * WdownT, const float * down_scales, const void * WgateupT, const float * gateup_scales,
                              void * dA_bf16, void * dgate_dup_bf16 /* [T, 2f] kept for the weight gradients, or NULL */,
                              void * workspace, uint64_t workspace_bytes, void * stream);
/* Weight gradients (bf16): dWdown[d, f] = dOut^T H, dWgate[f, d] = dG^T A, dWup[f, d] = dU^T A, with H = bf16(silu(g) u) recomputed and
 * [dG | dU] = the dgate_dup_bf16 output of dfb200_swiglu_ffn_fp8_bwd. T, d, f multiples of 16. */
uint64_t dfb200_swiglu_ffn_fp8_wgrad_workspace_bytes(int T, int d, int f);
int dfb200_swiglu_ffn_fp8_wgrad(int T, int d, int f, const void * A_bf16, const void * dOut_bf16, const void * gate_saved_bf16,
                                const void * up_saved_bf16, const void * dgate_dup_bf16, void * dWgate_bf16, void * dWup_bf16, void * dWdown_bf16,
                                void * workspace, uint64_t workspace_bytes, void * stream);

/* Softmax of fp16 / bf16 rows into fp32 probabilities plus the index of each row's maximum: replaces softmax_fp16_fp32_kernel and
 * softmax_bf16_fp32_kernel (src/ops/nvidia/loss/softmax.cu:965-1249). Scratch roundings are in the input type as in the reference,
 * the probabilities are stored unrounded; arg_maxs (optional, uint32 [n_rows]) gets the SMALLEST index holding the maximum. */
int dfb200_softmax_fp32_out(int fwd_dt, int n_rows, int n_cols, const void * X, float * out, uint32_t * arg_maxs, void * stream);

/* ---- row gather / scatter ---------------------------------------------------------------
 * dfb200_embedding            output[t, :] = embedding_table[token_ids[t], :]
 *   replaces embedding_<dt>_kernel (src/ops/nvidia/preprocess/embedding.cu:3-24; the intended row copy -- the
 *   reference's offsets are scaled by the element size twice, :14-20). Any datatype of 1, 2 or 4 bytes.
 * dfb200_copy_to_seq_context  context[t][pos[t], :] = keys[t, :]; context[t][size[t] + pos[t], :] = values[t, :]
 *   replaces copy_to_seq_context_<dt>_kernel (src/ops/nvidia/attention/copy_to_seq_context.cu:3-20).
 *   seq_context_ptrs holds one device address per token; N must equal total_tokens * kv_dim. */
int dfb200_embedding(int dt, int num_tokens, int embed_dim, const uint32_t * token_ids, const void * embedding_table, void * output, void * stream);
int dfb200_copy_to_seq_context(int dt, uint64_t N, int total_tokens, int kv_dim, const void * keys, const void * values,
                               const int * seq_positions, const uint64_t * seq_context_ptrs, const int * seq_context_sizes, void * stream);

/* ---- mixture-of-experts router --------------------------------------------------------------
 * replaces select_experts_<dt>_kernel (src/ops/nvidia/moe/select_experts.cu:3-239): sigmoid scores, top-k by an
 * index-order scan with strict comparisons (slot order as the reference's), weights = score / sum of the chosen
 * scores in the tensor's datatype, uint16 expert ids, expert_counts[e] += tokens routed to e (caller zeroes;
 * n_experts + 1 entries, the last is the kernel's block counter and is left 0), inclusive prefix sum,
 * num_routed_by_expert zeroed. 1 <= top_k <= min(32, n_experts), n_experts <= 8192. Nothing spins. */
int dfb200_select_experts(int dt, int total_tokens, int n_experts, int top_k_experts, const void * X_routed, void * token_expert_weights,
                          uint16_t * chosen_experts, int * expert_counts, int * expert_counts_cumsum, int * num_routed_by_expert, void * stream);

#ifdef __cplusplus
}
#endif
#endif
