/*
 * dataflow_api.h -- host entry points of the library, with the names, argument meaning and
 * return conventions of als244/dataflow_lib (int 0 = ok, -1 = error with a message on stderr;
 * register_* return the number of functions added or -1; alloc_mem returns NULL on failure).
 *
 *   datatype helpers        src/datatype/include/dataflow_datatype.h:42-46, solo_conversion.h:6-16
 *   fingerprints            src/fingerprint/include/fingerprint.h:12-30
 *   hash table              src/table/include/table.h:73-102
 *   handle                  src/dataflow_handle/nvidia/include/cuda_dataflow_handle.h:65-67
 *   skeleton builders       src/set_ops/include/set_native_op_skeletons.h:11-32
 *   submit_* wrappers       src/dataflow_ops/include/dataflow_ops.h:146-215
 */
#ifndef DATAFLOW_API_H
#define DATAFLOW_API_H

#include <stdio.h>
#include "dataflow_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- datatypes ------------------------------------------------------------------------ */
size_t dataflow_sizeof_element(DataflowDatatype arr_dtype);      /* 0 for scalar/none kinds */
char * dataflow_datatype_as_string(DataflowDatatype dtype);      /* "BF16", ... ; "UNKNOWN" otherwise */
/* fp32/fp16/bf16 array conversion on `num_threads` host threads; round-to-nearest-even. */
int dataflow_convert_datatype(void * to, void * from, DataflowDatatype to_dt, DataflowDatatype from_dt, long n, int num_threads);
float solo_bf16_to_fp32(uint16_t a);
uint16_t solo_fp32_to_bf16(float f);
float solo_fp16_to_fp32(uint16_t h);
uint16_t solo_fp32_to_fp16(float f);
uint16_t solo_fp16_to_bf16(uint16_t h);
uint16_t solo_bf16_to_fp16(uint16_t a);

/* ---- fingerprints --------------------------------------------------------------------- */
typedef enum fingerprint_type {
	SHA256_HASH = 0, SHA512_HASH = 1, SHA1_HASH = 2, MD5_HASH = 3, BLAKE3_HASH = 4
} FingerprintType;

void dataflow_sha256(const void * data, uint64_t num_bytes, uint8_t digest[32]);
void do_fingerprinting(void * data, uint64_t num_bytes, uint8_t * ret_fingerprint, FingerprintType fingerprint_type);
uint64_t fingerprint_to_least_sig64(uint8_t * fingerprint, int fingerprint_num_bytes);
uint8_t get_fingerprint_num_bytes(FingerprintType fingerprint_type);
char * get_fingerprint_type_name(FingerprintType fingerprint_type);
void print_hex(uint8_t * fingerprint, int num_bytes);
void print_sha256(uint8_t * fingerprint);

/* ---- hash table ----------------------------------------------------------------------- */
int init_table(Table * table, Hash_Func hash_func, uint64_t key_size_bytes, uint64_t value_size_bytes,
               uint64_t min_table_size, uint64_t max_table_size, float load_factor, float shrink_factor);
void destroy_table(Table * table);
int insert_table(Table * table, void * key, void * value);
/* Returns the slot index or -1. to_copy_value: the value is copied INTO the buffer `ret_value`
 * points to; otherwise *ret_value is set to the value's address inside the table. */
long find_table(Table * table, void * key, bool to_copy_value, void ** ret_value);
int remove_table(Table * table, void * key, void * ret_value);

/* ---- handle --------------------------------------------------------------------------- */
/* Binds the handle to device `device_id`, creates `num_streams` non-blocking streams with one
 * event each and an empty op table, and fills the function-pointer table. The handle uses the
 * device's PRIMARY context (ctx_flags are applied to it when it is not yet active), so memory
 * and streams are interchangeable with CUDA-runtime code in the same process. */
int init_cuda_dataflow_handle(Dataflow_Handle * dataflow_handle, ComputeType compute_type, int device_id,
                              int ctx_id, unsigned int ctx_flags,
                              int num_streams, int * opt_stream_prios, char ** opt_stream_names);
/* Not in the reference: releases streams, events, modules, the op table and the device scratch this library's ops keep. */
void destroy_cuda_dataflow_handle(Dataflow_Handle * dataflow_handle);
/* Not in the reference. The ops with device scratch (rms_norm_bwd_w, softmax_cross_entropy without a row_loss buffer,
 * swiglu_ffn_fp8, swiglu_ffn_fp8_bwd) keep one grow-only block per (op identity, stream id); a block is allocated by the first
 * submission that needs it. dataflow_b200_reserve_workspace sizes the block of (skeleton, stream_id) ahead of time -- `bytes` from
 * the matching dfb200_*_workspace_bytes function of dataflow_b200_kernels.h -- so that no submission inside a step loop allocates
 * (growing a block calls cudaFree, which waits for the whole device). 0 on success, -1 otherwise.
 * dataflow_b200_workspace_release is what destroy_cuda_dataflow_handle calls on every op-table value. */
int dataflow_b200_reserve_workspace(Dataflow_Handle * dataflow_handle, Op_Skeleton * skeleton, int stream_id, uint64_t bytes);
void dataflow_b200_workspace_release(void * op_table_value);

/* ---- op skeletons and registration ---------------------------------------------------- */
/* Registers the 54 (op x datatype) identities of the reference's native op set, plus copy_to_seq_context,
 * select_experts and this library's fused ops, on the handle. `native_function_code_filename` names the shared object
 * that exports the ops; NULL, or a path that is not such a shared object (the reference's "lib/cuda_kernels.cubin", say, in a caller
 * that was not changed), selects the library containing this function, with a notice on stderr;
 * `native_function_config_filename` is accepted for source compatibility and ignored.
 * Returns the number of ops registered. */
int register_native_ops(Dataflow_Handle * dataflow_handle, char * native_function_code_filename, char * native_function_config_filename);
int set_native_op_skeleton(Op_Skeleton * skeleton, char * op_name, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt);
void set_native_embedding_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
void set_native_rms_norm_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
void set_native_rms_norm_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
void set_native_rms_norm_bwd_w_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
/* Not in the reference: "rms_norm_bwd_w_sums_<F>_<B>", the RMSNorm weight gradient written as fp32 column sums (dfb200_rms_norm_bwd_w_sums). */
void set_native_rms_norm_bwd_w_sums_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
/* Not in the reference: "rms_norm_bwd_x_w_<F>_<B>" and "rms_norm_bwd_x_w_sums_<F>_<B>", rms_norm_bwd_x and rms_norm_bwd_w (or its
 * fp32-sums form) in one pass over X and dY (dfb200_rms_norm_bwd_x_w, dfb200_rms_norm_bwd_x_w_sums). */
void set_native_rms_norm_bwd_x_w_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
void set_native_rms_norm_bwd_x_w_sums_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
void set_native_rope_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
void set_native_rope_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype bwd_datatype);
void set_native_copy_to_seq_context_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
void set_native_swiglu_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
void set_native_swiglu_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
void set_native_softmax_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);
void set_native_cross_entropy_loss_skeleton(Op_Skeleton * skeleton, DataflowDatatype bwd_datatype);
/* The reference declares the select_experts kernels (src/ops/nvidia/include/nvidia_ops.h:110-114) but gives them no skeleton;
 * this one is "select_experts_<DT>": total_tokens, n_experts, top_k, X_routed, weights, chosen (uint16), counts, cumsum, num_routed. */
void set_native_select_experts_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
/* The reference's softmax_fp16_fp32 / softmax_bf16_fp32 kernels (fp32 probabilities + arg-max; src/ops/nvidia/loss/softmax.cu:965-1249)
 * have no skeleton either; this one is "softmax_argmax_<F>_FP32": n_rows, n_cols, X, out (fp32), arg_maxs (uint32). */
void set_native_softmax_argmax_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype);
/* Not in the reference: the FP8-weight SwiGLU FFN, forward ("swiglu_ffn_fp8_BF16") and input gradient ("swiglu_ffn_fp8_bwd_BF16").
 * Activations bf16, weights e4m3 codes (DATAFLOW_FP8E4M3) with fp32 per-output-channel scales; argument lists as submit_swiglu_ffn_fp8*. */
void set_native_swiglu_ffn_fp8_skeleton(Op_Skeleton * skeleton);
void set_native_swiglu_ffn_fp8_bwd_skeleton(Op_Skeleton * skeleton);
/* External ops (src/set_ops/include/set_external_op_skeletons.h:10-16): identities of the cuBLASLt matmul and FlashAttention-3 plug-ins. */
void set_external_matmul_skeleton(Op_Skeleton * skeleton);
void set_external_flash3_attention_fwd_skeleton(Op_Skeleton * skeleton);
void set_external_flash3_attention_bwd_skeleton(Op_Skeleton * skeleton);
/* Not in the reference: the fused softmax + cross-entropy op ("softmax_cross_entropy_<F>_<B>"). */
void set_native_softmax_cross_entropy_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd_datatype, DataflowDatatype bwd_datatype);

/* ---- op submission -------------------------------------------------------------------- */
int submit_embedding(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                     int num_tokens, int embed_dim, uint32_t * token_ids, void * embedding_table, void * output);
int submit_copy_to_seq_context(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                               uint64_t N, int total_tokens, int kv_dim,
                               void * X_k, void * X_v, int * seq_positions, uint64_t * seq_context_ptrs, int * seq_context_sizes);
/* No reference wrapper exists for the router; argument order is the kernel's (src/ops/nvidia/include/nvidia_ops.h:110). */
int submit_select_experts(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                          int total_tokens, int n_experts, int top_k_experts, void * X_routed, void * token_expert_weights,
                          uint16_t * chosen_experts, int * expert_counts, int * expert_counts_cumsum, int * num_routed_by_expert);
int submit_rms_norm(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                    int n_rows, int n_cols, float eps,
                    void * rms_weight, void * X, void * out, float * weighted_sums, float * rms_vals);
int submit_rms_norm_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                          int n_rows, int n_cols, float eps,
                          float * fwd_weighted_sums, float * fwd_rms_vals,
                          void * rms_weight, void * X_inp, void * upstream_dX, void * dX);
int submit_rms_norm_bwd_w(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                          int n_rows, int n_cols, float eps,
                          float * fwd_rms_vals, void * X_inp, void * upstream_dX, void * dW);
/* Not in the reference: column_sums[c] = sum over the rows of dY * X * rms, fp32, overwritten (a slot of a packed exchange buffer). */
int submit_rms_norm_bwd_w_sums(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                               int n_rows, int n_cols, float eps,
                               float * fwd_rms_vals, void * X_inp, void * upstream_dX, float * column_sums);
/* Not in the reference (it submits rms_norm_bwd_x, then rms_norm_bwd_w, each reading X and dY): both gradients of the norm in one
 * pass. dX gets what submit_rms_norm_bwd_x gives, bit for bit; dW what submit_rms_norm_bwd_w gives up to the order of the fp32
 * additions over the rows; the _sums form writes the fp32 column sums like submit_rms_norm_bwd_w_sums. */
int submit_rms_norm_bwd_x_w(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                            int n_rows, int n_cols, float eps,
                            float * fwd_weighted_sums, float * fwd_rms_vals,
                            void * rms_weight, void * X_inp, void * upstream_dX, void * dX, void * dW);
int submit_rms_norm_bwd_x_w_sums(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                                 int n_rows, int n_cols, float eps,
                                 float * fwd_weighted_sums, float * fwd_rms_vals,
                                 void * rms_weight, void * X_inp, void * upstream_dX, void * dX, float * column_sums);
int submit_rope(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                int * seq_positions, void * X_q, void * X_k);
int submit_rope_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype bwd_dt,
                      uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                      int * seq_positions, void * dX_q, void * dX_k);
int submit_swiglu(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                  int num_rows, int num_cols, void * x_w1, void * x_w3, void * out);
int submit_swiglu_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                        int num_rows, int num_cols,
                        void * x_w1, void * x_w3, void * upstream_dX, void * dX_w1, void * dX_w3);
int submit_softmax(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                   int n_rows, int n_cols, void * X, void * out);
int submit_cross_entropy_loss(Dataflow_Handle * handle, int stream_id, DataflowDatatype bwd_dt,
                              int n_rows, int n_cols, void * pred_logits, uint32_t * labels);
int submit_softmax_argmax(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt,
                          int n_rows, int n_cols, void * X, float * out, uint32_t * arg_maxs);
/* Not in the reference: one pass producing dlogits = softmax - onehot, per-row losses and
 * {loss sum, valid-row count} (row_loss and loss_sum are optional device pointers). */
int submit_softmax_cross_entropy(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                                 int n_rows, int n_cols, void * logits, uint32_t * labels, void * dlogits,
                                 float * row_loss, float * loss_sum);

/* Not in the reference: out = down(silu(gate(A)) * up(A)) + residual with e4m3 weights (include/dataflow_b200_kernels.h,
 * dfb200_swiglu_ffn_fp8). residual, gate_save and up_save may be NULL (gate_save and up_save together); the op keeps its own
 * device workspace. The backward op needs the transposed codes made by dfb200_ffn_fp8_prepare_bwd_weights. */
int submit_swiglu_ffn_fp8(Dataflow_Handle * handle, int stream_id, int num_tokens, int model_dim, int ffn_dim,
                          void * A, void * Wgate, float * gate_scales, void * Wup, float * up_scales, void * Wdown, float * down_scales,
                          void * residual, void * out, void * gate_save, void * up_save);
int submit_swiglu_ffn_fp8_bwd(Dataflow_Handle * handle, int stream_id, int num_tokens, int model_dim, int ffn_dim,
                              void * dOut, void * gate_saved, void * up_saved, void * WdownT, float * down_scales,
                              void * WgateupT, float * gateup_scales, void * dA);

/* External ops (src/dataflow_ops/include/dataflow_ops.h:69-76, 112-120, 130-140). The op itself comes from a plug-in that the user
 * registers on the handle (register_external_code); these wrappers only build the Op and submit it. submit_matmul: with A, C, D
 * row-major and B column-major, D = alpha * A B + beta * C. Return 0 on success, -1 if the op is not registered or fails. */
int submit_matmul(Dataflow_Handle * handle, int stream_id, DataflowDatatype a_dt, DataflowDatatype b_dt, DataflowDatatype c_dt,
                  DataflowDatatype d_dt, DataflowDatatype compute_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                  float alpha, float beta, void * A, void * B, void * C, void * D, uint64_t workspaceBytes, void * workspace);
int submit_attention(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int num_seqs, int total_q, int total_k,
                     int * q_seq_offsets, int * q_seq_lens, int max_seqlen_q, int * k_seq_offsets, int * k_seq_lens, int max_seqlen_k,
                     int num_q_heads, int num_kv_heads, int head_dim, void * x_q, void * x_k, void * x_v, void * x_attn_out,
                     void * softmax_lse, uint64_t workspaceBytes, void * workspace);
int submit_attention_bwd(Dataflow_Handle * handle, int stream_id, DataflowDatatype bwd_dt, int num_seqs, int total_q, int total_k,
                         int * q_seq_offsets, int * q_seq_lens, int max_seqlen_q, int * k_seq_offsets, int * k_seq_lens, int max_seqlen_k,
                         int num_q_heads, int num_kv_heads, int head_dim, void * x_q, void * x_k, void * x_v, void * x_attn_out,
                         void * softmax_lse, void * dx_out, void * dx_q, void * dx_k, void * dx_v, uint64_t workspaceBytes,
                         void * workspace);

#ifdef __cplusplus
}
#endif
#endif
