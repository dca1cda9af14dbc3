/*
 * submit_* wrappers: build an Op on the stack (skeleton + pointers to the argument values)
 * and hand it to handle->submit_op. Argument order per op is the one fixed by
 * als244/dataflow_lib (src/dataflow_ops/src/norm_ops.c:17-24,52-60,85-91, attn_misc_ops.c:17-24,
 * mlp_misc_ops.c:15-19,46-52, loss_misc_ops.c:19-22,47-50), because plug-ins index op_args by
 * position. Every wrapper returns 0 on success and -1 on failure.
 */
#include "dataflow_api.h"

static int submit(Dataflow_Handle * handle, Op * op, int stream_id, const char * what) {
	if (!handle || !handle->submit_op) { fprintf(stderr, "Error: %s submitted to an uninitialised handle\n", what); return -1; }
	if (handle->submit_op(handle, op, stream_id)) { fprintf(stderr, "Error: failed to submit %s op...\n", what); return -1; }
	return 0;
}

/* ARGS(op, a, b, ...) stores &a, &b, ... into op.op_args in order. */
#define ARGS(op, ...) do { void * args_[] = {__VA_ARGS__}; for (unsigned i_ = 0; i_ < sizeof(args_) / sizeof(args_[0]); i_++) (op).op_args[i_] = args_[i_]; } while (0)

int submit_rms_norm(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int n_rows, int n_cols, float eps,
                    void * rms_weight, void * X, void * out, float * weighted_sums, float * rms_vals) {
	Op op;
	set_native_rms_norm_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &n_rows, &n_cols, &eps, &rms_weight, &X, &out, &weighted_sums, &rms_vals);
	return submit(handle, &op, stream_id, "rms norm");
}

int submit_rms_norm_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                          int n_rows, int n_cols, float eps, float * fwd_weighted_sums, float * fwd_rms_vals,
                          void * rms_weight, void * X_inp, void * upstream_dX, void * dX) {
	Op op;
	set_native_rms_norm_bwd_x_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &eps, &fwd_weighted_sums, &fwd_rms_vals, &rms_weight, &X_inp, &upstream_dX, &dX);
	return submit(handle, &op, stream_id, "rms norm bwd x");
}

int submit_rms_norm_bwd_w(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                          int n_rows, int n_cols, float eps, float * fwd_rms_vals, void * X_inp, void * upstream_dX, void * dW) {
	Op op;
	set_native_rms_norm_bwd_w_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &eps, &fwd_rms_vals, &X_inp, &upstream_dX, &dW);
	return submit(handle, &op, stream_id, "rms norm bwd w");
}

int submit_rms_norm_bwd_w_sums(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                               int n_rows, int n_cols, float eps, float * fwd_rms_vals, void * X_inp, void * upstream_dX, float * column_sums) {
	Op op;
	set_native_rms_norm_bwd_w_sums_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &eps, &fwd_rms_vals, &X_inp, &upstream_dX, &column_sums);
	return submit(handle, &op, stream_id, "rms norm bwd w (fp32 column sums)");
}

int submit_rms_norm_bwd_x_w(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                            int n_rows, int n_cols, float eps, float * fwd_weighted_sums, float * fwd_rms_vals,
                            void * rms_weight, void * X_inp, void * upstream_dX, void * dX, void * dW) {
	Op op;
	set_native_rms_norm_bwd_x_w_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &eps, &fwd_weighted_sums, &fwd_rms_vals, &rms_weight, &X_inp, &upstream_dX, &dX, &dW);
	return submit(handle, &op, stream_id, "rms norm bwd x and w");
}

int submit_rms_norm_bwd_x_w_sums(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                                 int n_rows, int n_cols, float eps, float * fwd_weighted_sums, float * fwd_rms_vals,
                                 void * rms_weight, void * X_inp, void * upstream_dX, void * dX, float * column_sums) {
	Op op;
	set_native_rms_norm_bwd_x_w_sums_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &eps, &fwd_weighted_sums, &fwd_rms_vals, &rms_weight, &X_inp, &upstream_dX, &dX, &column_sums);
	return submit(handle, &op, stream_id, "rms norm bwd x and w (fp32 column sums)");
}

int submit_rope(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, uint64_t N, int model_dim, int head_dim,
                int num_kv_heads, int theta, int * seq_positions, void * X_q, void * X_k) {
	Op op;
	set_native_rope_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &N, &model_dim, &head_dim, &num_kv_heads, &theta, &seq_positions, &X_q, &X_k);
	return submit(handle, &op, stream_id, "rope");
}

int submit_rope_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype bwd_dt, uint64_t N, int model_dim, int head_dim,
                      int num_kv_heads, int theta, int * seq_positions, void * dX_q, void * dX_k) {
	Op op;
	set_native_rope_bwd_x_skeleton(&op.op_skeleton, bwd_dt);
	ARGS(op, &N, &model_dim, &head_dim, &num_kv_heads, &theta, &seq_positions, &dX_q, &dX_k);
	return submit(handle, &op, stream_id, "rope bwd x");
}

int submit_swiglu(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int num_rows, int num_cols,
                  void * x_w1, void * x_w3, void * out) {
	Op op;
	set_native_swiglu_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &num_rows, &num_cols, &x_w1, &x_w3, &out);
	return submit(handle, &op, stream_id, "swiglu");
}

int submit_swiglu_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                        int num_rows, int num_cols, void * x_w1, void * x_w3, void * upstream_dX, void * dX_w1, void * dX_w3) {
	Op op;
	set_native_swiglu_bwd_x_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &num_rows, &num_cols, &x_w1, &x_w3, &upstream_dX, &dX_w1, &dX_w3);
	return submit(handle, &op, stream_id, "swiglu bwd x");
}

int submit_softmax(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                   int n_rows, int n_cols, void * X, void * out) {
	Op op;
	set_native_softmax_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &X, &out);
	return submit(handle, &op, stream_id, "softmax");
}

int submit_cross_entropy_loss(Dataflow_Handle * handle, int stream_id, DataflowDatatype bwd_dt, int n_rows, int n_cols,
                              void * pred_logits, uint32_t * labels) {
	Op op;
	set_native_cross_entropy_loss_skeleton(&op.op_skeleton, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &pred_logits, &labels);
	return submit(handle, &op, stream_id, "cross entropy loss");
}

int submit_softmax_cross_entropy(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt,
                                 int n_rows, int n_cols, void * logits, uint32_t * labels, void * dlogits,
                                 float * row_loss, float * loss_sum) {
	Op op;
	set_native_softmax_cross_entropy_skeleton(&op.op_skeleton, fwd_dt, bwd_dt);
	ARGS(op, &n_rows, &n_cols, &logits, &labels, &dlogits, &row_loss, &loss_sum);
	return submit(handle, &op, stream_id, "softmax cross entropy");
}

/* src/dataflow_ops/src/preprocess_ops.c:3-34 */
int submit_embedding(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int num_tokens, int embed_dim,
                     uint32_t * token_ids, void * embedding_table, void * output) {
	Op op;
	set_native_embedding_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &num_tokens, &embed_dim, &token_ids, &embedding_table, &output);
	return submit(handle, &op, stream_id, "embedding");
}

/* src/dataflow_ops/src/attn_misc_ops.c:69-101 */
int submit_copy_to_seq_context(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, uint64_t N, int total_tokens, int kv_dim,
                               void * X_k, void * X_v, int * seq_positions, uint64_t * seq_context_ptrs, int * seq_context_sizes) {
	Op op;
	set_native_copy_to_seq_context_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &N, &total_tokens, &kv_dim, &X_k, &X_v, &seq_positions, &seq_context_ptrs, &seq_context_sizes);
	return submit(handle, &op, stream_id, "copy to seq context");
}

int submit_select_experts(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int total_tokens, int n_experts, int top_k_experts,
                          void * X_routed, void * token_expert_weights, uint16_t * chosen_experts, int * expert_counts,
                          int * expert_counts_cumsum, int * num_routed_by_expert) {
	Op op;
	set_native_select_experts_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &total_tokens, &n_experts, &top_k_experts, &X_routed, &token_expert_weights, &chosen_experts, &expert_counts, &expert_counts_cumsum,
	     &num_routed_by_expert);
	return submit(handle, &op, stream_id, "select experts");
}

int submit_softmax_argmax(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int n_rows, int n_cols, void * X, float * out,
                          uint32_t * arg_maxs) {
	Op op;
	set_native_softmax_argmax_skeleton(&op.op_skeleton, fwd_dt);
	ARGS(op, &n_rows, &n_cols, &X, &out, &arg_maxs);
	return submit(handle, &op, stream_id, "softmax argmax");
}

int submit_swiglu_ffn_fp8(Dataflow_Handle * handle, int stream_id, int num_tokens, int model_dim, int ffn_dim, void * A, void * Wgate,
                          float * gate_scales, void * Wup, float * up_scales, void * Wdown, float * down_scales, void * residual, void * out,
                          void * gate_save, void * up_save) {
	Op op;
	set_native_swiglu_ffn_fp8_skeleton(&op.op_skeleton);
	ARGS(op, &num_tokens, &model_dim, &ffn_dim, &A, &Wgate, &gate_scales, &Wup, &up_scales, &Wdown, &down_scales, &residual, &out, &gate_save, &up_save);
	return submit(handle, &op, stream_id, "swiglu ffn fp8");
}

int submit_swiglu_ffn_fp8_bwd(Dataflow_Handle * handle, int stream_id, int num_tokens, int model_dim, int ffn_dim, void * dOut, void * gate_saved,
                              void * up_saved, void * WdownT, float * down_scales, void * WgateupT, float * gateup_scales, void * dA) {
	Op op;
	set_native_swiglu_ffn_fp8_bwd_skeleton(&op.op_skeleton);
	ARGS(op, &num_tokens, &model_dim, &ffn_dim, &dOut, &gate_saved, &up_saved, &WdownT, &down_scales, &WgateupT, &gateup_scales, &dA);
	return submit(handle, &op, stream_id, "swiglu ffn fp8 bwd");
}

/* ---- external ops (als244/dataflow_lib src/dataflow_ops/src/matmul_op.c:10-66, attention_op.c:36-82, 88-138): the op must have been
 * registered on the handle by the user (register_external_code with the plug-in's shared object); this library only builds the Op.
 * A, C, D row-major and B column-major give D = alpha * A B + beta * C. num_sms = 0 means "all". */
int submit_matmul(Dataflow_Handle * handle, int stream_id, DataflowDatatype a_dt, DataflowDatatype b_dt, DataflowDatatype c_dt,
                  DataflowDatatype d_dt, DataflowDatatype compute_dt, int to_trans_a, int to_trans_b, int M, int K, int N,
                  float alpha, float beta, void * A, void * B, void * C, void * D, uint64_t workspaceBytes, void * workspace) {
	Op op;
	set_external_matmul_skeleton(&op.op_skeleton);
	int num_sms = 0;
	ARGS(op, &num_sms, &a_dt, &b_dt, &c_dt, &d_dt, &compute_dt, &to_trans_a, &to_trans_b, &M, &K, &N, &alpha, &beta, &A, &B, &C, &D,
	     &workspaceBytes, &workspace);
	return submit(handle, &op, stream_id, "matmul");
}

int submit_attention(Dataflow_Handle * handle, int stream_id, DataflowDatatype fwd_dt, int num_seqs, int total_q, int total_k,
                     int * q_seq_offsets, int * q_seq_lens, int max_seqlen_q, int * k_seq_offsets, int * k_seq_lens, int max_seqlen_k,
                     int num_q_heads, int num_kv_heads, int head_dim, void * x_q, void * x_k, void * x_v, void * x_attn_out,
                     void * softmax_lse, uint64_t workspaceBytes, void * workspace) {
	Op op;
	set_external_flash3_attention_fwd_skeleton(&op.op_skeleton);
	ARGS(op, &fwd_dt, &num_seqs, &total_q, &total_k, &q_seq_offsets, &q_seq_lens, &max_seqlen_q, &k_seq_offsets, &k_seq_lens, &max_seqlen_k,
	     &num_q_heads, &num_kv_heads, &head_dim, &x_q, &x_k, &x_v, &x_attn_out, &softmax_lse, &workspaceBytes, &workspace);
	return submit(handle, &op, stream_id, "attention");
}

int submit_attention_bwd(Dataflow_Handle * handle, int stream_id, DataflowDatatype bwd_dt, int num_seqs, int total_q, int total_k,
                         int * q_seq_offsets, int * q_seq_lens, int max_seqlen_q, int * k_seq_offsets, int * k_seq_lens, int max_seqlen_k,
                         int num_q_heads, int num_kv_heads, int head_dim, void * x_q, void * x_k, void * x_v, void * x_attn_out,
                         void * softmax_lse, void * dx_out, void * dx_q, void * dx_k, void * dx_v, uint64_t workspaceBytes, void * workspace) {
	Op op;
	set_external_flash3_attention_bwd_skeleton(&op.op_skeleton);
	ARGS(op, &bwd_dt, &num_seqs, &total_q, &total_k, &q_seq_offsets, &q_seq_lens, &max_seqlen_q, &k_seq_offsets, &k_seq_lens, &max_seqlen_k,
	     &num_q_heads, &num_kv_heads, &head_dim, &x_q, &x_k, &x_v, &x_attn_out, &softmax_lse, &dx_out, &dx_q, &dx_k, &dx_v,
	     &workspaceBytes, &workspace);
	return submit(handle, &op, stream_id, "attention bwd");
}
