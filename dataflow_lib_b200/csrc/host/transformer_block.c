/*
 * submit_transformer_block, submit_transformer_block_bwd_x, submit_transformer_block_bwd_w: one block of the reference's transformer
 * as chains of op submissions on one compute stream (als244/dataflow_lib
 * src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:6-298, 521-851, 853-1003). The order of the steps is the
 * reference's; the places where its text cannot be what was meant are listed in include/dataflow_transformer.h.
 *
 * Matrices are row-major here; the matmul plug-in (cuBLASLt conventions) sees each as the column-major transpose. With a weight
 * W [out, in] row-major (= in x out column-major), activations x [T, in] (= in x T) and y [T, out] (= out x T):
 *   forward   y(out x T)   = W^T(out x in) . x(in x T) [+ c]     -> to_trans_a = 1, M = out, K = in, N = T, A = W, B = x
 *   dgrad     dx(in x T)   = W(in x out) . dy(out x T) [+ c]     -> no transposes,  M = in,  K = out, N = T, A = W, B = dy
 *   wgrad     dW(in x out) += x(in x T) . dy^T(T x out)          -> to_trans_b = 1, M = in,  K = T,  N = out, A = x, B = dy, C = D = dW
 */
#include "dataflow_transformer.h"

#define STEP(call, what) do { const int rc_ = (call); if (rc_) { fprintf(stderr, "Error: transformer block: %s failed\n", what); return rc_; } } while (0)

/* y = x W^T (+ c when given) */
static int project(Dataflow_Handle * h, int stream, DataflowDatatype dt, DataflowDatatype compute_dt, int out_f, int in_f, int tokens,
                   void * W, void * x, void * c, void * y, Seq_Batch_Activation_Workspace * ws) {
	return submit_matmul(h, stream, dt, dt, c ? dt : DATAFLOW_NONE, dt, compute_dt, 1, 0, out_f, in_f, tokens, 1.0f, c ? 1.0f : 0.0f,
	                     W, x, c, y, ws->kernel_workspaceBytes, ws->kernel_workspace);
}

/* dx = dy W, or dx += dy W when accumulate */
static int project_bwd_x(Dataflow_Handle * h, int stream, DataflowDatatype dt, DataflowDatatype compute_dt, int out_f, int in_f, int tokens,
                         void * W, void * dy, void * dx, int accumulate, Seq_Batch_Activation_Workspace * ws) {
	return submit_matmul(h, stream, dt, dt, accumulate ? dt : DATAFLOW_NONE, dt, compute_dt, 0, 0, in_f, out_f, tokens, 1.0f,
	                     accumulate ? 1.0f : 0.0f, W, dy, accumulate ? dx : NULL, dx, ws->kernel_workspaceBytes, ws->kernel_workspace);
}

/* dW += dy^T x */
static int project_bwd_w(Dataflow_Handle * h, int stream, DataflowDatatype dt, DataflowDatatype compute_dt, int out_f, int in_f, int tokens,
                         void * x, void * dy, void * dW, Seq_Batch_Activation_Workspace * ws) {
	return submit_matmul(h, stream, dt, dt, dt, dt, compute_dt, 0, 1, in_f, tokens, out_f, 1.0f, 1.0f, x, dy, dW, dW,
	                     ws->kernel_workspaceBytes, ws->kernel_workspace);
}

/* dst = src on copy_stream, after everything submitted to compute_stream so far */
static int copy_after(Dataflow_Handle * h, int compute_stream, int copy_stream, void * dst, void * src, uint64_t bytes) {
	if (copy_stream != compute_stream) {
		void * state = h->get_stream_state(h, compute_stream);
		if (!state) { fprintf(stderr, "Error: transformer block: no stream state for stream %d\n", compute_stream); return -1; }
		const int rc = h->submit_dependency(h, copy_stream, state);
		if (rc) { fprintf(stderr, "Error: transformer block: dependency of the copy stream on the compute stream failed\n"); return rc; }
	}
	return h->submit_peer_transfer(h, copy_stream, dst, src, bytes);
}

static int containers_ok(const Transformer_Block_Activations * a) {
	return a && a->batch_config && a->saved_activations && a->context && a->activation_workspace &&
	       a->saved_activations->x_1 && a->saved_activations->x_2 && a->saved_activations->x_3;
}

int submit_transformer_block(Dataflow_Handle * dataflow_handle, int compute_stream_id, int out_copy_stream_id,
                             Transformer_Block_Transition * block_input, Transformer_Block * transformer_block,
                             Transformer_Block_Activations * activations, Transformer_Block_Transition * block_output) {
	if (!dataflow_handle || !block_input || !transformer_block || !containers_ok(activations) || !transformer_block->w_1 ||
	    !transformer_block->w_2 || !transformer_block->w_3) {
		fprintf(stderr, "Error: transformer block: NULL argument or incomplete activation containers\n");
		return -1;
	}
	Dataflow_Handle * h = dataflow_handle;
	const Transformer_Block_Config * cfg = &transformer_block->config;
	const Transformer_Block * w = transformer_block;
	const Seq_Batch_Config * bc = activations->batch_config;
	Seq_Batch_Saved_Activations * sv = activations->saved_activations;
	Seq_Batch_Activation_Workspace * ws = activations->activation_workspace;
	Seq_Batch_Context * ctx = activations->context;
	const DataflowDatatype dt = cfg->block_dt, cdt = cfg->compute_dt;
	const int T = bc->total_q, d = cfg->model_dim, kv = cfg->kv_dim, f = cfg->ffn_dim, s = compute_stream_id;

	STEP(submit_rms_norm(h, s, dt, T, d, cfg->eps, w->w_attn_norm, block_input->X, ws->x_temp,
	                     (float *) sv->attn_norm_weighted_sums, (float *) sv->attn_norm_rms_vals), "attention RMSNorm");
	STEP(project(h, s, dt, cdt, d, d, T, w->w_q, ws->x_temp, NULL, sv->x_q, ws), "Q projection");
	STEP(project(h, s, dt, cdt, kv, d, T, w->w_k, ws->x_temp, NULL, sv->x_k_local, ws), "K projection");
	STEP(project(h, s, dt, cdt, kv, d, T, w->w_v, ws->x_temp, NULL, sv->x_v_local, ws), "V projection");
	STEP(submit_rope(h, s, dt, (uint64_t) T * (uint64_t) d, d, cfg->head_dim, cfg->num_kv_heads, cfg->theta, bc->seq_positions,
	                 sv->x_q, sv->x_k_local), "RoPE");
	STEP(h->set_mem(h, s, ws->kernel_workspace, 0, ws->kernel_workspaceBytes), "zeroing the attention workspace");
	STEP(submit_attention(h, s, dt, bc->num_seqs, T, bc->total_k, bc->q_seq_offsets, bc->q_seq_lens, bc->max_seqlen_q,
	                      bc->k_seq_offsets, bc->k_seq_lens, bc->max_seqlen_k, cfg->num_q_heads, cfg->num_kv_heads, cfg->head_dim,
	                      sv->x_q, ctx->x_k, ctx->x_v, sv->x_attn_out, sv->softmax_lse, ws->kernel_workspaceBytes, ws->kernel_workspace),
	     "attention");
	STEP(project(h, s, dt, cdt, d, d, T, w->w_o, sv->x_attn_out, block_input->X, sv->x_o, ws), "attention output projection + residual");
	STEP(submit_rms_norm(h, s, dt, T, d, cfg->eps, w->w_ffn_norm, sv->x_o, ws->x_temp,
	                     (float *) sv->ffn_norm_weighted_sums, (float *) sv->ffn_norm_rms_vals), "FFN RMSNorm");
	STEP(project(h, s, dt, cdt, f, d, T, w->w_1[0], ws->x_temp, NULL, sv->x_1[0], ws), "FFN w1 projection");
	STEP(project(h, s, dt, cdt, f, d, T, w->w_3[0], ws->x_temp, NULL, sv->x_3[0], ws), "FFN w3 projection");
	STEP(submit_swiglu(h, s, dt, T, f, sv->x_1[0], sv->x_3[0], ws->x_temp_mlp), "SwiGLU");
	STEP(project(h, s, dt, cdt, d, f, T, w->w_2[0], ws->x_temp_mlp, sv->x_o, sv->x_2[0], ws), "FFN w2 projection + residual");
	if (block_output && block_output->X)
		STEP(copy_after(h, s, out_copy_stream_id, block_output->X, sv->x_2[0], (uint64_t) T * (uint64_t) d * dataflow_sizeof_element(dt)),
		     "copy of the block output");
	return 0;
}

int submit_transformer_block_bwd_x(Dataflow_Handle * dataflow_handle, int compute_stream_id, int out_copy_stream_id,
                                   Transformer_Block * transformer_block, Transformer_Block_Transition * inp_grad_stream,
                                   Transformer_Block_Activations * activations, Transformer_Block_Transition * fwd_block_input,
                                   Transformer_Block_Activations * grad_activations, Transformer_Block * grad_weights,
                                   Transformer_Block_Transition * out_grad_stream) {
	if (!dataflow_handle || !transformer_block || !inp_grad_stream || !fwd_block_input || !grad_weights || !containers_ok(activations) ||
	    !containers_ok(grad_activations) || !transformer_block->w_1 || !transformer_block->w_2 || !transformer_block->w_3) {
		fprintf(stderr, "Error: transformer block (input gradients): NULL argument or incomplete activation containers\n");
		return -1;
	}
	Dataflow_Handle * h = dataflow_handle;
	const Transformer_Block_Config * cfg = &transformer_block->config;
	const Transformer_Block * w = transformer_block;
	const Seq_Batch_Config * bc = grad_activations->batch_config;
	Seq_Batch_Saved_Activations * fwd = activations->saved_activations, * bwd = grad_activations->saved_activations;
	Seq_Batch_Context * fwd_ctx = activations->context, * bwd_ctx = grad_activations->context;
	Seq_Batch_Activation_Workspace * ws = grad_activations->activation_workspace;
	const DataflowDatatype dt = cfg->block_dt, cdt = cfg->compute_dt;
	const int T = bc->total_q, d = cfg->model_dim, kv = cfg->kv_dim, f = cfg->ffn_dim, s = compute_stream_id;
	const uint64_t stream_bytes = (uint64_t) T * (uint64_t) d * dataflow_sizeof_element(dt);
	void * dX = inp_grad_stream->X;

	/* FFN half */
	STEP(project_bwd_x(h, s, dt, cdt, d, f, T, w->w_2[0], dX, ws->x_temp_mlp, 0, ws), "w2 input gradient");
	STEP(submit_swiglu_bwd_x(h, s, dt, dt, T, f, fwd->x_1[0], fwd->x_3[0], ws->x_temp_mlp, bwd->x_1[0], bwd->x_3[0]), "SwiGLU gradient");
	STEP(project_bwd_x(h, s, dt, cdt, f, d, T, w->w_1[0], bwd->x_1[0], ws->x_temp, 0, ws), "w1 input gradient");
	STEP(project_bwd_x(h, s, dt, cdt, f, d, T, w->w_3[0], bwd->x_3[0], ws->x_temp, 1, ws), "w3 input gradient");
	STEP(submit_rms_norm_bwd_x(h, s, dt, dt, T, d, cfg->eps, (float *) fwd->ffn_norm_weighted_sums, (float *) fwd->ffn_norm_rms_vals,
	                           w->w_ffn_norm, fwd->x_o, ws->x_temp, dX), "FFN RMSNorm input gradient");
	STEP(submit_rms_norm_bwd_w(h, s, dt, dt, T, d, cfg->eps, (float *) fwd->ffn_norm_rms_vals, fwd->x_o, ws->x_temp,
	                           grad_weights->w_ffn_norm), "FFN RMSNorm weight gradient");
	/* the stream gradient now is d(x_o): kept for the W_o weight gradient, read by the W_o input gradient */
	STEP(h->submit_peer_transfer(h, s, bwd->x_o, dX, stream_bytes), "keeping d(x_o)");

	/* attention half */
	STEP(project_bwd_x(h, s, dt, cdt, d, d, T, w->w_o, bwd->x_o, ws->x_temp, 0, ws), "attention output projection input gradient");
	STEP(h->set_mem(h, s, ws->kernel_workspace, 0, ws->kernel_workspaceBytes), "zeroing the attention workspace");
	STEP(submit_attention_bwd(h, s, dt, bc->num_seqs, T, bc->total_k, bc->q_seq_offsets, bc->q_seq_lens, bc->max_seqlen_q,
	                          bc->k_seq_offsets, bc->k_seq_lens, bc->max_seqlen_k, cfg->num_q_heads, cfg->num_kv_heads, cfg->head_dim,
	                          fwd->x_q, fwd_ctx->x_k, fwd_ctx->x_v, fwd->x_attn_out, fwd->softmax_lse, ws->x_temp,
	                          bwd->x_q, bwd_ctx->x_k, bwd_ctx->x_v, ws->kernel_workspaceBytes, ws->kernel_workspace), "attention gradient");
	STEP(submit_rope_bwd_x(h, s, dt, (uint64_t) T * (uint64_t) d, d, cfg->head_dim, cfg->num_kv_heads, cfg->theta, bc->seq_positions,
	                       bwd->x_q, bwd->x_k_local), "RoPE gradient");
	STEP(project_bwd_x(h, s, dt, cdt, d, d, T, w->w_q, bwd->x_q, ws->x_temp, 0, ws), "Q projection input gradient");
	STEP(project_bwd_x(h, s, dt, cdt, kv, d, T, w->w_k, bwd->x_k_local, ws->x_temp, 1, ws), "K projection input gradient");
	STEP(project_bwd_x(h, s, dt, cdt, kv, d, T, w->w_v, bwd->x_v_local, ws->x_temp, 1, ws), "V projection input gradient");
	STEP(submit_rms_norm_bwd_x(h, s, dt, dt, T, d, cfg->eps, (float *) fwd->attn_norm_weighted_sums, (float *) fwd->attn_norm_rms_vals,
	                           w->w_attn_norm, fwd_block_input->X, ws->x_temp, dX), "attention RMSNorm input gradient");
	STEP(submit_rms_norm_bwd_w(h, s, dt, dt, T, d, cfg->eps, (float *) fwd->attn_norm_rms_vals, fwd_block_input->X, ws->x_temp,
	                           grad_weights->w_attn_norm), "attention RMSNorm weight gradient");

	/* while the block's weights are at hand: the two RMSNorm outputs again, for the weight-gradient chain */
	STEP(submit_rms_norm(h, s, dt, T, d, cfg->eps, w->w_attn_norm, fwd_block_input->X, ws->recomputed_attn_norm, NULL, NULL),
	     "recomputing the attention RMSNorm");
	STEP(submit_rms_norm(h, s, dt, T, d, cfg->eps, w->w_ffn_norm, fwd->x_o, ws->recomputed_ffn_norm, NULL, NULL),
	     "recomputing the FFN RMSNorm");
	if (out_grad_stream && out_grad_stream->X)
		STEP(copy_after(h, s, out_copy_stream_id, out_grad_stream->X, dX, stream_bytes), "copy of the block's input gradient");
	return 0;
}

int submit_transformer_block_bwd_w(Dataflow_Handle * dataflow_handle, int compute_stream_id,
                                   Transformer_Block_Transition * grad_stream, Transformer_Block_Activations * activations,
                                   Transformer_Block_Activations * grad_activations, Transformer_Block * grad_weights) {
	if (!dataflow_handle || !grad_stream || !grad_weights || !containers_ok(activations) || !containers_ok(grad_activations) ||
	    !grad_weights->w_1 || !grad_weights->w_2 || !grad_weights->w_3) {
		fprintf(stderr, "Error: transformer block (weight gradients): NULL argument or incomplete activation containers\n");
		return -1;
	}
	Dataflow_Handle * h = dataflow_handle;
	const Transformer_Block_Config * cfg = &grad_weights->config;
	Transformer_Block * gw = grad_weights;
	const Seq_Batch_Config * bc = activations->batch_config;
	Seq_Batch_Saved_Activations * fwd = activations->saved_activations, * bwd = grad_activations->saved_activations;
	Seq_Batch_Activation_Workspace * ws = grad_activations->activation_workspace;
	const DataflowDatatype dt = cfg->block_dt, cdt = cfg->compute_dt;
	const int T = bc->total_q, d = cfg->model_dim, kv = cfg->kv_dim, f = cfg->ffn_dim, s = compute_stream_id;

	STEP(submit_swiglu(h, s, dt, T, f, fwd->x_1[0], fwd->x_3[0], ws->x_temp_mlp), "recomputing SwiGLU");
	STEP(project_bwd_w(h, s, dt, cdt, d, f, T, ws->x_temp_mlp, grad_stream->X, gw->w_2[0], ws), "w2 weight gradient");
	STEP(project_bwd_w(h, s, dt, cdt, f, d, T, ws->recomputed_ffn_norm, bwd->x_1[0], gw->w_1[0], ws), "w1 weight gradient");
	STEP(project_bwd_w(h, s, dt, cdt, f, d, T, ws->recomputed_ffn_norm, bwd->x_3[0], gw->w_3[0], ws), "w3 weight gradient");
	STEP(project_bwd_w(h, s, dt, cdt, d, d, T, fwd->x_attn_out, bwd->x_o, gw->w_o, ws), "attention output projection weight gradient");
	STEP(project_bwd_w(h, s, dt, cdt, kv, d, T, ws->recomputed_attn_norm, bwd->x_v_local, gw->w_v, ws), "V projection weight gradient");
	STEP(project_bwd_w(h, s, dt, cdt, kv, d, T, ws->recomputed_attn_norm, bwd->x_k_local, gw->w_k, ws), "K projection weight gradient");
	STEP(project_bwd_w(h, s, dt, cdt, d, d, T, ws->recomputed_attn_norm, bwd->x_q, gw->w_q, ws), "Q projection weight gradient");
	return 0;
}
