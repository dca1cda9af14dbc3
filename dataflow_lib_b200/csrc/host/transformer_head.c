/*
 * submit_transformer_head: the reference's model head as a chain of op submissions on one compute stream
 * (als244/dataflow_lib src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:300-492). The order of the steps is the
 * reference's; the places where its text cannot be what was meant are listed in include/dataflow_transformer.h.
 *
 * Matrices are row-major here; the matmul plug-in (cuBLASLt conventions) sees each as the column-major transpose:
 *   w_head   [V, d] row-major = d x V column-major        head_norm_out [T, d] = d x T        logits [T, V] = V x T
 *   forward   logits(V x T)  = w_head^T (V x d) . hn (d x T)              -> to_trans_a = 1, M = V, K = d, N = T
 *   dgrad     dhn(d x T)     = w_head (d x V) . dlogits (V x T)           -> no transposes,  M = d, K = V, N = T
 *   wgrad     dW(d x V)     += hn (d x T) . dlogits^T (T x V)             -> to_trans_b = 1, M = d, K = T, N = V, beta = 1
 */
#include "dataflow_transformer.h"

#define STEP(call, what) do { const int rc_ = (call); if (rc_) { fprintf(stderr, "Error: transformer head: %s failed\n", what); return rc_; } } while (0)

int submit_transformer_head(Dataflow_Handle * dataflow_handle, int compute_stream_id, int out_copy_stream_id,
                            Transformer_Block_Transition * block_input, Transformer_Head * transformer_head,
                            Transformer_Head_Activations * head_activations, Transformer_Model_Output * model_output,
                            Transformer_Head * grad_transformer_head, Transformer_Head_Activations * grad_head_activations,
                            Transformer_Block_Transition * grad_stream, Transformer_Block_Transition * next_grad_stream) {
	if (!dataflow_handle || !block_input || !transformer_head || !head_activations || !model_output) {
		fprintf(stderr, "Error: transformer head: NULL argument\n");
		return -1;
	}
	if (grad_transformer_head && (!grad_head_activations || !grad_stream)) {
		fprintf(stderr, "Error: transformer head: a backward pass needs grad_head_activations and grad_stream\n");
		return -1;
	}
	Dataflow_Handle * h = dataflow_handle;
	const Transformer_Head * head = transformer_head;
	Transformer_Head_Activations * act = head_activations;
	const int V = head->embedding_config.vocab_size, d = head->embedding_config.embedding_size, T = act->num_tokens;
	const DataflowDatatype fwd = head->fwd_dt, bwd = head->bwd_dt;

	STEP(submit_rms_norm(h, compute_stream_id, fwd, T, d, head->eps, head->w_head_norm, block_input->X, act->head_norm_out,
	                     (float *) act->head_norm_weighted_sums, (float *) act->head_norm_rms_vals), "final RMSNorm");
	STEP(submit_matmul(h, compute_stream_id, fwd, fwd, DATAFLOW_NONE, fwd, head->compute_dt, 1, 0, V, d, T, 1.0f, 0.0f,
	                   head->w_head, act->head_norm_out, NULL, act->head_out, act->kernel_workspaceBytes, act->kernel_workspace),
	     "vocabulary projection");

	if (!grad_transformer_head) {
		STEP(submit_softmax(h, compute_stream_id, fwd, bwd, T, V, act->head_out, model_output->logits), "softmax");
		return 0;
	}

	/* backward: softmax and the cross-entropy step in one pass over the logits */
	Transformer_Head * gw = grad_transformer_head;
	Transformer_Head_Activations * gact = grad_head_activations;
	STEP(submit_softmax_cross_entropy(h, compute_stream_id, fwd, bwd, T, V, act->head_out, model_output->labels, model_output->logits,
	                                  (float *) model_output->loss, NULL), "softmax + cross entropy");
	STEP(submit_matmul(h, compute_stream_id, bwd, bwd, DATAFLOW_NONE, bwd, head->compute_dt, 0, 0, d, V, T, 1.0f, 0.0f,
	                   head->w_head, model_output->logits, NULL, gact->head_norm_out, gact->kernel_workspaceBytes, gact->kernel_workspace),
	     "projection input gradient");
	STEP(submit_matmul(h, compute_stream_id, bwd, bwd, bwd, bwd, head->compute_dt, 0, 1, d, T, V, 1.0f, 1.0f,
	                   act->head_norm_out, model_output->logits, gw->w_head, gw->w_head, gact->kernel_workspaceBytes, gact->kernel_workspace),
	     "projection weight gradient");
	STEP(submit_rms_norm_bwd_x(h, compute_stream_id, fwd, bwd, T, d, head->eps, (float *) act->head_norm_weighted_sums,
	                           (float *) act->head_norm_rms_vals, head->w_head_norm, block_input->X, gact->head_norm_out, grad_stream->X),
	     "RMSNorm input gradient");
	STEP(submit_rms_norm_bwd_w(h, compute_stream_id, fwd, bwd, T, d, head->eps, (float *) act->head_norm_rms_vals, block_input->X,
	                           gact->head_norm_out, gw->w_head_norm), "RMSNorm weight gradient");

	if (next_grad_stream) {
		/* the copy runs on its own stream, after everything submitted to the compute stream so far */
		void * state = h->get_stream_state(h, compute_stream_id);
		if (!state) { fprintf(stderr, "Error: transformer head: no stream state for stream %d\n", compute_stream_id); return -1; }
		STEP(h->submit_dependency(h, out_copy_stream_id, state), "dependency of the copy stream on the compute stream");
		const uint64_t bytes = (uint64_t) T * (uint64_t) d * dataflow_sizeof_element(bwd);
		STEP(h->submit_peer_transfer(h, out_copy_stream_id, next_grad_stream->X, grad_stream->X, bytes), "copy of the head gradient");
	}
	return 0;
}
