/*
 * The head of the reference's transformer as one host call: final RMSNorm -> vocabulary projection -> softmax, and when
 * gradient containers are passed, cross entropy -> projection input gradient -> projection weight gradient -> RMSNorm
 * input and weight gradients (als244/dataflow_lib src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:300-492).
 *
 * Struct names and field orders are the reference's (src/dataflow_models/dataflow_transformer/include/transformer_structs.h:94-150,
 * src/dataflow_models/include/dataflow_models.h:33-39), reduced to the members this call reads: the reference's
 * Seq_Batch_Config pointer is carried as an opaque pointer and never dereferenced.
 *
 * The native ops come from this library; the two projections go through submit_matmul, i.e. through whatever plug-in the
 * user registered under the reference's "matmul" identity (its cuBLASLt helper, unchanged, works).
 */
#ifndef DATAFLOW_TRANSFORMER_H
#define DATAFLOW_TRANSFORMER_H

#include "dataflow_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct embedding_config {
	int vocab_size;
	int embedding_size;          /* = model_dim */
} Embedding_Config;

typedef struct transformer_head {
	DataflowDatatype fwd_dt;
	DataflowDatatype bwd_dt;
	DataflowDatatype compute_dt; /* accumulation type of the projections */
	float eps;
	Embedding_Config embedding_config;
	void * buffer;
	void * w_head_norm;          /* [embedding_size] */
	void * w_head;               /* [vocab_size, embedding_size] row-major = the reference's column-major [embedding_size, vocab_size] */
} Transformer_Head;

typedef struct transformer_head_activations {
	int num_tokens;
	void * buffer;
	void * head_norm_out;            /* [num_tokens, embedding_size]; in the gradient container: d(head_norm_out) */
	void * head_norm_weighted_sums;  /* fp32 [num_tokens] */
	void * head_norm_rms_vals;       /* fp32 [num_tokens] */
	void * head_out;                 /* [num_tokens, vocab_size] logits */
	void * kernel_workspace;         /* handed to the matmul plug-in */
	uint64_t kernel_workspaceBytes;
} Transformer_Head_Activations;

typedef struct transformer_block_transition {
	void * batch_config;             /* Seq_Batch_Config * in the reference; opaque here */
	void * X;                        /* [num_tokens, embedding_size] */
} Transformer_Block_Transition;

typedef struct transformer_model_output {
	void * batch_config;
	uint32_t * token_ids;
	uint32_t * labels;               /* [num_tokens]; a label >= vocab_size marks a row without a target */
	void * logits;                   /* [num_tokens, vocab_size] in bwd_dt: probabilities after the forward part, softmax - onehot after the backward part */
	void * loss;                     /* optional fp32 [num_tokens]: per-row loss, written by the backward part */
	float loss_avg;
} Transformer_Model_Output;

/*
 * Forward only when grad_transformer_head is NULL (model_output->logits then holds the probabilities). Otherwise also the
 * backward pass: grad_transformer_head->w_head and ->w_head_norm ACCUMULATE the weight gradients (the caller zeroes them),
 * grad_head_activations->head_norm_out receives d(head_norm_out), grad_stream->X the gradient with respect to block_input->X
 * (it is accumulated into: zero it first, as for submit_rms_norm_bwd_x), and next_grad_stream->X, if given, a copy of it made on
 * out_copy_stream_id after the compute stream's work (the streams are ordered through the handle's stream-state events).
 *
 * Differences from the reference text, which this follows in intent: the weight-gradient projection reads the gradient of
 * the logits from model_output->logits (the reference passes grad_head_activations->head_out, a buffer nothing has written,
 * dataflow_transformer.c:440) and the RMSNorm weight gradient reads block_input->X (the reference passes the logits,
 * :476); softmax and cross entropy run as this library's fused op when a backward pass is asked for.
 * Returns 0, or the failing op's non-zero code after printing which step failed.
 */
int submit_transformer_head(Dataflow_Handle * dataflow_handle, int compute_stream_id, int out_copy_stream_id,
                            Transformer_Block_Transition * block_input, Transformer_Head * transformer_head,
                            Transformer_Head_Activations * head_activations, Transformer_Model_Output * model_output,
                            Transformer_Head * grad_transformer_head, Transformer_Head_Activations * grad_head_activations,
                            Transformer_Block_Transition * grad_stream, Transformer_Block_Transition * next_grad_stream);

#ifdef __cplusplus
}
#endif
#endif
