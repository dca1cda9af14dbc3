/*
 * The callers of the reference's transformer layer as host calls: a block's forward chain, its input-gradient chain, its
 * weight-gradient chain, and the head (als244/dataflow_lib src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:6-298,
 * 300-492, 521-851, 853-1003; prototypes include/dataflow_transformer.h:43-73).
 *
 * Struct names and field orders are the reference's (src/dataflow_models/dataflow_transformer/include/transformer_structs.h:10-150,
 * seq_batch_structs.h:6-125, src/dataflow_models/include/dataflow_models.h:4-55), with the two things that stop the reference's
 * headers from compiling put right: Seq_Batch_Saved_Activations lists attn_norm_weighted_sums, attn_norm_rms_vals and x_q once
 * (twice in seq_batch_structs.h:57-63), and the prototypes use Transformer_Block_Transition, the type the reference's function
 * DEFINITIONS use (its header names the undeclared Transformer_Block_Input / Transformer_Block_Output, dataflow_transformer.h:44-46).
 *
 * The native ops (RMSNorm, RoPE, SwiGLU and their gradients, softmax, cross entropy) come from this library. Every projection goes
 * through submit_matmul and attention through submit_attention / submit_attention_bwd, i.e. through whatever plug-ins the user
 * registered under the reference's "matmul", "flash3_attention_fwd" and "flash3_attention_bwd" identities (its cuBLASLt helper,
 * unchanged, serves the first; its FlashAttention-3 helper is Hopper code, so on B200 the attention plug-in is the user's).
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

/* ---- sequence batch (seq_batch_structs.h) ---- */
typedef struct seq_batch_config {
	int num_seqs;
	int total_q;                     /* tokens of this batch = rows of every activation */
	int total_k;                     /* keys / values the attention sees */
	int * seq_positions;             /* device, [total_q]: RoPE positions */
	int * q_seq_offsets;             /* device, [num_seqs + 1] */
	int * q_seq_lens;                /* device, [num_seqs] */
	int max_seqlen_q;
	int * k_seq_offsets;
	int * k_seq_lens;
	int max_seqlen_k;
} Seq_Batch_Config;

typedef struct seq_batch_saved_activations {
	Seq_Batch_Config * config;
	void * buffer;
	uint64_t activationBufferBytes;
	void * attn_norm_weighted_sums;  /* fp32 [total_q] */
	void * attn_norm_rms_vals;       /* fp32 [total_q] */
	void * x_q;                      /* [total_q, model_dim], rotated in place */
	void * x_k_local;                /* [total_q, kv_dim], rotated in place */
	void * x_v_local;                /* [total_q, kv_dim] */
	void * softmax_lse;
	void * x_attn_out;               /* [total_q, model_dim] */
	void * x_o;                      /* [total_q, model_dim]: input + attention projection; in a gradient container: d(x_o) */
	void * ffn_norm_weighted_sums;
	void * ffn_norm_rms_vals;
	void ** x_1;                     /* host arrays of one device pointer (one per local expert in the reference); [total_q, ffn_dim] */
	void ** x_2;                     /* [total_q, model_dim]: the block's output */
	void ** x_3;
} Seq_Batch_Saved_Activations;

typedef struct seq_batch_context {
	Seq_Batch_Config * config;
	void * buffer;
	uint64_t contextBufferBytes;
	void * x_k;                      /* what the attention reads: the caller places x_k_local / x_v_local inside (or points these at them) */
	void * x_v;
} Seq_Batch_Context;

typedef struct seq_batch_activation_workspace {
	Seq_Batch_Config * config;
	void * buffer;
	uint64_t activationWorkspaceBytes;
	void * x_temp;                   /* [total_q, model_dim] */
	void * x_temp_mlp;               /* [total_q, ffn_dim] */
	void * recomputed_attn_norm;     /* [total_q, model_dim], written at the end of the input-gradient chain for the weight-gradient chain */
	void * recomputed_ffn_norm;
	void * kernel_workspace;         /* handed to the matmul and attention plug-ins; zeroed before each attention call */
	uint64_t kernel_workspaceBytes;
} Seq_Batch_Activation_Workspace;

/* ---- block (dataflow_models.h, transformer_structs.h) ---- */
typedef enum dataflow_normalization_type { DATAFLOW_RMSNORM, DATAFLOW_LAYERNORM } DataflowNormalizationType;
typedef enum dataflow_actviation_type { DATAFLOW_SWIGLU, DATAFLOW_RELU, DATAFLOW_GELU } DataflowActivationType;
typedef enum dataflow_attention_type { DATAFLOW_EXACT_ATTENTION, DATAFLOW_SPARSE_ATTENTION } DataflowAttentionType;
typedef enum dataflow_mlp_type { DATAFLOW_GATED_MLP, DATAFLOW_VANILLA_MLP, DATAFLOW_MOE_MLP } DataflowMLPType;

typedef struct moe_config {
	int top_k_experts;
	int num_global_experts;
	int num_local_experts;
	int * local_expert_inds;
} MoE_Config;

typedef struct transformer_block_weight_offsets {
	uint64_t w_attn_norm, w_q, w_k, w_v, w_o, w_ffn_norm, w_router;
	uint64_t * w_1;
	uint64_t * w_2;
	uint64_t * w_3;
} Transformer_Block_Weight_Offsets;

typedef struct transformer_block_config {
	DataflowDatatype block_dt;
	DataflowDatatype compute_dt;     /* accumulation type of the projections */
	DataflowNormalizationType normalization_type;
	DataflowAttentionType attention_type;
	DataflowMLPType mlp_type;
	DataflowActivationType activation_type;
	float eps;
	int theta;
	int num_q_heads;
	int num_kv_heads;
	int head_dim;
	int model_dim;                   /* num_q_heads * head_dim */
	int kv_dim;                      /* num_kv_heads * head_dim */
	int ffn_dim;
	MoE_Config moe_config;
	int pointer_alignment;
	Transformer_Block_Weight_Offsets weight_offsets;
	uint64_t block_raw_size;
	uint64_t block_aligned_size;
} Transformer_Block_Config;

/* Weights are [out_features, in_features] row-major (= the reference's column-major [in, out]); in a gradient container the
 * same members hold the weight gradients. */
typedef struct transformer_block {
	Transformer_Block_Config config;
	void * buffer;
	void * w_attn_norm;              /* [model_dim] */
	void * w_q;                      /* [model_dim, model_dim] */
	void * w_k;                      /* [kv_dim, model_dim] */
	void * w_v;
	void * w_o;                      /* [model_dim, model_dim] */
	void * w_ffn_norm;
	void * w_router;
	void ** w_1;                     /* host arrays of one device pointer: gate [ffn_dim, model_dim] */
	void ** w_2;                     /* down [model_dim, ffn_dim] */
	void ** w_3;                     /* up   [ffn_dim, model_dim] */
} Transformer_Block;

typedef struct transformer_block_activations {
	Transformer_Block * block;
	Seq_Batch_Config * batch_config;
	Seq_Batch_Saved_Activations * saved_activations;
	Seq_Batch_Context * context;
	Seq_Batch_Activation_Workspace * activation_workspace;
} Transformer_Block_Activations;

typedef struct transformer_block_transition {
	Seq_Batch_Config * batch_config; /* never dereferenced by these calls */
	void * X;                        /* [num_tokens, embedding_size] */
} Transformer_Block_Transition;

typedef struct transformer_model_output {
	Seq_Batch_Config * batch_config;
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

/*
 * One transformer block forward, in the reference's step order (dataflow_transformer.c:72-264), all on compute_stream_id:
 *   rms_norm(X) -> x_temp;  Q, K, V projections of x_temp -> x_q, x_k_local, x_v_local;  rope in place on x_q, x_k_local;
 *   kernel_workspace zeroed;  attention(x_q, context x_k, context x_v) -> x_attn_out, softmax_lse;
 *   x_o = x_attn_out W_o^T + X (beta = 1);  rms_norm(x_o) -> x_temp;  x_1 = x_temp W_1^T, x_3 = x_temp W_3^T;
 *   swiglu(x_1, x_3) -> x_temp_mlp;  x_2 = x_temp_mlp W_2^T + x_o (beta = 1);  block_output->X = copy of x_2 on out_copy_stream_id,
 *   ordered after the compute stream through the handle's stream state.
 * Where the reference's text cannot be what was meant: the K and V projections are given M = model_dim, K = kv_dim (:103,117; the
 * output has kv_dim features and the contraction runs over model_dim: M = kv_dim, K = model_dim here); w_1 and w_3 are passed as the
 * arrays themselves instead of their first entries (:224,238); the output copy is not ordered after the compute stream (:280-283).
 * Nothing moves x_k_local / x_v_local into the context: the caller points context->x_k / x_v at them (one sequence without a
 * cache) or copies with submit_copy_to_seq_context, as in the reference.
 */
int submit_transformer_block(Dataflow_Handle * dataflow_handle, int compute_stream_id, int out_copy_stream_id,
                             Transformer_Block_Transition * block_input, Transformer_Block * transformer_block,
                             Transformer_Block_Activations * activations, Transformer_Block_Transition * block_output);

/*
 * Input gradients of one block, in the reference's step order (:565-822). inp_grad_stream->X holds the gradient with respect to the
 * block's output on entry and the gradient with respect to its input on return: both RMSNorm input-gradient ops ACCUMULATE into it
 * (the residual connections), which is the dX += contract of submit_rms_norm_bwd_x. Steps:
 *   d(x_temp_mlp) = dOut W_2;  swiglu_bwd_x -> d(x_1), d(x_3) (grad_activations saved x_1 / x_3);  x_temp = d(x_1) W_1 + d(x_3) W_3;
 *   rms_norm_bwd_x(ffn) accumulates into the stream gradient;  rms_norm_bwd_w(ffn) into grad_weights->w_ffn_norm;
 *   grad_activations x_o = copy of the stream gradient (= d(x_o), kept for the W_o weight gradient);
 *   x_temp = d(x_o) W_o;  workspace zeroed;  attention_bwd -> d(x_q), grad context x_k / x_v;  rope_bwd_x in place on d(x_q), d(x_k_local);
 *   x_temp = d(x_q) W_q + d(x_k_local) W_k + d(x_v_local) W_v;  rms_norm_bwd_x(attn) accumulates into the stream gradient;
 *   rms_norm_bwd_w(attn) into grad_weights->w_attn_norm;  the two RMSNorm outputs recomputed (statistics pointers NULL) into
 *   recomputed_attn_norm / recomputed_ffn_norm of the gradient workspace;  out_grad_stream->X (optional) = copy on out_copy_stream_id.
 * Where the reference's text cannot be what was meant: the W_3, W_k and W_v products are "added to the previous gradient" with
 * beta = 1 but no C matrix (:628,773,785: C = x_temp, c_dt = the block type here); the W_o product reads grad_activations x_o, which
 * nothing has written (:665: it is the stream gradient after the FFN half, copied there here); the two recompute calls treat a
 * SUCCESSFUL submission as the error (:806,818); num_seqs, total_q and total_k are declared twice (:536-542).
 */
int submit_transformer_block_bwd_x(Dataflow_Handle * dataflow_handle, int compute_stream_id, int out_copy_stream_id,
                                   Transformer_Block * transformer_block, Transformer_Block_Transition * inp_grad_stream,
                                   Transformer_Block_Activations * activations, Transformer_Block_Transition * fwd_block_input,
                                   Transformer_Block_Activations * grad_activations, Transformer_Block * grad_weights,
                                   Transformer_Block_Transition * out_grad_stream);

/*
 * Weight gradients of one block (:853-1003), accumulated (beta = 1) into grad_weights: swiglu recomputed into x_temp_mlp, then
 *   dW_2 += dOut^T x_temp_mlp;  dW_1 += d(x_1)^T ffn_norm;  dW_3 += d(x_3)^T ffn_norm;  dW_o += d(x_o)^T x_attn_out;
 *   dW_v += d(x_v_local)^T attn_norm;  dW_k += d(x_k_local)^T attn_norm;  dW_q += d(x_q)^T attn_norm
 * with attn_norm / ffn_norm = the recomputed RMSNorm outputs left by submit_transformer_block_bwd_x. grad_stream->X must hold the
 * gradient with respect to the block's OUTPUT (what the input-gradient chain received, before it accumulated into that buffer).
 * The RMSNorm weight gradients were made by the input-gradient chain. Where the reference's text cannot be what was meant: every
 * product is submitted with to_trans_a = 1 and M, K, N = (out, in, tokens) (:899-989), which contracts over the wrong index for a
 * weight gradient (here: dW(in x out, column-major) += x(in x T) dy^T(T x out): to_trans_b = 1, M = in, K = tokens, N = out, A = the
 * layer input, B = the output gradient -- the form the head uses); dW_v and dW_q read the recomputed FFN norm instead of the
 * attention norm (:954,980).
 */
int submit_transformer_block_bwd_w(Dataflow_Handle * dataflow_handle, int compute_stream_id,
                                   Transformer_Block_Transition * grad_stream, Transformer_Block_Activations * activations,
                                   Transformer_Block_Activations * grad_activations, Transformer_Block * grad_weights);

#ifdef __cplusplus
}
#endif
#endif
