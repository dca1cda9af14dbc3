/*
 * A stand-in attention plug-in for the block-caller tests: External_Lib_Func functions registered under the reference's
 * "flash3_attention_fwd" / "flash3_attention_bwd" identities (als244/dataflow_lib src/dataflow_ops/src/attention_op.c:55-130 gives the
 * argument order). It does no attention arithmetic -- the reference's plug-in is FlashAttention-3, Hopper code -- only copies that make
 * every buffer's wiring observable:
 *     forward   x_attn_out = x_q
 *     backward  dx_q = dx_out,  dx_k = x_k,  dx_v = x_v
 * through the handle's own device-to-device transfer on the op's stream, so the file needs no CUDA header and links nothing.
 */
#include "dataflow_api.h"

#define ARG(op, i, type) (*(type *) (op)->op_args[i])

static uint64_t elem_bytes(DataflowDatatype dt) { return dt == DATAFLOW_FP32 ? 4 : (dt == DATAFLOW_FP16 || dt == DATAFLOW_BF16) ? 2 : 1; }

int standin_attention_fwd(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	const uint64_t e = elem_bytes((DataflowDatatype) ARG(op, 0, int));
	const uint64_t total_q = (uint64_t) ARG(op, 2, int), q_heads = (uint64_t) ARG(op, 10, int), head_dim = (uint64_t) ARG(op, 12, int);
	return h->submit_peer_transfer(h, stream_id, ARG(op, 16, void *), ARG(op, 13, void *), total_q * q_heads * head_dim * e);
}

int standin_attention_bwd(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	const uint64_t e = elem_bytes((DataflowDatatype) ARG(op, 0, int));
	const uint64_t total_q = (uint64_t) ARG(op, 2, int), total_k = (uint64_t) ARG(op, 3, int);
	const uint64_t q_heads = (uint64_t) ARG(op, 10, int), kv_heads = (uint64_t) ARG(op, 11, int), head_dim = (uint64_t) ARG(op, 12, int);
	int rc = h->submit_peer_transfer(h, stream_id, ARG(op, 19, void *), ARG(op, 18, void *), total_q * q_heads * head_dim * e);
	if (!rc) rc = h->submit_peer_transfer(h, stream_id, ARG(op, 20, void *), ARG(op, 14, void *), total_k * kv_heads * head_dim * e);
	if (!rc) rc = h->submit_peer_transfer(h, stream_id, ARG(op, 21, void *), ARG(op, 15, void *), total_k * kv_heads * head_dim * e);
	return rc;
}
