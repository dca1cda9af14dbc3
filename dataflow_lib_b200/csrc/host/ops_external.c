/*
 * The ops as external plug-in functions (External_Lib_Func: handle, stream id, Op, op_extra;
 * als244/dataflow_lib src/dataflow_handle/include/dataflow_handle.h:131-136). Each function
 * unpacks op_args by the positions the submit_* wrappers use, reads the datatypes from the
 * skeleton header, resolves the stream the way the reference's external matmul does
 * (((CUstream *) handle->streams)[stream_id], src/ops/nvidia/external/matmul_helper/src/matmul_helper.c:596-598)
 * and calls the C-ABI kernel launcher. One exported symbol serves every datatype variant of an
 * op family, because the variant is recoverable from the skeleton.
 */
#include "dataflow_api.h"
#include "dataflow_b200_kernels.h"

#include <cuda_runtime_api.h>
#include <stdlib.h>

#define ARG(op, i, type) (*(type *) (op)->op_args[i])
#define DT(op, i) ((int) (op)->op_skeleton.header.arg_dtypes[i])

static void * stream_of(Dataflow_Handle * h, int stream_id) {
	return stream_id == -1 ? NULL : ((void **) h->streams)[stream_id];
}

static int finish(int rc, const char * what) {
	if (rc == DFB200_OK) return 0;
	fprintf(stderr, "Error: %s failed (%d): %s\n", what, rc, dfb200_last_error());
	return -1;
}

/* Per-op device scratch kept in Cuda_Function.op_extra. It grows on demand; growing frees the
 * old block, which waits for all work on the device first (cudaFree synchronises). */
typedef struct { void * ptr; uint64_t bytes; } Op_Workspace;

int dataflow_b200_workspace_init(Dataflow_Handle * handle, void * op_table_value) {
	(void) handle;
	Op_Workspace * ws = (Op_Workspace *) calloc(1, sizeof(Op_Workspace));
	if (!ws) return -1;
	((Cuda_Function *) op_table_value)->op_extra = ws;
	return 0;
}

static int ensure_workspace(Op_Workspace * ws, uint64_t bytes) {
	if (!ws) { fprintf(stderr, "Error: op was registered without its workspace init function\n"); return -1; }
	if (ws->bytes >= bytes) return 0;
	if (ws->ptr) cudaFree(ws->ptr);
	ws->ptr = NULL; ws->bytes = 0;
	const uint64_t rounded = (bytes + ((1u << 20) - 1)) & ~(uint64_t) ((1u << 20) - 1);
	cudaError_t e = cudaMalloc(&ws->ptr, rounded);
	if (e != cudaSuccess) { fprintf(stderr, "Error: cannot allocate %lu bytes of op workspace: %s\n", (unsigned long) rounded, cudaGetErrorString(e)); cudaGetLastError(); return -1; }
	ws->bytes = rounded;
	return 0;
}

int dataflow_b200_rms_norm(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_rms_norm(DT(op, 3), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, float), ARG(op, 3, void *), ARG(op, 4, void *),
	                              ARG(op, 5, void *), ARG(op, 6, float *), ARG(op, 7, float *), stream_of(h, stream_id)), "rms_norm");
}

int dataflow_b200_rms_norm_bwd_x(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_rms_norm_bwd_x(DT(op, 5), DT(op, 7), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, float), ARG(op, 3, float *),
	                                    ARG(op, 4, float *), ARG(op, 5, void *), ARG(op, 6, void *), ARG(op, 7, void *), ARG(op, 8, void *),
	                                    stream_of(h, stream_id)), "rms_norm_bwd_x");
}

int dataflow_b200_rms_norm_bwd_w(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	Op_Workspace * ws = (Op_Workspace *) op_extra;
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	if (ensure_workspace(ws, dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols))) return -1;
	return finish(dfb200_rms_norm_bwd_w(DT(op, 4), DT(op, 5), n_rows, n_cols, ARG(op, 2, float), ARG(op, 3, float *), ARG(op, 4, void *),
	                                    ARG(op, 5, void *), ARG(op, 6, void *), ws->ptr, ws->bytes, stream_of(h, stream_id)), "rms_norm_bwd_w");
}

int dataflow_b200_rope(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_rope(DT(op, 6), ARG(op, 0, uint64_t), ARG(op, 1, int), ARG(op, 2, int), ARG(op, 3, int), ARG(op, 4, int),
	                          ARG(op, 5, int *), ARG(op, 6, void *), ARG(op, 7, void *), stream_of(h, stream_id)), "rope");
}

int dataflow_b200_rope_bwd_x(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_rope_bwd_x(DT(op, 6), ARG(op, 0, uint64_t), ARG(op, 1, int), ARG(op, 2, int), ARG(op, 3, int), ARG(op, 4, int),
	                                ARG(op, 5, int *), ARG(op, 6, void *), ARG(op, 7, void *), stream_of(h, stream_id)), "rope_bwd_x");
}

int dataflow_b200_swiglu(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_swiglu(DT(op, 2), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, void *), ARG(op, 3, void *), ARG(op, 4, void *),
	                            stream_of(h, stream_id)), "swiglu");
}

int dataflow_b200_swiglu_bwd_x(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_swiglu_bwd_x(DT(op, 2), DT(op, 4), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, void *), ARG(op, 3, void *),
	                                  ARG(op, 4, void *), ARG(op, 5, void *), ARG(op, 6, void *), stream_of(h, stream_id)), "swiglu_bwd_x");
}

int dataflow_b200_softmax(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_softmax(DT(op, 2), DT(op, 3), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, void *), ARG(op, 3, void *),
	                             stream_of(h, stream_id)), "softmax");
}

int dataflow_b200_cross_entropy_loss(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_cross_entropy_loss(DT(op, 2), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, void *), ARG(op, 3, uint32_t *),
	                                        stream_of(h, stream_id)), "cross_entropy_loss");
}

int dataflow_b200_softmax_cross_entropy(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	Op_Workspace * ws = (Op_Workspace *) op_extra;
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	float * row_loss = ARG(op, 5, float *), * loss_sum = ARG(op, 6, float *);
	void * scratch = NULL; uint64_t scratch_bytes = 0;
	if (!row_loss && loss_sum) {
		if (ensure_workspace(ws, dfb200_softmax_cross_entropy_workspace_bytes(n_rows, n_cols))) return -1;
		scratch = ws->ptr; scratch_bytes = ws->bytes;
	}
	return finish(dfb200_softmax_cross_entropy(DT(op, 2), DT(op, 4), n_rows, n_cols, ARG(op, 2, void *), ARG(op, 3, uint32_t *),
	                                           ARG(op, 4, void *), row_loss, loss_sum, scratch, scratch_bytes, stream_of(h, stream_id)),
	              "softmax_cross_entropy");
}

int dataflow_b200_embedding(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_embedding(DT(op, 3), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, uint32_t *), ARG(op, 3, void *), ARG(op, 4, void *),
	                               stream_of(h, stream_id)), "embedding");
}

int dataflow_b200_copy_to_seq_context(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_copy_to_seq_context(DT(op, 3), ARG(op, 0, uint64_t), ARG(op, 1, int), ARG(op, 2, int), ARG(op, 3, void *), ARG(op, 4, void *),
	                                         ARG(op, 5, int *), ARG(op, 6, uint64_t *), ARG(op, 7, int *), stream_of(h, stream_id)), "copy_to_seq_context");
}

int dataflow_b200_select_experts(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_select_experts(DT(op, 3), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, int), ARG(op, 3, void *), ARG(op, 4, void *),
	                                    ARG(op, 5, uint16_t *), ARG(op, 6, int *), ARG(op, 7, int *), ARG(op, 8, int *), stream_of(h, stream_id)),
	              "select_experts");
}

int dataflow_b200_softmax_argmax(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	(void) op_extra;
	return finish(dfb200_softmax_fp32_out(DT(op, 2), ARG(op, 0, int), ARG(op, 1, int), ARG(op, 2, void *), ARG(op, 3, float *), ARG(op, 4, uint32_t *),
	                                      stream_of(h, stream_id)), "softmax_argmax");
}

int dataflow_b200_swiglu_ffn_fp8(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	Op_Workspace * ws = (Op_Workspace *) op_extra;
	const int T = ARG(op, 0, int), d = ARG(op, 1, int), f = ARG(op, 2, int);
	if (ensure_workspace(ws, dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f))) return -1;
	return finish(dfb200_swiglu_ffn_fp8(T, d, f, ARG(op, 3, void *), ARG(op, 4, void *), ARG(op, 5, float *), ARG(op, 6, void *), ARG(op, 7, float *),
	                                    ARG(op, 8, void *), ARG(op, 9, float *), ARG(op, 10, void *), ARG(op, 11, void *), ARG(op, 12, void *),
	                                    ARG(op, 13, void *), ws->ptr, ws->bytes, stream_of(h, stream_id)), "swiglu_ffn_fp8");
}

int dataflow_b200_swiglu_ffn_fp8_bwd(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	Op_Workspace * ws = (Op_Workspace *) op_extra;
	const int T = ARG(op, 0, int), d = ARG(op, 1, int), f = ARG(op, 2, int);
	if (ensure_workspace(ws, dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f))) return -1;
	return finish(dfb200_swiglu_ffn_fp8_bwd(T, d, f, ARG(op, 3, void *), ARG(op, 4, void *), ARG(op, 5, void *), ARG(op, 6, void *), ARG(op, 7, float *),
	                                        ARG(op, 8, void *), ARG(op, 9, float *), ARG(op, 10, void *), NULL, ws->ptr, ws->bytes, stream_of(h, stream_id)),
	              "swiglu_ffn_fp8_bwd");
}
