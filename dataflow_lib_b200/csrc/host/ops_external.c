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

/* Per-op device scratch kept in Cuda_Function.op_extra: one grow-only block per (op identity, stream), so that submissions of
 * the same op on different streams of a handle never share scratch (slot 0 serves stream id -1, the default stream). A block is
 * allocated at the first submission that needs it, or ahead of time with dataflow_b200_reserve_workspace so that no submission in a
 * step loop allocates; growing a block frees the old one, which waits for all work on the device first (cudaFree synchronises).
 * destroy_cuda_dataflow_handle releases the blocks through dataflow_b200_workspace_release. */
typedef struct { void * ptr; uint64_t bytes; } Ws_Block;
typedef struct { Ws_Block by_stream[MAX_STREAMS + 1]; } Op_Workspace;

int dataflow_b200_workspace_init(Dataflow_Handle * handle, void * op_table_value) {
	(void) handle;
	Op_Workspace * ws = (Op_Workspace *) calloc(1, sizeof(Op_Workspace));
	if (!ws) return -1;
	((Cuda_Function *) op_table_value)->op_extra = ws;
	return 0;
}

static Ws_Block * ensure_workspace(Op_Workspace * all, int stream_id, uint64_t bytes) {
	if (!all) { fprintf(stderr, "Error: op was registered without its workspace init function\n"); return NULL; }
	if (stream_id < -1 || stream_id >= MAX_STREAMS) { fprintf(stderr, "Error: no op workspace for stream id %d\n", stream_id); return NULL; }
	Ws_Block * ws = &all->by_stream[stream_id + 1];
	if (ws->bytes >= bytes && ws->ptr) return ws;
	if (ws->ptr) cudaFree(ws->ptr);
	ws->ptr = NULL; ws->bytes = 0;
	const uint64_t rounded = ((bytes ? bytes : 1) + ((1u << 20) - 1)) & ~(uint64_t) ((1u << 20) - 1);
	cudaError_t e = cudaMalloc(&ws->ptr, rounded);
	if (e != cudaSuccess) { fprintf(stderr, "Error: cannot allocate %lu bytes of op workspace: %s\n", (unsigned long) rounded, cudaGetErrorString(e)); cudaGetLastError(); ws->ptr = NULL; return NULL; }
	ws->bytes = rounded;
	return ws;
}

int dataflow_b200_rms_norm_bwd_w(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);
int dataflow_b200_rms_norm_bwd_w_sums(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);
int dataflow_b200_rms_norm_bwd_x_w(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);
int dataflow_b200_rms_norm_bwd_x_w_sums(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);
int dataflow_b200_softmax_cross_entropy(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);
int dataflow_b200_swiglu_ffn_fp8(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);
int dataflow_b200_swiglu_ffn_fp8_bwd(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra);

static int owns_workspace(const Cuda_Function * fn) {
	return fn && !fn->is_native && fn->op_extra &&
	       (fn->cuda_external_func == dataflow_b200_rms_norm_bwd_w || fn->cuda_external_func == dataflow_b200_rms_norm_bwd_w_sums ||
	        fn->cuda_external_func == dataflow_b200_rms_norm_bwd_x_w || fn->cuda_external_func == dataflow_b200_rms_norm_bwd_x_w_sums ||
	        fn->cuda_external_func == dataflow_b200_softmax_cross_entropy ||
	        fn->cuda_external_func == dataflow_b200_swiglu_ffn_fp8 || fn->cuda_external_func == dataflow_b200_swiglu_ffn_fp8_bwd);
}

/* Makes the scratch block of (op, stream_id) at least `bytes` large now, so that later submissions of that op on that stream do not
 * allocate. `bytes` comes from the matching dfb200_*_workspace_bytes function. Returns 0, or -1 when the op is not registered on the
 * handle, keeps no scratch, or the allocation fails. */
int dataflow_b200_reserve_workspace(Dataflow_Handle * handle, Op_Skeleton * skeleton, int stream_id, uint64_t bytes) {
	Cuda_Function * fn = NULL;
	if (!handle || !skeleton || find_table(&handle->op_table, skeleton->identifier.fingerprint, false, (void **) &fn) < 0 || !owns_workspace(fn)) {
		fprintf(stderr, "Error: cannot reserve op workspace: op %s is not registered or keeps no scratch\n", skeleton ? skeleton->header.op_nickname : "(null)");
		return -1;
	}
	int cur = -1;
	if (cudaGetDevice(&cur) != cudaSuccess || cur != handle->device_id) {
		if (cudaSetDevice(handle->device_id) != cudaSuccess) { cudaGetLastError(); return -1; }
	}
	return ensure_workspace((Op_Workspace *) fn->op_extra, stream_id, bytes) ? 0 : -1;
}

/* Frees the scratch blocks of one op-table entry if that entry is one of this library's ops with scratch (the caller has made the
 * device current and idle). Entries of other plug-ins are left alone: their op_extra is theirs. */
void dataflow_b200_workspace_release(void * op_table_value) {
	Cuda_Function * fn = (Cuda_Function *) op_table_value;
	if (!owns_workspace(fn)) return;
	Op_Workspace * all = (Op_Workspace *) fn->op_extra;
	for (int i = 0; i <= MAX_STREAMS; i++)
		if (all->by_stream[i].ptr && cudaFree(all->by_stream[i].ptr) != cudaSuccess) cudaGetLastError();
	free(all);
	fn->op_extra = NULL;
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
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols));
	if (!ws) return -1;
	return finish(dfb200_rms_norm_bwd_w(DT(op, 4), DT(op, 5), n_rows, n_cols, ARG(op, 2, float), ARG(op, 3, float *), ARG(op, 4, void *),
	                                    ARG(op, 5, void *), ARG(op, 6, void *), ws->ptr, ws->bytes, stream_of(h, stream_id)), "rms_norm_bwd_w");
}

int dataflow_b200_rms_norm_bwd_w_sums(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols));
	if (!ws) return -1;
	return finish(dfb200_rms_norm_bwd_w_sums(DT(op, 4), DT(op, 5), n_rows, n_cols, ARG(op, 2, float), ARG(op, 3, float *), ARG(op, 4, void *),
	                                         ARG(op, 5, void *), ARG(op, 6, float *), ws->ptr, ws->bytes, stream_of(h, stream_id)), "rms_norm_bwd_w_sums");
}

/* args: n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, dW (or fp32 column_sums) */
int dataflow_b200_rms_norm_bwd_x_w(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols));
	if (!ws) return -1;
	return finish(dfb200_rms_norm_bwd_x_w(DT(op, 5), DT(op, 7), n_rows, n_cols, ARG(op, 2, float), ARG(op, 3, float *), ARG(op, 4, float *),
	                                      ARG(op, 5, void *), ARG(op, 6, void *), ARG(op, 7, void *), ARG(op, 8, void *), ARG(op, 9, void *), ws->ptr,
	                                      ws->bytes, stream_of(h, stream_id)), "rms_norm_bwd_x_w");
}

int dataflow_b200_rms_norm_bwd_x_w_sums(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols));
	if (!ws) return -1;
	return finish(dfb200_rms_norm_bwd_x_w_sums(DT(op, 5), DT(op, 7), n_rows, n_cols, ARG(op, 2, float), ARG(op, 3, float *), ARG(op, 4, float *),
	                                           ARG(op, 5, void *), ARG(op, 6, void *), ARG(op, 7, void *), ARG(op, 8, void *), ARG(op, 9, float *),
	                                           ws->ptr, ws->bytes, stream_of(h, stream_id)), "rms_norm_bwd_x_w_sums");
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
	const int n_rows = ARG(op, 0, int), n_cols = ARG(op, 1, int);
	float * row_loss = ARG(op, 5, float *), * loss_sum = ARG(op, 6, float *);
	void * scratch = NULL; uint64_t scratch_bytes = 0;
	if (!row_loss && loss_sum) {
		Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_softmax_cross_entropy_workspace_bytes(n_rows, n_cols));
		if (!ws) return -1;
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
	const int T = ARG(op, 0, int), d = ARG(op, 1, int), f = ARG(op, 2, int);
	Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f));
	if (!ws) return -1;
	return finish(dfb200_swiglu_ffn_fp8(T, d, f, ARG(op, 3, void *), ARG(op, 4, void *), ARG(op, 5, float *), ARG(op, 6, void *), ARG(op, 7, float *),
	                                    ARG(op, 8, void *), ARG(op, 9, float *), ARG(op, 10, void *), ARG(op, 11, void *), ARG(op, 12, void *),
	                                    ARG(op, 13, void *), ws->ptr, ws->bytes, stream_of(h, stream_id)), "swiglu_ffn_fp8");
}

int dataflow_b200_swiglu_ffn_fp8_bwd(Dataflow_Handle * h, int stream_id, Op * op, void * op_extra) {
	const int T = ARG(op, 0, int), d = ARG(op, 1, int), f = ARG(op, 2, int);
	Ws_Block * ws = ensure_workspace((Op_Workspace *) op_extra, stream_id, dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f));
	if (!ws) return -1;
	return finish(dfb200_swiglu_ffn_fp8_bwd(T, d, f, ARG(op, 3, void *), ARG(op, 4, void *), ARG(op, 5, void *), ARG(op, 6, void *), ARG(op, 7, float *),
	                                        ARG(op, 8, void *), ARG(op, 9, float *), ARG(op, 10, void *), NULL, ws->ptr, ws->bytes, stream_of(h, stream_id)),
	              "swiglu_ffn_fp8_bwd");
}
