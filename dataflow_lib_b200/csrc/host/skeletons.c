/*
 * Op skeletons: the (nickname, argument datatypes) records whose SHA-256 is an op's registry
 * key, and registration of this library's ops under those keys.
 *
 * Nicknames ("<op>_<DTYPE>[_<DTYPE>]", upper-case datatype names) and argument lists are the
 * ones als244/dataflow_lib builds in src/set_ops/src/set_native_op_skeletons.c:234-611, so the
 * fingerprints are bit-identical and a submit_*() call written for that library finds the op
 * here. The ops themselves are exported by this shared object as EXTERNAL functions
 * (External_Lib_Func signature, see ops_external.c) rather than as cubin symbols with
 * launch-config callbacks: an external function is free to launch clusters and several
 * kernels per op, which a bare cuLaunchKernel of one symbol is not.
 */
#define _GNU_SOURCE
#include "dataflow_api.h"

#include <dlfcn.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

/* Fill the header from a nickname and a datatype list terminated by -1, then fingerprint it. */
static void build_skeleton(Op_Skeleton * skeleton, const char * nickname, ...) {
	Op_Skeleton_Header * h = &skeleton->header;
	memset(h, 0, sizeof(*h));
	strncpy(h->op_nickname, nickname, MAX_OP_NICKNAME_SIZE);
	va_list ap;
	va_start(ap, nickname);
	int n = 0;
	for (;;) {
		const int dt = va_arg(ap, int);
		if (dt < 0 || n == MAX_OP_ARGS) break;
		h->arg_dtypes[n++] = (DataflowDatatype) dt;
	}
	va_end(ap);
	h->num_args = n;
	for (int i = n; i < MAX_OP_ARGS; i++) h->arg_dtypes[i] = DATAFLOW_NONE;
	do_fingerprinting(h, sizeof(*h), skeleton->identifier.fingerprint, OP_IDENTIFIER_FINGERPRINT_TYPE);
}

static const char * nick1(char * buf, const char * op, DataflowDatatype a) {
	snprintf(buf, MAX_OP_NICKNAME_SIZE, "%s_%s", op, dataflow_datatype_as_string(a));
	return buf;
}
static const char * nick2(char * buf, const char * op, DataflowDatatype a, DataflowDatatype b) {
	snprintf(buf, MAX_OP_NICKNAME_SIZE, "%s_%s_%s", op, dataflow_datatype_as_string(a), dataflow_datatype_as_string(b));
	return buf;
}

#define END -1
#define I_S DATAFLOW_INT_SCALAR
#define F_S DATAFLOW_FP32_SCALAR
#define U64_S DATAFLOW_UINT64_SCALAR

void set_native_embedding_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* num_tokens, embed_dim, token_ids, table, out */
	build_skeleton(skeleton, nick1(nick, "embedding", fwd), I_S, I_S, DATAFLOW_UINT32, fwd, fwd, END);
}
void set_native_rms_norm_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, eps, weight, X, out, weighted_sums, rms_vals */
	build_skeleton(skeleton, nick1(nick, "rms_norm", fwd), I_S, I_S, F_S, fwd, fwd, fwd, DATAFLOW_FP32, DATAFLOW_FP32, END);
}
void set_native_rms_norm_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, eps, weighted_sums, rms_vals, weight, X, dY, dX */
	build_skeleton(skeleton, nick2(nick, "rms_norm_bwd_x", fwd, bwd), I_S, I_S, F_S, DATAFLOW_FP32, DATAFLOW_FP32, fwd, fwd, bwd, bwd, END);
}
void set_native_rms_norm_bwd_w_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, eps, rms_vals, X, dY, dW */
	build_skeleton(skeleton, nick2(nick, "rms_norm_bwd_w", fwd, bwd), I_S, I_S, F_S, DATAFLOW_FP32, fwd, bwd, bwd, END);
}
void set_native_rms_norm_bwd_w_sums_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, eps, rms_vals, X, dY, column sums (fp32) */
	build_skeleton(skeleton, nick2(nick, "rms_norm_bwd_w_sums", fwd, bwd), I_S, I_S, F_S, DATAFLOW_FP32, fwd, bwd, DATAFLOW_FP32, END);
}
void set_native_rms_norm_bwd_x_w_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, eps, weighted_sums, rms_vals, weight, X, dY, dX, dW */
	build_skeleton(skeleton, nick2(nick, "rms_norm_bwd_x_w", fwd, bwd), I_S, I_S, F_S, DATAFLOW_FP32, DATAFLOW_FP32, fwd, fwd, bwd, bwd, bwd, END);
}
void set_native_rms_norm_bwd_x_w_sums_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, eps, weighted_sums, rms_vals, weight, X, dY, dX, column sums (fp32) */
	build_skeleton(skeleton, nick2(nick, "rms_norm_bwd_x_w_sums", fwd, bwd), I_S, I_S, F_S, DATAFLOW_FP32, DATAFLOW_FP32, fwd, fwd, bwd, bwd, DATAFLOW_FP32, END);
}
void set_native_rope_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* N, model_dim, head_dim, num_kv_heads, theta, seq_positions, X_q, X_k */
	build_skeleton(skeleton, nick1(nick, "rope", fwd), U64_S, I_S, I_S, I_S, I_S, DATAFLOW_INT, fwd, fwd, END);
}
void set_native_rope_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];
	build_skeleton(skeleton, nick1(nick, "rope_bwd_x", bwd), U64_S, I_S, I_S, I_S, I_S, DATAFLOW_INT, bwd, bwd, END);
}
void set_native_copy_to_seq_context_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* N, total_tokens, kv_dim, X_k, X_v, seq_positions, seq_context_ptrs, seq_context_sizes */
	build_skeleton(skeleton, nick1(nick, "copy_to_seq_context", fwd), U64_S, I_S, I_S, fwd, fwd, DATAFLOW_INT, DATAFLOW_UINT64, DATAFLOW_INT, END);
}
void set_native_swiglu_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* num_rows, num_cols, x_w1, x_w3, out */
	build_skeleton(skeleton, nick1(nick, "swiglu", fwd), I_S, I_S, fwd, fwd, fwd, END);
}
void set_native_swiglu_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* num_rows, num_cols, x_w1, x_w3, dY, dX_w1, dX_w3 */
	build_skeleton(skeleton, nick2(nick, "swiglu_bwd_x", fwd, bwd), I_S, I_S, fwd, fwd, bwd, bwd, bwd, END);
}
void set_native_softmax_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, X, out */
	build_skeleton(skeleton, nick2(nick, "softmax", fwd, bwd), I_S, I_S, fwd, bwd, END);
}
void set_native_cross_entropy_loss_skeleton(Op_Skeleton * skeleton, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, pred_logits, labels */
	build_skeleton(skeleton, nick1(nick, "cross_entropy_loss", bwd), I_S, I_S, bwd, DATAFLOW_UINT32, END);
}
void set_native_swiglu_ffn_fp8_skeleton(Op_Skeleton * skeleton) {
	/* T, d, f, A, Wgate, gate_scales, Wup, up_scales, Wdown, down_scales, residual, out, gate_save, up_save */
	const DataflowDatatype a = DATAFLOW_BF16, w = DATAFLOW_FP8E4M3, sc = DATAFLOW_FP32;
	build_skeleton(skeleton, "swiglu_ffn_fp8_BF16", I_S, I_S, I_S, a, w, sc, w, sc, w, sc, a, a, a, a, END);
}
void set_native_swiglu_ffn_fp8_bwd_skeleton(Op_Skeleton * skeleton) {
	/* T, d, f, dOut, gate_saved, up_saved, WdownT, down_scales, WgateupT, gateup_scales, dA */
	const DataflowDatatype a = DATAFLOW_BF16, w = DATAFLOW_FP8E4M3, sc = DATAFLOW_FP32;
	build_skeleton(skeleton, "swiglu_ffn_fp8_bwd_BF16", I_S, I_S, I_S, a, a, a, w, sc, w, sc, a, END);
}
void set_native_softmax_argmax_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, X, out, arg_maxs */
	build_skeleton(skeleton, nick2(nick, "softmax_argmax", fwd, DATAFLOW_FP32), I_S, I_S, fwd, DATAFLOW_FP32, DATAFLOW_UINT32, END);
}
void set_native_select_experts_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* total_tokens, n_experts, top_k, X_routed, weights, chosen_experts, counts, cumsum, num_routed */
	build_skeleton(skeleton, nick1(nick, "select_experts", fwd), I_S, I_S, I_S, fwd, fwd, DATAFLOW_UINT16, DATAFLOW_INT, DATAFLOW_INT, DATAFLOW_INT, END);
}
void set_native_softmax_cross_entropy_skeleton(Op_Skeleton * skeleton, DataflowDatatype fwd, DataflowDatatype bwd) {
	char nick[MAX_OP_NICKNAME_SIZE];   /* n_rows, n_cols, logits, labels, dlogits, row_loss, loss_sum */
	build_skeleton(skeleton, nick2(nick, "softmax_cross_entropy", fwd, bwd), I_S, I_S, fwd, DATAFLOW_UINT32, bwd, DATAFLOW_FP32, DATAFLOW_FP32, END);
}

/* ---- external ops: the identities under which a user registers the cuBLASLt matmul and FlashAttention-3 plug-ins
 * (als244/dataflow_lib src/set_ops/src/set_external_op_skeletons.c:4-73, 75-155, 157-243). This library ships no such plug-in;
 * the skeletons exist so that code written against the reference finds the same fingerprints here. Datatypes travel as
 * integer scalars, tensors as untyped pointers. */
#define V_P DATAFLOW_VOID
void set_external_matmul_skeleton(Op_Skeleton * skeleton) {
	/* num_sms, a_dt, b_dt, c_dt, d_dt, compute_dt, to_trans_a, to_trans_b, M, K, N, alpha, beta, A, B, C, D, workspaceBytes, workspace */
	build_skeleton(skeleton, "matmul", I_S, I_S, I_S, I_S, I_S, I_S, I_S, I_S, I_S, I_S, I_S, F_S, F_S, V_P, V_P, V_P, V_P,
	               DATAFLOW_UINT64, V_P, END);
}
/* dtype, num_seqs, total_q, total_k, q_seq_offsets, q_seq_lens, max_seqlen_q, k_seq_offsets, k_seq_lens, max_seqlen_k,
 * num_q_heads, num_kv_heads, head_dim, x_q, x_k, x_v, x_attn_out, softmax_lse, [dx_out, dx_q, dx_k, dx_v,] workspaceBytes, workspace */
void set_external_flash3_attention_fwd_skeleton(Op_Skeleton * skeleton) {
	build_skeleton(skeleton, "flash3_attention_fwd", I_S, I_S, I_S, I_S, DATAFLOW_INT, DATAFLOW_INT, I_S, DATAFLOW_INT, DATAFLOW_INT, I_S,
	               I_S, I_S, I_S, V_P, V_P, V_P, V_P, V_P, U64_S, V_P, END);
}
void set_external_flash3_attention_bwd_skeleton(Op_Skeleton * skeleton) {
	build_skeleton(skeleton, "flash3_attention_bwd", I_S, I_S, I_S, I_S, DATAFLOW_INT, DATAFLOW_INT, I_S, DATAFLOW_INT, DATAFLOW_INT, I_S,
	               I_S, I_S, I_S, V_P, V_P, V_P, V_P, V_P, V_P, V_P, V_P, V_P, U64_S, V_P, END);
}

int set_native_op_skeleton(Op_Skeleton * skeleton, char * op_name, DataflowDatatype fwd_dt, DataflowDatatype bwd_dt) {
	if (!strcmp(op_name, "embedding")) set_native_embedding_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "rms_norm")) set_native_rms_norm_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "rms_norm_bwd_x")) set_native_rms_norm_bwd_x_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "rms_norm_bwd_w")) set_native_rms_norm_bwd_w_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "rms_norm_bwd_w_sums")) set_native_rms_norm_bwd_w_sums_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "rms_norm_bwd_x_w")) set_native_rms_norm_bwd_x_w_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "rms_norm_bwd_x_w_sums")) set_native_rms_norm_bwd_x_w_sums_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "rope")) set_native_rope_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "rope_bwd_x")) set_native_rope_bwd_x_skeleton(skeleton, bwd_dt);
	else if (!strcmp(op_name, "copy_to_seq_context")) set_native_copy_to_seq_context_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "swiglu")) set_native_swiglu_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "swiglu_bwd_x")) set_native_swiglu_bwd_x_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "softmax")) set_native_softmax_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "cross_entropy_loss")) set_native_cross_entropy_loss_skeleton(skeleton, bwd_dt);
	else if (!strcmp(op_name, "softmax_cross_entropy")) set_native_softmax_cross_entropy_skeleton(skeleton, fwd_dt, bwd_dt);
	else if (!strcmp(op_name, "select_experts")) set_native_select_experts_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "softmax_argmax")) set_native_softmax_argmax_skeleton(skeleton, fwd_dt);
	else if (!strcmp(op_name, "swiglu_ffn_fp8")) set_native_swiglu_ffn_fp8_skeleton(skeleton);
	else if (!strcmp(op_name, "swiglu_ffn_fp8_bwd")) set_native_swiglu_ffn_fp8_bwd_skeleton(skeleton);
	else {
		printf("Cannot set skeleton, unknown op: %s, with fwd_dt: %s, bwd_dt: %s\n", op_name,
		       dataflow_datatype_as_string(fwd_dt), dataflow_datatype_as_string(bwd_dt));
		return -1;
	}
	return 0;
}

/* ---- registration ---------------------------------------------------------------------- */

typedef enum { KEY_FWD, KEY_BWD, KEY_PAIR, KEY_HALF, KEY_ONE } Key_Kind;   /* KEY_HALF: fp16 and bf16 inputs only; KEY_ONE: a single identity */

typedef struct {
	const char * op;          /* skeleton family == exported symbol "dataflow_b200_<op>" */
	Key_Kind kind;            /* which datatypes enumerate the family */
	bool needs_workspace;     /* give the op an init function that allocates per-handle scratch */
} Op_Family;

/* The reference registers 54 identities (set_native_op_skeletons.c:13-39): all of them are here. Added: the 5
 * copy_to_seq_context identities (the reference has the skeleton, the wrapper and the kernels but leaves them out of
 * its registration list), 5 select_experts identities (kernels only in the reference) and the 7 datatype pairs of
 * the fused softmax+cross-entropy op, 2 softmax_argmax identities (fp16 / bf16 -> fp32), the FP8 FFN forward and backward, the 7
 * pairs of rms_norm_bwd_w_sums (the weight gradient written as fp32 column sums for a data-parallel exchange), and the 7 + 7 pairs of
 * rms_norm_bwd_x_w and rms_norm_bwd_x_w_sums (input and weight gradient of the norm in one pass over X and dY): 96 in total. */
static const Op_Family FAMILIES[] = {
	{"embedding", KEY_FWD, false},      {"copy_to_seq_context", KEY_FWD, false}, {"select_experts", KEY_FWD, false},
	{"rms_norm", KEY_FWD, false},       {"rms_norm_bwd_x", KEY_PAIR, false}, {"rms_norm_bwd_w", KEY_PAIR, true},
	{"rms_norm_bwd_w_sums", KEY_PAIR, true},
	{"rms_norm_bwd_x_w", KEY_PAIR, true}, {"rms_norm_bwd_x_w_sums", KEY_PAIR, true},
	{"rope", KEY_FWD, false},           {"rope_bwd_x", KEY_BWD, false},
	{"swiglu", KEY_FWD, false},         {"swiglu_bwd_x", KEY_PAIR, false},
	{"softmax", KEY_PAIR, false},       {"cross_entropy_loss", KEY_BWD, false},
	{"softmax_cross_entropy", KEY_PAIR, true},
	{"softmax_argmax", KEY_HALF, false},
	{"swiglu_ffn_fp8", KEY_ONE, true},  {"swiglu_ffn_fp8_bwd", KEY_ONE, true},
};

static const DataflowDatatype FWD_DTS[5] = {DATAFLOW_FP32, DATAFLOW_FP16, DATAFLOW_BF16, DATAFLOW_FP8E4M3, DATAFLOW_FP8E5M2};
static const DataflowDatatype BWD_DTS[3] = {DATAFLOW_FP32, DATAFLOW_FP16, DATAFLOW_BF16};
static const DataflowDatatype PAIR_FWD[7] = {DATAFLOW_FP32, DATAFLOW_FP16, DATAFLOW_BF16, DATAFLOW_FP8E4M3, DATAFLOW_FP8E4M3, DATAFLOW_FP8E5M2, DATAFLOW_FP8E5M2};
static const DataflowDatatype PAIR_BWD[7] = {DATAFLOW_FP32, DATAFLOW_FP16, DATAFLOW_BF16, DATAFLOW_FP16, DATAFLOW_BF16, DATAFLOW_FP16, DATAFLOW_BF16};

#define MAX_REGISTERED 128

int register_native_ops(Dataflow_Handle * dataflow_handle, char * native_function_code_filename, char * native_function_config_filename) {
	(void) native_function_config_filename;
	if (!dataflow_handle || !dataflow_handle->register_external_code) {
		fprintf(stderr, "Error: register_native_ops needs an initialised handle\n");
		return -1;
	}
	/* A caller written against the reference passes its cubin and launch-config library here
	 * (register_native_ops(&handle, "lib/cuda_kernels.cubin", "lib/cuda_kernels_config.so")). The ops of this library live in this
	 * shared object, so a path that is not a loadable shared object exporting them -- a cubin, a missing file, another library -- is
	 * replaced by this library's own path, with a one-line notice. */
	char self_path[4096];
	char * lib = native_function_code_filename;
	bool use_self = !lib;
	if (lib) {
		void * probe = dlopen(lib, RTLD_LAZY | RTLD_LOCAL);
		if (!probe || !dlsym(probe, "dataflow_b200_rms_norm")) use_self = true;
		if (probe) dlclose(probe);
		if (use_self) fprintf(stderr, "Notice: register_native_ops: %s does not export this library's ops; registering them from this library instead\n", lib);
	}
	if (use_self) {
		Dl_info info;
		if (!dladdr((void *) &register_native_ops, &info) || !info.dli_fname) {
			fprintf(stderr, "Error: cannot locate the shared object that holds the ops\n");
			return -1;
		}
		snprintf(self_path, sizeof(self_path), "%s", info.dli_fname);
		lib = self_path;
	}

	Op_Skeleton * skeletons = (Op_Skeleton *) calloc(MAX_REGISTERED, sizeof(Op_Skeleton));
	char ** symbols = (char **) calloc(MAX_REGISTERED, sizeof(char *));
	char ** init_symbols = (char **) calloc(MAX_REGISTERED, sizeof(char *));
	if (!skeletons || !symbols || !init_symbols) { free(skeletons); free(symbols); free(init_symbols); return -1; }

	int n = 0;
	for (size_t f = 0; f < sizeof(FAMILIES) / sizeof(FAMILIES[0]); f++) {
		const Op_Family * fam = &FAMILIES[f];
		const int variants = fam->kind == KEY_FWD ? 5 : fam->kind == KEY_BWD ? 3 : fam->kind == KEY_HALF ? 2 : fam->kind == KEY_ONE ? 1 : 7;
		for (int v = 0; v < variants && n < MAX_REGISTERED; v++, n++) {
			const DataflowDatatype fwd = fam->kind == KEY_FWD ? FWD_DTS[v] : fam->kind == KEY_PAIR ? PAIR_FWD[v] : fam->kind == KEY_HALF ? FWD_DTS[1 + v] : DATAFLOW_NONE;
			const DataflowDatatype bwd = fam->kind == KEY_BWD ? BWD_DTS[v] : fam->kind == KEY_PAIR ? PAIR_BWD[v] : DATAFLOW_NONE;
			set_native_op_skeleton(&skeletons[n], (char *) fam->op, fwd, bwd);
			symbols[n] = (char *) malloc(FUNC_SYMBOL_MAX_LEN);
			snprintf(symbols[n], FUNC_SYMBOL_MAX_LEN, "dataflow_b200_%s", fam->op);
			if (fam->needs_workspace) {
				init_symbols[n] = (char *) malloc(FUNC_SYMBOL_MAX_LEN);
				snprintf(init_symbols[n], FUNC_SYMBOL_MAX_LEN, "dataflow_b200_workspace_init");
			}
		}
	}

	const int added = dataflow_handle->register_external_code(dataflow_handle, lib, n, skeletons, symbols, init_symbols);
	if (added != n) fprintf(stderr, "WARNING: failed to register all native ops, expected %d functions, got %d...\n", n, added);

	for (int i = 0; i < n; i++) { free(symbols[i]); free(init_symbols[i]); }
	free(symbols); free(init_symbols); free(skeletons);
	return added;
}
