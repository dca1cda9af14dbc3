/*
 * A C caller written the way programs against als244/dataflow_lib are written (its test mains: init_cuda_dataflow_handle,
 * register_native_ops, alloc_mem, submit_inbound_transfer, submit_<op>, submit_outbound_transfer, sync_stream), compiled
 * against this repository's headers and linked with libdataflow_b200.so only. It runs RMSNorm -> SwiGLU on the GPU and
 * checks the results against the same arithmetic done here on the host in double precision (bf16 tolerance: 1e-2 of
 * max(|ref|, rms(ref))). Exit status 0 = every check passed. With the argument "link" it only proves that the program
 * links and the library loads (no device needed).
 */
#include "dataflow_api.h"
#include "dataflow_transformer.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float uniform(unsigned * state) {              /* small LCG: values in (-1, 1) */
	*state = *state * 1664525u + 1013904223u;
	return ((float) (*state >> 8) / 8388608.0f) - 1.0f;
}

static int check(const char * what, const uint16_t * got, const double * ref, long n) {
	double ss = 0.0;
	for (long i = 0; i < n; i++) ss += ref[i] * ref[i];
	const double rms = sqrt(ss / (double) n);
	for (long i = 0; i < n; i++) {
		const double g = (double) solo_bf16_to_fp32(got[i]);
		const double tol = 1e-2 * fmax(fabs(ref[i]), rms);
		if (!(fabs(g - ref[i]) <= tol)) { fprintf(stderr, "%s: element %ld is %g, expected %g\n", what, i, g, ref[i]); return 1; }
	}
	printf("%s: %ld elements within tolerance\n", what, n);
	return 0;
}

int main(int argc, char ** argv) {
	if (argc > 1 && !strcmp(argv[1], "link")) {
		Op_Skeleton sk;
		set_native_rms_norm_skeleton(&sk, DATAFLOW_BF16);
		printf("linked; %s has %d arguments\n", sk.header.op_nickname, sk.header.num_args);
		if (sk.header.num_args != 8) return 1;
		/* the external-op identities and the head caller are reachable from C as well; a call without its containers is refused */
		Op_Skeleton mm;
		set_external_matmul_skeleton(&mm);
		Transformer_Head head = { DATAFLOW_BF16, DATAFLOW_BF16, DATAFLOW_FP32, 1e-5f, { 128, 64 }, NULL, NULL, NULL };
		printf("%s has %d arguments; head of %d x %d\n", mm.header.op_nickname, mm.header.num_args, head.embedding_config.vocab_size,
		       head.embedding_config.embedding_size);
		const int refused = submit_transformer_head(NULL, 0, 1, NULL, &head, NULL, NULL, NULL, NULL, NULL, NULL);
		return (mm.header.num_args == 19 && refused == -1) ? 0 : 1;
	}
	const int rows = 512, cols = 1024, ffn = 2048;
	const float eps = 1e-5f;
	Dataflow_Handle handle;
	if (init_cuda_dataflow_handle(&handle, COMPUTE_CUDA, 0, 0, 0, 2, NULL, NULL)) { fprintf(stderr, "handle init failed\n"); return 1; }
	const int n_ops = register_native_ops(&handle, NULL, NULL);
	if (n_ops < 54) { fprintf(stderr, "only %d ops registered\n", n_ops); return 1; }

	const size_t xb = (size_t) rows * cols * 2, gb = (size_t) rows * ffn * 2;
	uint16_t * hX = malloc(xb), * hW = malloc(cols * 2), * hY = malloc(xb), * hG = malloc(gb), * hU = malloc(gb), * hS = malloc(gb);
	float * h_rms = malloc(rows * 4), * h_ws = malloc(rows * 4);
	unsigned st = 12345u;
	for (long i = 0; i < (long) rows * cols; i++) hX[i] = solo_fp32_to_bf16(2.0f * uniform(&st));
	for (int i = 0; i < cols; i++) hW[i] = solo_fp32_to_bf16(1.0f + 0.1f * uniform(&st));
	for (long i = 0; i < (long) rows * ffn; i++) { hG[i] = solo_fp32_to_bf16(3.0f * uniform(&st)); hU[i] = solo_fp32_to_bf16(2.0f * uniform(&st)); }

	/* one allocation, sub-allocated by the caller (256-byte aligned pieces), as the reference's programs do */
	const size_t total = 3 * xb + 3 * gb + 2 * 4096 + 2 * (size_t) rows * 4 + 10 * 256;
	char * base = handle.alloc_mem(&handle, total);
	if (!base) { fprintf(stderr, "alloc_mem failed\n"); return 1; }
	size_t off = 0;
#define TAKE(bytes) (base + off); off += (((size_t) (bytes)) + 255) & ~(size_t) 255
	void * dX = TAKE(xb); void * dY = TAKE(xb); void * dW = TAKE(cols * 2);
	void * dG = TAKE(gb); void * dU = TAKE(gb); void * dS = TAKE(gb);
	float * d_ws = (float *) TAKE(rows * 4); float * d_rms = (float *) TAKE(rows * 4);
	void * dXg = TAKE(xb); void * dWg = TAKE(cols * 2);                       /* gradients of the norm's input and weight */
	uint16_t * hXg = calloc(1, xb), * hWg = calloc(1, cols * 2);

	int rc = 0;
	rc |= handle.submit_inbound_transfer(&handle, 0, dX, hX, xb);
	rc |= handle.submit_inbound_transfer(&handle, 0, dW, hW, cols * 2);
	rc |= handle.submit_inbound_transfer(&handle, 0, dG, hG, gb);
	rc |= handle.submit_inbound_transfer(&handle, 0, dU, hU, gb);
	rc |= submit_rms_norm(&handle, 0, DATAFLOW_BF16, rows, cols, eps, dW, dX, dY, d_ws, d_rms);
	rc |= submit_swiglu(&handle, 0, DATAFLOW_BF16, rows, ffn, dG, dU, dS);
	/* the norm's backward in one pass (this library's rms_norm_bwd_x_w), with the norm's own output standing in for the upstream
	 * gradient; both gradient buffers start at zero */
	rc |= handle.submit_inbound_transfer(&handle, 0, dXg, hXg, xb);
	rc |= handle.submit_inbound_transfer(&handle, 0, dWg, hWg, cols * 2);
	rc |= submit_rms_norm_bwd_x_w(&handle, 0, DATAFLOW_BF16, DATAFLOW_BF16, rows, cols, eps, d_ws, d_rms, dW, dX, dY, dXg, dWg);
	/* results leave on the second stream, behind a dependency on the compute stream */
	rc |= handle.submit_dependency(&handle, 1, handle.get_stream_state(&handle, 0));
	rc |= handle.submit_outbound_transfer(&handle, 1, hY, dY, xb);
	rc |= handle.submit_outbound_transfer(&handle, 1, hS, dS, gb);
	rc |= handle.submit_outbound_transfer(&handle, 1, h_rms, d_rms, rows * 4);
	rc |= handle.submit_outbound_transfer(&handle, 1, h_ws, d_ws, rows * 4);
	rc |= handle.submit_outbound_transfer(&handle, 1, hXg, dXg, xb);
	rc |= handle.submit_outbound_transfer(&handle, 1, hWg, dWg, cols * 2);
	rc |= handle.sync_stream(&handle, 1);
	if (rc) { fprintf(stderr, "a submission failed\n"); return 1; }

	double * ref = malloc((size_t) rows * (cols > ffn ? cols : ffn) * sizeof(double));
	int bad = 0;
	for (int r = 0; r < rows; r++) {
		double ss = 0.0, wsum = 0.0;
		for (int c = 0; c < cols; c++) { const double x = solo_bf16_to_fp32(hX[(long) r * cols + c]); ss += x * x; wsum += x * solo_bf16_to_fp32(hW[c]); }
		const double rinv = 1.0 / sqrt(ss / cols + eps);
		for (int c = 0; c < cols; c++) ref[(long) r * cols + c] = solo_bf16_to_fp32(hX[(long) r * cols + c]) * rinv * solo_bf16_to_fp32(hW[c]);
		if (fabs(h_rms[r] - rinv) > 1e-5 * rinv || fabs(h_ws[r] - wsum) > 1e-4 * fmax(fabs(wsum), 1.0)) { fprintf(stderr, "row %d statistics: %g %g, expected %g %g\n", r, h_rms[r], h_ws[r], rinv, wsum); bad = 1; break; }
	}
	bad |= check("rms_norm", hY, ref, (long) rows * cols);
	{	/* dW[c] = sum_r dY[r,c] x[r,c] r_r and dX[r,c] = dY[r,c] (w_c r_r - x[r,c] r_r^3 ws_r / n), from the device's own Y, rms and ws */
		double * dw = calloc(cols, sizeof(double)), * dx = malloc((size_t) rows * cols * sizeof(double));
		for (int r = 0; r < rows; r++)
			for (int c = 0; c < cols; c++) {
				const double x = solo_bf16_to_fp32(hX[(long) r * cols + c]), g = solo_bf16_to_fp32(hY[(long) r * cols + c]), rr = h_rms[r];
				dw[c] += g * x * rr;
				dx[(long) r * cols + c] = g * (solo_bf16_to_fp32(hW[c]) * rr - x * rr * rr * rr / cols * h_ws[r]);
			}
		bad |= check("rms_norm_bwd_x_w dX", hXg, dx, (long) rows * cols);
		double scale = 0.0;
		for (int c = 0; c < cols; c++) scale = fmax(scale, fabs(dw[c]));
		for (int c = 0; c < cols && !bad; c++)
			if (fabs(solo_bf16_to_fp32(hWg[c]) - dw[c]) > 1e-2 * fmax(fabs(dw[c]), 0.05 * scale)) { fprintf(stderr, "rms_norm_bwd_x_w dW[%d]: %g, expected %g\n", c, solo_bf16_to_fp32(hWg[c]), dw[c]); bad = 1; }
		free(dw); free(dx);
	}
	for (long i = 0; i < (long) rows * ffn; i++) { const double g = solo_bf16_to_fp32(hG[i]); ref[i] = g / (1.0 + exp(-g)) * solo_bf16_to_fp32(hU[i]); }
	bad |= check("swiglu", hS, ref, (long) rows * ffn);

	handle.free_mem(&handle, base);
	destroy_cuda_dataflow_handle(&handle);
	printf(bad ? "FAILED\n" : "C caller: %d ops registered, all checks passed\n", n_ops);
	return bad;
}
