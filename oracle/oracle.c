/*
 * oracle.c -- CPU restatement of the arithmetic of als244/dataflow_lib's native transformer
 * op kernels. TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA kernels and the timed
 * "CPU port" baseline of the benchmark; nothing in the product path links or calls it.
 *
 * The reference implements these ops only as CUDA kernels (there is no host version), so each
 * function below restates one kernel, rounding point by rounding point, citing the lines it
 * follows. Pinning: the reference's tests hold no expected outputs for these ops; the oracle
 * is pinned (a) by the fingerprint/struct-size known answers in tests/golden, which come from
 * the reference's own host sources compiled unchanged, and (b) on a GPU box by running the
 * reference's kernels themselves, compiled for sm_100a from the reference tree into
 * oracle/_ref (see oracle/Makefile), on the same inputs (tests/test_reference_kernels_gpu.py).
 *
 * Conventions: tensors are row-major and contiguous; `dt` arguments are DataflowDatatype
 * values (3 fp32, 4 fp16, 5 bf16, 6 fp8e4m3, 7 fp8e5m2); n_threads host threads split the rows.
 * Transcendentals are libm's (the reference build uses --use_fast_math approximations of the
 * same functions); float expressions are evaluated without fused multiply-add unless noted
 * (compile with -ffp-contract=off).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { DT_FP32 = 3, DT_FP16 = 4, DT_BF16 = 5, DT_E4M3 = 6, DT_E5M2 = 7 };

/* ------------------------------------------------------------------------------------------
 * element conversions (round-to-nearest-even; fp8 saturates to the largest finite value, as
 * the CUDA conversions __float2bfloat16 / __float2half / __nv_fp8_e4m3(float) do)
 * ---------------------------------------------------------------------------------------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float oracle_bf16_to_f32(uint16_t h) { return u2f((uint32_t) h << 16); }

uint16_t oracle_f32_to_bf16(float f) {
	uint32_t u = f2u(f);
	if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
	u += 0x7fffu + ((u >> 16) & 1u);
	return (uint16_t) (u >> 16);
}

/* Generic small-float encoder: exp_bits/man_bits with IEEE-style bias, subnormals, RNE.
 * `max_finite_bits` is the encoding of the largest finite magnitude; `has_inf` selects whether
 * overflow goes to infinity (fp16) or saturates (fp8, satfinite). */
static uint32_t encode_small(float f, int exp_bits, int man_bits, uint32_t max_finite_bits, int has_inf, uint32_t nan_bits) {
	const uint32_t u = f2u(f);
	const uint32_t sign = (u >> 31) << (exp_bits + man_bits);
	const uint32_t a = u & 0x7fffffffu;
	if (a > 0x7f800000u) return sign | nan_bits;
	const int bias = (1 << (exp_bits - 1)) - 1;
	if (a == 0x7f800000u) return sign | (has_inf ? (uint32_t) (((1u << exp_bits) - 1) << man_bits) : max_finite_bits);
	if (a == 0) return sign;
	int e = (int) (a >> 23) - 127;
	uint32_t m = (a & 0x7fffffu) | 0x800000u;            /* 24-bit significand */
	if ((a >> 23) == 0) { e = -126; m = a & 0x7fffffu; } /* fp32 subnormal: far below any target subnormal */
	int shift = 23 - man_bits;
	uint32_t base;
	if (e < 1 - bias) { shift += (1 - bias) - e; base = 0; }
	else { base = (uint32_t) (e + bias) << man_bits; m &= 0x7fffffu; }
	uint32_t q;
	if (shift > 31) q = 0;
	else {
		q = m >> shift;
		const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
		if (rem > half || (rem == half && (q & 1u))) q++;
	}
	uint32_t r = base + q;
	if (r > max_finite_bits) r = has_inf ? (uint32_t) (((1u << exp_bits) - 1) << man_bits) : max_finite_bits;
	return sign | r;
}

static float decode_small(uint32_t v, int exp_bits, int man_bits, int ieee_specials) {
	const uint32_t sign = (v >> (exp_bits + man_bits)) & 1u;
	const uint32_t e = (v >> man_bits) & ((1u << exp_bits) - 1), m = v & ((1u << man_bits) - 1);
	const int bias = (1 << (exp_bits - 1)) - 1;
	float r;
	if (ieee_specials && e == (1u << exp_bits) - 1) r = m ? NAN : INFINITY;
	else if (!ieee_specials && e == (1u << exp_bits) - 1 && m == (1u << man_bits) - 1) r = NAN;   /* e4m3: only S.1111.111 is NaN */
	else if (e == 0) r = ldexpf((float) m, 1 - bias - man_bits);
	else r = ldexpf((float) (m | (1u << man_bits)), (int) e - bias - man_bits);
	return sign ? -r : r;
}

uint16_t oracle_f32_to_fp16(float f) { return (uint16_t) encode_small(f, 5, 10, 0x7bff, 1, 0x7e00); }
float oracle_fp16_to_f32(uint16_t h) { return decode_small(h, 5, 10, 1); }
uint8_t oracle_f32_to_e4m3(float f) { return (uint8_t) encode_small(f, 4, 3, 0x7e, 0, 0x7f); }
float oracle_e4m3_to_f32(uint8_t v) { return decode_small(v, 4, 3, 0); }
uint8_t oracle_f32_to_e5m2(float f) { return (uint8_t) encode_small(f, 5, 2, 0x7b, 0, 0x7f); }
float oracle_e5m2_to_f32(uint8_t v) { return decode_small(v, 5, 2, 1); }

int oracle_sizeof(int dt) { return dt == DT_FP32 ? 4 : (dt == DT_FP16 || dt == DT_BF16) ? 2 : (dt == DT_E4M3 || dt == DT_E5M2) ? 1 : 0; }

static inline float ld(int dt, const void * p, size_t i) {
	switch (dt) {
		case DT_FP32: return ((const float *) p)[i];
		case DT_BF16: return oracle_bf16_to_f32(((const uint16_t *) p)[i]);
		case DT_FP16: return oracle_fp16_to_f32(((const uint16_t *) p)[i]);
		case DT_E4M3: return oracle_e4m3_to_f32(((const uint8_t *) p)[i]);
		default:      return oracle_e5m2_to_f32(((const uint8_t *) p)[i]);
	}
}
static inline void st(int dt, void * p, size_t i, float v) {
	switch (dt) {
		case DT_FP32: ((float *) p)[i] = v; break;
		case DT_BF16: ((uint16_t *) p)[i] = oracle_f32_to_bf16(v); break;
		case DT_FP16: ((uint16_t *) p)[i] = oracle_f32_to_fp16(v); break;
		case DT_E4M3: ((uint8_t *) p)[i] = oracle_f32_to_e4m3(v); break;
		default:      ((uint8_t *) p)[i] = oracle_f32_to_e5m2(v); break;
	}
}
/* value after a store to `dt` and a load back */
static inline float rnd(int dt, float v) {
	switch (dt) {
		case DT_FP32: return v;
		case DT_BF16: return oracle_bf16_to_f32(oracle_f32_to_bf16(v));
		case DT_FP16: return oracle_fp16_to_f32(oracle_f32_to_fp16(v));
		case DT_E4M3: return oracle_e4m3_to_f32(oracle_f32_to_e4m3(v));
		default:      return oracle_e5m2_to_f32(oracle_f32_to_e5m2(v));
	}
}
/* a (op) b computed exactly and rounded ONCE to `dt` (what a native bf16/fp16 instruction gives) */
static inline float rnd_d(int dt, double v) {
	if (dt == DT_FP32) return (float) v;
	/* double -> float can double-round only within 2^-29 of a tie of the narrow type; nudge via sticky bit */
	float f = (float) v;
	if ((double) f != v) {
		uint32_t u = f2u(f);
		if (((double) f > v) == (f > 0)) u -= 1;   /* truncate toward zero ... */
		u |= 1u;                                   /* ... and make it sticky-odd so the next rounding sees "inexact" */
		f = u2f(u);
	}
	return rnd(dt, f);
}

void oracle_convert(int to_dt, void * to, int from_dt, const void * from, long n) {
	for (long i = 0; i < n; i++) st(to_dt, to, (size_t) i, ld(from_dt, from, (size_t) i));
}

/* ------------------------------------------------------------------------------------------
 * row-parallel driver
 * ---------------------------------------------------------------------------------------- */

typedef void (*Row_Fn)(long row_begin, long row_end, void * ctx);
typedef struct { Row_Fn fn; void * ctx; long begin, end; } Row_Job;

static void * row_worker(void * p) { Row_Job * j = (Row_Job *) p; j->fn(j->begin, j->end, j->ctx); return NULL; }

static void for_rows(long n_rows, int n_threads, Row_Fn fn, void * ctx) {
	if (n_threads < 1) n_threads = 1;
	if (n_threads > 256) n_threads = 256;
	if (n_threads > n_rows) n_threads = n_rows > 0 ? (int) n_rows : 1;
	if (n_threads == 1) { fn(0, n_rows, ctx); return; }
	pthread_t th[256];
	Row_Job jobs[256];
	int ok[256];
	const long per = (n_rows + n_threads - 1) / n_threads;
	for (int t = 0; t < n_threads; t++) {
		jobs[t] = (Row_Job){fn, ctx, t * per, (t + 1) * per < n_rows ? (t + 1) * per : n_rows};
		ok[t] = 0;
		if (jobs[t].begin >= jobs[t].end) continue;
		if (t < n_threads - 1 && pthread_create(&th[t], NULL, row_worker, &jobs[t]) == 0) ok[t] = 1;
		else row_worker(&jobs[t]);
	}
	for (int t = 0; t < n_threads; t++) if (ok[t]) pthread_join(th[t], NULL);
}

/* Sum of 32 values in the order of a __shfl_down_sync tree (offsets 16, 8, 4, 2, 1) as seen by
 * lane 0: the pattern of every warp reduction in the reference kernels. */
static inline float tree32(float * v) {
	for (int off = 16; off > 0; off >>= 1)
		for (int i = 0; i < off; i++) v[i] = v[i] + v[i + off];
	return v[0];
}

/* ------------------------------------------------------------------------------------------
 * RMSNorm forward -- src/ops/nvidia/norm/rms_norm.cu:280-412 (bf16; :4,143 fp32/fp16 alike)
 * 1024 threads stride over the row accumulating w*x and x*x in fp32 (nvcc contracts both
 * updates into fma), warp tree, 32-slot tree; r = rsqrt(ss/n + eps); out = T((x*r)*w).
 * ---------------------------------------------------------------------------------------- */

typedef struct { int dt, n_cols; float eps; const void * w, * X; void * out; float * ws, * rms; } Rms_Fwd;

static void rms_fwd_rows(long r0, long r1, void * p) {
	Rms_Fwd * a = (Rms_Fwd *) p;
	const int n = a->n_cols;
	float * part_ws = (float *) malloc(2 * 1024 * sizeof(float)), * part_ss = part_ws + 1024;
	for (long r = r0; r < r1; r++) {
		const size_t base = (size_t) r * n;
		for (int t = 0; t < 1024; t++) {
			float ws = 0.0f, ss = 0.0f;
			for (int i = t; i < n; i += 1024) {
				const float x = ld(a->dt, a->X, base + i);
				ws = fmaf(ld(a->dt, a->w, i), x, ws);
				ss = fmaf(x, x, ss);
			}
			part_ws[t] = ws; part_ss[t] = ss;
		}
		float wws[32], wss[32];
		for (int w = 0; w < 32; w++) { wws[w] = tree32(part_ws + 32 * w); wss[w] = tree32(part_ss + 32 * w); }
		const float ws = tree32(wws), ss = tree32(wss);
		const float rr = 1.0f / sqrtf(ss / (float) n + a->eps);
		if (a->ws) a->ws[r] = ws;
		if (a->rms) a->rms[r] = rr;
		for (int i = 0; i < n; i++) st(a->dt, a->out, base + i, (ld(a->dt, a->X, base + i) * rr) * ld(a->dt, a->w, i));
	}
	free(part_ws);
}

void oracle_rms_norm(int dt, int n_rows, int n_cols, float eps, const void * w, const void * X, void * out,
                     float * weighted_sums, float * rms_vals, int n_threads) {
	Rms_Fwd a = {dt, n_cols, eps, w, X, out, weighted_sums, rms_vals};
	for_rows(n_rows, n_threads, rms_fwd_rows, &a);
}

/* ------------------------------------------------------------------------------------------
 * RMSNorm backward-x -- src/ops/nvidia/norm/rms_norm_bwd_x.cu:243-252
 *   deriv = (w*r) - (((x*r^3)/n) * ws)          fp32
 *   dX   += dY * B(deriv)                        in the backward type B
 * fused == 1: one rounding of dX + dY*B(deriv) -- the fma.rn.bf16x2 / f16x2 the reference binary executes (its outputs
 *             in tests/golden/reference_vectors.npz match this variant bit for bit);
 * fused == 0: product and sum rounded to B separately (the C++ expression read literally), kept for comparison.
 * For B = fp32 the update is a single fmaf either way.
 * ---------------------------------------------------------------------------------------- */

typedef struct { int fdt, bdt, n_cols, fused; const float * ws, * rms; const void * w, * X, * dY; void * dX; } Rms_Bx;

static void rms_bx_rows(long r0, long r1, void * p) {
	Rms_Bx * a = (Rms_Bx *) p;
	const int n = a->n_cols;
	for (long r = r0; r < r1; r++) {
		const size_t base = (size_t) r * n;
		const float rr = a->rms[r], ws = a->ws[r];
		const float r3 = rr * rr * rr;
		for (int i = 0; i < n; i++) {
			const float x = ld(a->fdt, a->X, base + i);
			const float deriv = (ld(a->fdt, a->w, i) * rr) - (((x * r3) / (float) n) * ws);
			const float g = ld(a->bdt, a->dY, base + i), d = ld(a->bdt, a->dX, base + i);
			float o;
			if (a->bdt == DT_FP32) o = fmaf(g, deriv, d);
			else if (a->fused) o = rnd_d(a->bdt, (double) d + (double) g * (double) rnd(a->bdt, deriv));
			else o = rnd(a->bdt, d + rnd(a->bdt, g * rnd(a->bdt, deriv)));
			st(a->bdt, a->dX, base + i, o);
		}
	}
}

void oracle_rms_norm_bwd_x(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const float * weighted_sums, const float * rms_vals,
                           const void * w, const void * X, const void * dY, void * dX, int fused, int n_threads) {
	Rms_Bx a = {fwd_dt, bwd_dt, n_cols, fused, weighted_sums, rms_vals, w, X, dY, dX};
	for_rows(n_rows, n_threads, rms_bx_rows, &a);
}

/* ------------------------------------------------------------------------------------------
 * RMSNorm backward-w -- src/ops/nvidia/norm/rms_norm_bwd_w.cu:270-307
 * term(r,c) = f32(dY)*f32(x)*rms[r] in fp32 (left to right).
 * n_blocks == 0: exact-sum semantics: dW[c] = B(f32(dW[c]) + sum_r term) with the sum in fp64
 *                (the order-independent value the reference's atomics approximate).
 * n_blocks  > 0: emulation of the reference launch with that many blocks: each block sums its
 *                contiguous rows per column in fp32, and the blocks' B-rounded sums are added
 *                to dW one after the other in block order with a rounding to B per add (one
 *                of the orders the bf16 atomicAdd can take).
 * ---------------------------------------------------------------------------------------- */

typedef struct { int fdt, bdt, n_rows, n_cols, n_blocks; const float * rms; const void * X, * dY; void * dW; } Rms_Bw;

static void rms_bw_cols(long c0, long c1, void * p) {
	Rms_Bw * a = (Rms_Bw *) p;
	const int n = a->n_cols, R = a->n_rows;
	for (long c = c0; c < c1; c++) {
		if (a->n_blocks <= 0) {
			double s = 0.0;
			for (int r = 0; r < R; r++) s += (double) (ld(a->bdt, a->dY, (size_t) r * n + c) * ld(a->fdt, a->X, (size_t) r * n + c) * a->rms[r]);
			st(a->bdt, a->dW, c, (float) ((double) ld(a->bdt, a->dW, c) + s));
		} else {
			const int G = a->n_blocks < R ? a->n_blocks : R;
			float dw = ld(a->bdt, a->dW, c);
			for (int b = 0; b < G; b++) {
				int rows = R / G, off;
				const int rem = R % G;
				if (b < rem) { rows += 1; off = b * rows; } else off = b * rows + rem;
				float s = 0.0f;
				for (int r = off; r < off + rows; r++) s += ld(a->bdt, a->dY, (size_t) r * n + c) * ld(a->fdt, a->X, (size_t) r * n + c) * a->rms[r];
				dw = rnd(a->bdt, dw + rnd(a->bdt, s));
			}
			st(a->bdt, a->dW, c, dw);
		}
	}
}

void oracle_rms_norm_bwd_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const float * rms_vals, const void * X, const void * dY,
                           void * dW, int n_blocks, int n_threads) {
	Rms_Bw a = {fwd_dt, bwd_dt, n_rows, n_cols, n_blocks, rms_vals, X, dY, dW};
	for_rows(n_cols, n_threads, rms_bw_cols, &a);
}

/* ------------------------------------------------------------------------------------------
 * RoPE forward/backward -- src/ops/nvidia/attention/rope.cu:137-171, rope_bwd_x.cu:132-172
 * per even flat index i: d = i % head_dim, angle = powf(theta, -(d/head_dim)),
 * c = cosf(pos*angle), s = sinf(pos*angle); fwd (e,o) <- (c*e - s*o, c*o + s*e),
 * bwd (e,o) <- (c*e + s*o, -s*e + c*o); in place, one rounding to T per output.
 * ---------------------------------------------------------------------------------------- */

typedef struct { int dt, dim, head_dim, bwd; float theta; const int * pos; void * X; } Rope;

/* powf as its definition: the fp32 arguments' exact power, rounded once (libm's powf is within
 * 1 ulp of this but not always equal; the reference build's __powf is far looser). */
static inline float powf_once(float a, float b) { return (float) pow((double) a, (double) b); }

static void rope_rows(long r0, long r1, void * p) {
	Rope * a = (Rope *) p;
	for (long r = r0; r < r1; r++) {
		const float pos = (float) a->pos[r];
		for (int i = 0; i < a->dim; i += 2) {
			const int d = i % a->head_dim;
			const float angle = powf_once(a->theta, -1.0f * ((float) d / (float) a->head_dim));
			const float c = cosf(pos * angle), s = sinf(pos * angle);
			const size_t k = (size_t) r * a->dim + i;
			const float e = ld(a->dt, a->X, k), o = ld(a->dt, a->X, k + 1);
			if (!a->bwd) { st(a->dt, a->X, k, c * e - s * o); st(a->dt, a->X, k + 1, c * o + s * e); }
			else         { st(a->dt, a->X, k, c * e + s * o); st(a->dt, a->X, k + 1, -s * e + c * o); }
		}
	}
}

void oracle_rope(int dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta, const int * seq_positions,
                 void * X_q, void * X_k, int bwd, int n_threads) {
	const long tokens = (long) (N / (uint64_t) model_dim);
	Rope q = {dt, model_dim, head_dim, bwd, (float) theta, seq_positions, X_q};
	for_rows(tokens, n_threads, rope_rows, &q);
	if (num_kv_heads > 0) {
		Rope k = {dt, num_kv_heads * head_dim, head_dim, bwd, (float) theta, seq_positions, X_k};
		for_rows(tokens, n_threads, rope_rows, &k);
	}
}

/* ------------------------------------------------------------------------------------------
 * SwiGLU -- src/ops/nvidia/activations/swiglu.cu:58-65, swiglu_bwd_x.cu:68-77
 * ---------------------------------------------------------------------------------------- */

typedef struct { int fdt, bdt; long n_cols; const void * x1, * x3, * dY; void * out, * d1, * d3; } Swiglu;

static void swiglu_fwd_rows(long r0, long r1, void * p) {
	Swiglu * a = (Swiglu *) p;
	for (size_t i = (size_t) r0 * a->n_cols; i < (size_t) r1 * a->n_cols; i++) {
		const float x1 = ld(a->fdt, a->x1, i), x3 = ld(a->fdt, a->x3, i);
		const float silu = x1 / (1 + expf(-1 * x1));
		st(a->fdt, a->out, i, silu * x3);
	}
}
static void swiglu_bwd_rows(long r0, long r1, void * p) {
	Swiglu * a = (Swiglu *) p;
	for (size_t i = (size_t) r0 * a->n_cols; i < (size_t) r1 * a->n_cols; i++) {
		const float x1 = ld(a->fdt, a->x1, i), x3 = ld(a->fdt, a->x3, i), g = ld(a->bdt, a->dY, i);
		const float e = expf(-1 * x1);
		const float silu = x1 / (1 + e);
		st(a->bdt, a->d3, i, g * silu);
		st(a->bdt, a->d1, i, g * ((x3 * (1 + e + x1 * e)) / ((1 + e) * (1 + e))));
	}
}

void oracle_swiglu(int dt, int n_rows, int n_cols, const void * x_w1, const void * x_w3, void * out, int n_threads) {
	Swiglu a = {dt, dt, n_cols, x_w1, x_w3, NULL, out, NULL, NULL};
	for_rows(n_rows, n_threads, swiglu_fwd_rows, &a);
}
void oracle_swiglu_bwd_x(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void * x_w1, const void * x_w3, const void * dY,
                         void * dX_w1, void * dX_w3, int n_threads) {
	Swiglu a = {fwd_dt, bwd_dt, n_cols, x_w1, x_w3, dY, NULL, dX_w1, dX_w3};
	for_rows(n_rows, n_threads, swiglu_bwd_rows, &a);
}

/* ------------------------------------------------------------------------------------------
 * softmax -- src/ops/nvidia/loss/softmax.cu:273-407 (bf16; the other pairs alike, with the
 * working type W = the output type: :137-271 fp16, :409-544 fp8->fp16, ...)
 * One block of 32 warps per row. Warp w visits the 32-element groups w, w+32, w+64, ...
 *   pass 1: max in W (exact);
 *   pass 2: per group, e_j = expf(f32(W(x_j - max))) summed over the 32 lanes in shuffle-tree
 *           order, lane 0 adds the group sums one after the other in fp32; each warp's sum is
 *           stored as W, the 32 stored values are tree-summed in fp32 and the total stored as W;
 *   pass 3: out_j = W(e_j / total).
 * A ragged last group (n_cols % 32 != 0, which the reference does not support) is treated as
 * if its missing lanes contributed nothing.
 * Optional cross-entropy step and loss (labels != NULL):
 *   out[r, label] = W(out[r, label] - 1)      intended semantics of loss/cross_entropy.cu:33-44
 *   row_loss[r] = logf(total32) - (x_label - max)   in fp32, with total32 = the fp32 tree sum of the 32 warp sums BEFORE they
 *                 are rounded to W. No reference implementation exists (nothing in the reference computes a loss,
 *                 src/dataflow_models/dataflow_transformer/include/transformer_structs.h:148-149), so none of the reference's
 *                 roundings is owed to it except the one inside the exponentials it shares with the probabilities.
 * ---------------------------------------------------------------------------------------- */

typedef struct { int fdt, bdt, n_cols; const void * X; void * out; const uint32_t * labels; float * row_loss; int odt; uint32_t * arg_maxs; } Softmax;

static void softmax_rows(long r0, long r1, void * p) {
	Softmax * a = (Softmax *) p;
	const int n = a->n_cols, W = a->bdt;
	const int groups = (n + 31) / 32;
	for (long r = r0; r < r1; r++) {
		const size_t base = (size_t) r * n;
		float mx = -INFINITY;
		for (int i = 0; i < n; i++) { const float x = ld(a->fdt, a->X, base + i); if (x > mx) mx = x; }
		float warp_sums[32], warp_sums_f32[32];
		for (int w = 0; w < 32; w++) {
			float total = 0.0f;
			for (int g = w; g < groups; g += 32) {
				float lane[32];
				for (int l = 0; l < 32; l++) {
					const int i = g * 32 + l;
					lane[l] = i < n ? expf(rnd_d(W, (double) ld(a->fdt, a->X, base + i) - (double) mx)) : 0.0f;
				}
				total += tree32(lane);
			}
			warp_sums[w] = rnd(W, total);
			warp_sums_f32[w] = total;
		}
		const float total = rnd(W, tree32(warp_sums));
		for (int i = 0; i < n; i++)
			st(a->odt, a->out, base + i, expf(rnd_d(W, (double) ld(a->fdt, a->X, base + i) - (double) mx)) / total);
		if (a->arg_maxs) {                 /* the smallest index holding the maximum (the reference lets any such index win, :1057-1059) */
			uint32_t arg = 0xffffffffu;
			for (int i = n - 1; i >= 0; i--) if (ld(a->fdt, a->X, base + i) == mx) arg = (uint32_t) i;
			a->arg_maxs[r] = arg;
		}
		if (a->labels) {
			const uint32_t lab = a->labels[r];
			if (lab < (uint32_t) n) {
				st(W, a->out, base + lab, ld(W, a->out, base + lab) - 1.0f);
				if (a->row_loss) a->row_loss[r] = logf(tree32(warp_sums_f32)) - (ld(a->fdt, a->X, base + lab) - mx);
			} else if (a->row_loss) a->row_loss[r] = 0.0f;
		}
	}
}

void oracle_softmax(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void * X, void * out, int n_threads) {
	Softmax a = {fwd_dt, bwd_dt, n_cols, X, out, NULL, NULL, bwd_dt, NULL};
	for_rows(n_rows, n_threads, softmax_rows, &a);
}

/* softmax_fp16_fp32_kernel / softmax_bf16_fp32_kernel (loss/softmax.cu:965-1249): the same three passes with the scratch
 * (x - max, warp sums, total) held in the INPUT type, the probabilities stored unrounded in fp32, and the index of the
 * row maximum written to arg_maxs (optional). */
void oracle_softmax_fp32_out(int fwd_dt, int n_rows, int n_cols, const void * X, float * out, uint32_t * arg_maxs, int n_threads) {
	Softmax a = {fwd_dt, fwd_dt, n_cols, X, out, NULL, NULL, DT_FP32, arg_maxs};
	for_rows(n_rows, n_threads, softmax_rows, &a);
}

/* pred[r, labels[r]] -= 1 in the tensor's type -- intended semantics of loss/cross_entropy.cu:33-44 */
void oracle_cross_entropy_loss(int bwd_dt, int n_rows, int n_cols, void * pred, const uint32_t * labels) {
	for (int r = 0; r < n_rows; r++) {
		if (labels[r] >= (uint32_t) n_cols) continue;
		const size_t k = (size_t) r * n_cols + labels[r];
		st(bwd_dt, pred, k, ld(bwd_dt, pred, k) - 1.0f);
	}
}

/* softmax followed by the cross-entropy step, plus per-row losses and {sum, valid rows}. */
void oracle_softmax_cross_entropy(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void * logits, const uint32_t * labels,
                                  void * dlogits, float * row_loss, float * loss_sum, int n_threads) {
	float * losses = row_loss ? row_loss : (float *) malloc(sizeof(float) * (size_t) (n_rows > 0 ? n_rows : 1));
	Softmax a = {fwd_dt, bwd_dt, n_cols, logits, dlogits, labels, losses, bwd_dt, NULL};
	for_rows(n_rows, n_threads, softmax_rows, &a);
	if (loss_sum) {
		double s = 0.0; long cnt = 0;
		for (int r = 0; r < n_rows; r++) if (labels[r] < (uint32_t) n_cols) { s += (double) losses[r]; cnt++; }
		loss_sum[0] = (float) s; loss_sum[1] = (float) cnt;
	}
	if (!row_loss) free(losses);
}

/* ------------------------------------------------------------------------------------------
 * seeded inputs: counter-based (splitmix64) Box-Muller normals, so any slice of a tensor can be
 * generated independently and identically in C and in the tests.
 * ---------------------------------------------------------------------------------------- */

static inline uint64_t splitmix64(uint64_t x) {
	x += 0x9e3779b97f4a7c15ull;
	x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
	x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
	return x ^ (x >> 31);
}

typedef struct { int dt; uint64_t seed; float mean, std; void * out; long per_row; } Fill;

static void fill_rows(long r0, long r1, void * p) {
	Fill * a = (Fill *) p;
	for (size_t i = (size_t) r0 * a->per_row; i < (size_t) r1 * a->per_row; i++) {
		const uint64_t h1 = splitmix64(a->seed * 0x100000001b3ull + 2 * i), h2 = splitmix64(a->seed * 0x100000001b3ull + 2 * i + 1);
		const double u1 = ((double) (h1 >> 11) + 1.0) / 9007199254740993.0, u2 = (double) (h2 >> 11) / 9007199254740992.0;
		const double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
		st(a->dt, a->out, i, (float) (a->mean + a->std * z));
	}
}

/* out[i] = T(mean + std * z_i), z_i ~ N(0,1) a pure function of (seed, i). n = n_rows * per_row. */
void oracle_fill_normal(int dt, void * out, long n_rows, long per_row, uint64_t seed, float mean, float std, int n_threads) {
	Fill a = {dt, seed, mean, std, out, per_row};
	for_rows(n_rows, n_threads, fill_rows, &a);
}

void oracle_fill_labels(uint32_t * out, long n, uint64_t seed, uint32_t n_classes) {
	for (long i = 0; i < n; i++) out[i] = (uint32_t) (splitmix64(seed * 0x100000001b3ull + (uint64_t) i) % n_classes);
}

/* ------------------------------------------------------------------------------------------
 * FP8-weight SwiGLU FFN (no counterpart in the reference: parity unpinned; this restatement IS the contract)
 *   row quantisation   q[r,k] = e4m3( x[r,k] * (448 / amax_r) ),  scale[r] = amax_r / 448   (1 for an all-zero row)
 *   projections        acc[m,n] = sum_k f32(A[m,k]) * f32(W[n,k])       weights stored [out, in]; sum in fp64 here
 *   gate/up epilogue   g = (acc_g * sa[m]) * sg[n];  u = (acc_u * sa[m]) * su[n];  h = bf16( (g / (1 + exp(-g))) * u )
 *   plain epilogue     out = bf16( (acc * sa[m]) * sw[n] )
 * ---------------------------------------------------------------------------------------- */

typedef struct { int n_cols; const uint16_t * X; const float * col; uint8_t * Q; float * scales; } Quant;

static void quant_rows(long r0, long r1, void * p) {
	Quant * a = (Quant *) p;
	for (long r = r0; r < r1; r++) {
		const uint16_t * x = a->X + (size_t) r * a->n_cols;
		float amax = 0.0f;
		for (int k = 0; k < a->n_cols; k++) { const float v = fabsf(oracle_bf16_to_f32(x[k]) * (a->col ? a->col[k] : 1.0f)); if (v > amax) amax = v; }
		const float inv = amax > 0.0f ? 448.0f / amax : 1.0f;
		a->scales[r] = amax > 0.0f ? amax / 448.0f : 1.0f;
		for (int k = 0; k < a->n_cols; k++)
			a->Q[(size_t) r * a->n_cols + k] = oracle_f32_to_e4m3((oracle_bf16_to_f32(x[k]) * (a->col ? a->col[k] : 1.0f)) * inv);
	}
}

/* col_factors (optional, n_cols floats): v = f32(x) * factor is what gets quantised (scales that sit on a contraction index) */
void oracle_quantize_rows_e4m3(int n_rows, int n_cols, const void * X_bf16, const float * col_factors, void * Q, float * scales, int n_threads) {
	Quant a = {n_cols, (const uint16_t *) X_bf16, col_factors, (uint8_t *) Q, scales};
	for_rows(n_rows, n_threads, quant_rows, &a);
}

/* mode 0 plain, 1 gate/up + SwiGLU (optionally saving g and u), 2 SwiGLU backward from saved g and u */
typedef struct { int N, K, mode; const uint8_t * A, * W0, * W1; const float * sa, * s0, * s1; uint16_t * out, * g_save, * u_save; const float * lut; } Gemm8;

static void gemm8_rows(long r0, long r1, void * p) {
	Gemm8 * a = (Gemm8 *) p;
	float * arow = (float *) malloc(sizeof(float) * (size_t) a->K);
	for (long m = r0; m < r1; m++) {
		for (int k = 0; k < a->K; k++) arow[k] = a->lut[a->A[(size_t) m * a->K + k]];
		for (int n = 0; n < a->N; n++) {
			const uint8_t * w0 = a->W0 + (size_t) n * a->K;
			double acc0 = 0.0, acc1 = 0.0;
			for (int k = 0; k < a->K; k++) acc0 += (double) (arow[k] * a->lut[w0[k]]);       /* products of two e4m3 values are exact in fp32 */
			if (a->mode == 1) {
				const uint8_t * w1 = a->W1 + (size_t) n * a->K;
				for (int k = 0; k < a->K; k++) acc1 += (double) (arow[k] * a->lut[w1[k]]);
				const float g = ((float) acc0 * a->sa[m]) * a->s0[n], u = ((float) acc1 * a->sa[m]) * a->s1[n];
				a->out[(size_t) m * a->N + n] = oracle_f32_to_bf16((g / (1.0f + expf(-g))) * u);
				if (a->g_save) { a->g_save[(size_t) m * a->N + n] = oracle_f32_to_bf16(g); a->u_save[(size_t) m * a->N + n] = oracle_f32_to_bf16(u); }
			} else if (a->mode == 2) {
				/* dh from the accumulator; gate and up gradients with the expressions of swiglu_bwd_x.cu:68-77 on the saved bf16 g, u */
				const float dh = (float) acc0 * a->sa[m];
				const float g = oracle_bf16_to_f32(a->g_save[(size_t) m * a->N + n]), u = oracle_bf16_to_f32(a->u_save[(size_t) m * a->N + n]);
				const float e = expf(-g);
				a->out[(size_t) m * 2 * a->N + n] = oracle_f32_to_bf16(dh * ((u * (1 + e + g * e)) / ((1 + e) * (1 + e))));
				a->out[(size_t) m * 2 * a->N + a->N + n] = oracle_f32_to_bf16(dh * (g / (1 + e)));
			} else {
				a->out[(size_t) m * a->N + n] = oracle_f32_to_bf16(((float) acc0 * a->sa[m]) * (a->s0 ? a->s0[n] : 1.0f));
			}
		}
	}
	free(arow);
}

static void gemm8(int M, int N, int K, int mode, const void * A, const float * sa, const void * W0, const float * s0, const void * W1,
                  const float * s1, void * out, void * g_save, void * u_save, int n_threads) {
	float lut[256];
	for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_to_f32((uint8_t) i);
	lut[0x7f] = 0.0f; lut[0xff] = 0.0f;          /* NaN codes never occur in quantised data */
	Gemm8 a = {N, K, mode, (const uint8_t *) A, (const uint8_t *) W0, (const uint8_t *) W1, sa, s0, s1, (uint16_t *) out, (uint16_t *) g_save, (uint16_t *) u_save, lut};
	for_rows(M, n_threads, gemm8_rows, &a);
}

void oracle_gemm_e4m3(int M, int N, int K, const void * A, const float * sa, const void * W, const float * sw, void * out_bf16, int n_threads) {
	gemm8(M, N, K, 0, A, sa, W, sw, NULL, NULL, out_bf16, NULL, NULL, n_threads);
}

void oracle_gemm_e4m3_swiglu(int M, int N, int K, const void * A, const float * sa, const void * Wg, const float * sg, const void * Wu,
                             const float * su, void * H_bf16, void * g_save_bf16, void * u_save_bf16, int n_threads) {
	gemm8(M, N, K, 1, A, sa, Wg, sg, Wu, su, H_bf16, g_save_bf16, u_save_bf16, n_threads);
}

/* dGU [M, 2N]: gate gradients in columns [0, N), up gradients in [N, 2N) */
void oracle_gemm_e4m3_swiglu_bwd(int M, int N, int K, const void * dOq, const float * s_rows, const void * WdownT, const void * g_saved_bf16,
                                 const void * u_saved_bf16, void * dGU_bf16, int n_threads) {
	gemm8(M, N, K, 2, dOq, s_rows, WdownT, NULL, NULL, NULL, dGU_bf16, (void *) g_saved_bf16, (void *) u_saved_bf16, n_threads);
}

/* ------------------------------------------------------------------------------------------
 * embedding and copy_to_seq_context: row copies
 * ---------------------------------------------------------------------------------------- */

/* src/ops/nvidia/preprocess/embedding.cu:3-24, intended semantics: output[t, :] = table[token_ids[t], :]
 * (the reference scales its element offsets by sizeof(element) while indexing typed pointers, :14-20). */
void oracle_embedding(int dt, int num_tokens, int embed_dim, const uint32_t * token_ids, const void * table, void * out) {
	const size_t row = (size_t) embed_dim * (size_t) oracle_sizeof(dt);
	for (int t = 0; t < num_tokens; t++)
		memcpy((uint8_t *) out + (size_t) t * row, (const uint8_t *) table + (size_t) token_ids[t] * row, row);
}

/* src/ops/nvidia/attention/copy_to_seq_context.cu:3-20: token t's key row goes to row seq_positions[t] of its context,
 * its value row to row seq_context_sizes[t] + seq_positions[t] (keys of the whole context first, then values). */
void oracle_copy_to_seq_context(int dt, int total_tokens, int kv_dim, const void * keys, const void * values, const int * seq_positions,
                                const uint64_t * seq_context_ptrs, const int * seq_context_sizes) {
	const size_t row = (size_t) kv_dim * (size_t) oracle_sizeof(dt);
	for (int t = 0; t < total_tokens; t++) {
		uint8_t * ctx = (uint8_t *) (uintptr_t) seq_context_ptrs[t];
		memcpy(ctx + (size_t) seq_positions[t] * row, (const uint8_t *) keys + (size_t) t * row, row);
		memcpy(ctx + ((size_t) seq_context_sizes[t] + (size_t) seq_positions[t]) * row, (const uint8_t *) values + (size_t) t * row, row);
	}
}

/* ------------------------------------------------------------------------------------------
 * select_experts (src/ops/nvidia/moe/select_experts.cu:3-239)
 * ---------------------------------------------------------------------------------------- */

/* exp(x) as a fixed sequence of IEEE fp32 operations (Cody-Waite reduction, Cephes polynomial): the CUDA kernel runs
 * the same sequence with explicit round-to-nearest intrinsics, so scores agree bit for bit. The reference's fast-math
 * build uses the hardware approximation instead (a few ulps away). */
static inline float det_expf(float x) {
	x = fminf(fmaxf(x, -87.0f), 88.0f);
	const float n = rintf(x * 1.44269504088896341f);
	float r = fmaf(n, -0.693359375f, x);
	r = fmaf(n, 2.12194440e-4f, r);
	float p = 1.9875691500e-4f;
	p = fmaf(p, r, 1.3981999507e-3f);
	p = fmaf(p, r, 8.3334519073e-3f);
	p = fmaf(p, r, 4.1665795894e-2f);
	p = fmaf(p, r, 1.6666665459e-1f);
	p = fmaf(p, r, 5.0000001201e-1f);
	const float r2 = r * r;
	const float e = fmaf(p, r2, r) + 1.0f;
	return e * u2f((uint32_t) ((int) n + 127) << 23);
}

/* `1.0 / (1 + expf(-x))` (:112): fp32 add, double division, rounded to fp32 */
static inline float sigmoid_score(float x) {
	if (x != x) return x;
	const float denom = 1.0f + det_expf(-x);
	return (float) (1.0 / (double) denom);
}

float oracle_sigmoid_score(float x) { return sigmoid_score(x); }

typedef struct { int dt, n_experts, top_k; const void * X; void * w; uint16_t * ids; int * counts; pthread_mutex_t * mu; } Select_Ctx;

static void select_rows(long r0, long r1, void * p) {
	Select_Ctx * c = (Select_Ctx *) p;
	const int k = c->top_k, ne = c->n_experts;
	float vals[64];
	int ids[64];
	int * local = (int *) calloc((size_t) ne, sizeof(int));
	for (long t = r0; t < r1; t++) {
		for (int j = 0; j < k; j++) { vals[j] = -INFINITY; ids[j] = 0xFFFF; }     /* :96-101 */
		float min_val = -INFINITY, sum = 0.0f;
		int min_slot = 0;
		for (int e = 0; e < ne; e++) {
			const float score = sigmoid_score(ld(c->dt, c->X, (size_t) t * ne + e));
			if (score > min_val) {                                               /* :128, strict */
				if (vals[min_slot] != -INFINITY) sum -= vals[min_slot];          /* :130-132 */
				vals[min_slot] = score; ids[min_slot] = e;
				sum += score;                                                    /* :137 */
				min_val = INFINITY;                                              /* :141-147: first slot holding the minimum */
				for (int j = 0; j < k; j++)
					if (vals[j] < min_val) { min_val = vals[j]; min_slot = j; }
			}
		}
		for (int j = 0; j < k; j++) {                                            /* :158-172 */
			st(c->dt, c->w, (size_t) t * k + j, vals[j] / sum);
			c->ids[(size_t) t * k + j] = (uint16_t) ids[j];
			if (ids[j] < ne) local[ids[j]]++;
		}
	}
	pthread_mutex_lock(c->mu);
	for (int e = 0; e < ne; e++) c->counts[e] += local[e];
	pthread_mutex_unlock(c->mu);
	free(local);
}

/* expert_counts has n_experts + 1 entries and is ACCUMULATED into (the reference adds with atomicAdd, :185); entry
 * n_experts (the kernel's block counter) is left at 0. cumsum = inclusive prefix sum; num_routed_by_expert zeroed (:226-236). */
void oracle_select_experts(int dt, int total_tokens, int n_experts, int top_k, const void * X_routed, void * token_expert_weights,
                           uint16_t * chosen_experts, int * expert_counts, int * expert_counts_cumsum, int * num_routed_by_expert, int n_threads) {
	if (top_k > 64) return;
	pthread_mutex_t mu = PTHREAD_MUTEX_INITIALIZER;
	Select_Ctx c = {dt, n_experts, top_k, X_routed, token_expert_weights, chosen_experts, expert_counts, &mu};
	for_rows(total_tokens, n_threads, select_rows, &c);
	int run = 0;
	for (int e = 0; e < n_experts; e++) { run += expert_counts[e]; expert_counts_cumsum[e] = run; num_routed_by_expert[e] = 0; }
	expert_counts[n_experts] = 0;
}
