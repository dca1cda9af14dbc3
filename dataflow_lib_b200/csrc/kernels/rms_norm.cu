// RMSNorm forward, backward-x and backward-w.
//
// Layout: X, out, dY, dX are [n_rows, n_cols] row-major; a row is split into chunks of 8
// elements and thread t of a CTA owns chunks t, t+T, t+2T, ... (VPT of them, compile time),
// so a warp reads 32 consecutive 128-bit packets per request and the thread's slice of the
// weight vector stays in registers for every row the CTA processes. CTAs are persistent and
// walk rows blockIdx.x, blockIdx.x + gridDim.x, ... ; the packets of the next row are
// requested before the current row is reduced, so each thread keeps 2*VPT (fwd), up to 6*VPT
// (bwd_x) loads in flight.
#include "common.cuh"
#include "tma.cuh"
#include <math_constants.h>

namespace dfb200 {

constexpr int E = 8;                 // elements per chunk
constexpr int MAX_VPT = 8;
// Threads that share one row, chosen by measurement on B200 (8192 x 4096 bf16, persistent grids):
// forward 128 x 4 chunks (6.5 TB/s; 256 x 2: 5.9, 512 x 1: 4.7), backward-x 256 x 2 chunks (6.5 TB/s),
// backward-w row groups of 256 x 2 chunks, four groups per CTA (5.5 TB/s for the partial sums).
constexpr int FWD_ROW_THREADS = 128, BWD_X_ROW_THREADS = 256, BWD_W_ROW_THREADS = 256;
// CTA width limits (launch bounds): a row uses ROW_THREADS threads until VPT reaches its maximum, then up to 512.
constexpr int fwd_max_threads(int vpt) { return vpt < MAX_VPT ? FWD_ROW_THREADS : 512; }
constexpr int bwd_x_max_threads(int vpt) { return vpt < MAX_VPT ? BWD_X_ROW_THREADS : 512; }
constexpr int bwd_w_max_threads(int vpt) { return vpt <= 2 ? 1024 : 512; }

template <typename T> struct RawChunk { uint32_t w[E / Word<T>::EPW]; };

template <typename T>
__device__ __forceinline__ void ld_raw(const void * base, uint64_t elem_idx, RawChunk<T> & c) {
	ld_words<E / Word<T>::EPW, Hint::STREAM>(reinterpret_cast<const char *>(base) + elem_idx * (4 / Word<T>::EPW), c.w);
}
// the same load without the evict-first hint, for tensors that the next op of a backward pass reads again
template <typename T>
__device__ __forceinline__ void ld_raw_keep(const void * base, uint64_t elem_idx, RawChunk<T> & c) {
	ld_words<E / Word<T>::EPW, Hint::KEEP>(reinterpret_cast<const char *>(base) + elem_idx * (4 / Word<T>::EPW), c.w);
}
template <typename T>
__device__ __forceinline__ void to_f32(const RawChunk<T> & c, float (&f)[E]) {
	#pragma unroll
	for (int i = 0; i < E / Word<T>::EPW; i++) Word<T>::unpack(c.w[i], &f[i * Word<T>::EPW]);
}

// Sum `a` and `b` over the CTA; every thread gets both totals. `slot` must alternate between
// consecutive calls (two smem buffers make one barrier per call enough).
__device__ __forceinline__ void block_sum2(float & a, float & b, float (*smem)[2][32], int slot) {
	a = warp_sum(a);
	b = warp_sum(b);
	const int n_warps = blockDim.x >> 5;
	if (n_warps == 1) return;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	if (lane == 0) { smem[slot][0][warp] = a; smem[slot][1][warp] = b; }
	__syncthreads();
	float x = lane < n_warps ? smem[slot][0][lane] : 0.0f;
	float y = lane < n_warps ? smem[slot][1][lane] : 0.0f;
	a = warp_sum(x);
	b = warp_sum(y);
}

// ----------------------------------------------------------------------------------------
// forward:  out = T( (x * r) * w ),  r = rsqrt(sum x^2 / n + eps)   (fp32, one rounding)
// follows src/ops/nvidia/norm/rms_norm.cu:339-406
// ----------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(fwd_max_threads(VPT))
rms_norm_fwd_kernel(int n_rows, int n_cols, float eps, const void * __restrict__ weight, const void * __restrict__ X,
                    void * __restrict__ out, float * __restrict__ weighted_sums, float * __restrict__ rms_vals) {
	__shared__ float red[2][2][32];
	const int n_chunks = n_cols / E;
	const int tid = threadIdx.x, nthr = blockDim.x;
	cudaTriggerProgrammaticLaunchCompletion();
	if ((int) blockIdx.x < n_rows) {                 // while the previous kernel of the stream drains: the first row's lines on their way to L2
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) prefetch_l2(reinterpret_cast<const char *>(X) + ((uint64_t) blockIdx.x * n_cols + (uint64_t) c * E) * (4 / Word<T>::EPW));
		}
	}
	cudaGridDependencySynchronize();

	RawChunk<T> wr[VPT], cur[VPT], nxt[VPT];     // packed: 4 registers per chunk for 16-bit types
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		if (c < n_chunks) ld_words<E / Word<T>::EPW, Hint::KEEP>(reinterpret_cast<const char *>(weight) + (size_t) c * E * (4 / Word<T>::EPW), wr[v].w);
	}
	int row = blockIdx.x;
	if (row < n_rows) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) ld_raw<T>(X, (uint64_t) row * n_cols + (uint64_t) c * E, cur[v]);
		}
	}
	int slot = 0;
	for (; row < n_rows; row += gridDim.x, slot ^= 1) {
		const int next_row = row + gridDim.x;
		if (next_row < n_rows) {
			#pragma unroll
			for (int v = 0; v < VPT; v++) {
				const int c = tid + v * nthr;
				if (c < n_chunks) ld_raw<T>(X, (uint64_t) next_row * n_cols + (uint64_t) c * E, nxt[v]);
			}
		}
		float ss = 0.0f, ws = 0.0f;
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				float x[E], w[E];
				to_f32<T>(cur[v], x); to_f32<T>(wr[v], w);
				#pragma unroll
				for (int i = 0; i < E; i++) { ws = fmaf(w[i], x[i], ws); ss = fmaf(x[i], x[i], ss); }
			}
		}
		block_sum2(ss, ws, red, slot);
		const float r = rsqrtf(ss / (float) n_cols + eps);
		if (tid == 0) {
			if (weighted_sums) weighted_sums[row] = ws;
			if (rms_vals) rms_vals[row] = r;
		}
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				float x[E], w[E], o[E];
				to_f32<T>(cur[v], x); to_f32<T>(wr[v], w);
				#pragma unroll
				for (int i = 0; i < E; i++) o[i] = (x[i] * r) * w[i];
				store_elems<T, E>(out, (uint64_t) row * n_cols + (uint64_t) c * E, o);
			}
		}
		#pragma unroll
		for (int v = 0; v < VPT; v++) cur[v] = nxt[v];
	}
}

// ----------------------------------------------------------------------------------------
// backward-x:  dX += dY * B( w*r - ((x*r^3)/n) * ws )   follows
// src/ops/nvidia/norm/rms_norm_bwd_x.cu:243-252 : the derivative is formed in fp32 and rounded
// to the backward type B; the update dX + dY*B(deriv) is ONE fused multiply-add in B (a single
// rounding), which is what the reference's `dX += dY * deriv` compiles to (fma.rn.bf16x2 /
// fma.rn.f16x2 / fma.rn.f32) -- the reference kernels' outputs confirm it bit for bit.
// 16-bit types stay packed: dY and dX words go straight into the paired fma.
// ----------------------------------------------------------------------------------------
template <typename B> struct FusedUpdate;
template <> struct FusedUpdate<f32_t> {
	static __device__ __forceinline__ uint32_t apply(uint32_t dx, uint32_t dy, const float * deriv) {
		return __float_as_uint(fmaf(__uint_as_float(dy), deriv[0], __uint_as_float(dx)));
	}
};
template <> struct FusedUpdate<bf16_t> {
	static __device__ __forceinline__ uint32_t apply(uint32_t dx, uint32_t dy, const float * deriv) {
		const __nv_bfloat162 d = __floats2bfloat162_rn(deriv[0], deriv[1]);
		const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162 *>(&dy), d, *reinterpret_cast<const __nv_bfloat162 *>(&dx));
		return *reinterpret_cast<const uint32_t *>(&r);
	}
};
template <> struct FusedUpdate<f16_t> {
	static __device__ __forceinline__ uint32_t apply(uint32_t dx, uint32_t dy, const float * deriv) {
		const __half2 d = __floats2half2_rn(deriv[0], deriv[1]);
		const __half2 r = __hfma2(*reinterpret_cast<const __half2 *>(&dy), d, *reinterpret_cast<const __half2 *>(&dx));
		return *reinterpret_cast<const uint32_t *>(&r);
	}
};

template <typename F, typename B, int VPT>
__global__ void __launch_bounds__(bwd_x_max_threads(VPT))
rms_norm_bwd_x_kernel(int n_rows, int n_cols, const float * __restrict__ fwd_weighted_sums, const float * __restrict__ fwd_rms_vals,
                      const void * __restrict__ weight, const void * __restrict__ X, const void * __restrict__ dY, void * dX) {
	constexpr int BEPW = Word<B>::EPW, BW = E / BEPW;
	pdl_prologue();
	const int n_chunks = n_cols / E;
	const int tid = threadIdx.x, nthr = blockDim.x;
	const float n_cols_f = (float) n_cols;

	RawChunk<F> wr[VPT];
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		if (c < n_chunks) ld_words<E / Word<F>::EPW, Hint::KEEP>(reinterpret_cast<const char *>(weight) + (size_t) c * E * (4 / Word<F>::EPW), wr[v].w);
	}

	for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
		RawChunk<F> xr[VPT];
		RawChunk<B> gr[VPT], dr[VPT];
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				const uint64_t off = (uint64_t) row * n_cols + (uint64_t) c * E;
				ld_raw_keep<F>(X, off, xr[v]);           // X and dY are read again by rms_norm_bwd_w, which walks the rows backwards
				ld_raw_keep<B>(dY, off, gr[v]);
				ld_raw<B>(dX, off, dr[v]);
			}
		}
		const float r = __ldg(fwd_rms_vals + row);
		const float ws = __ldg(fwd_weighted_sums + row);
		const float r3 = r * r * r;
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				float x[E], w[E], deriv[E];
				to_f32<F>(xr[v], x); to_f32<F>(wr[v], w);
				#pragma unroll
				for (int i = 0; i < E; i++) deriv[i] = (w[i] * r) - (__fdividef(x[i] * r3, n_cols_f) * ws);
				uint32_t o[BW];
				#pragma unroll
				for (int k = 0; k < BW; k++) o[k] = FusedUpdate<B>::apply(dr[v].w[k], gr[v].w[k], &deriv[k * BEPW]);
				st_words<BW>(reinterpret_cast<char *>(dX) + ((uint64_t) row * n_cols + (uint64_t) c * E) * (4 / BEPW), o);
			}
		}
	}
}

// ----------------------------------------------------------------------------------------
// backward-w, stage 1: every CTA reduces dY*x*r over its rows into fp32 column sums.
// The CTA is GROUPS row-groups of `group_threads` threads; group g takes rows
// blockIdx.x*GROUPS + g, + gridDim.x*GROUPS, ... ; the groups are then summed through shared
// memory in group order and the CTA writes one fp32 row [n_cols] of partial sums.
// The arithmetic per term follows src/ops/nvidia/norm/rms_norm_bwd_w.cu:295 (f32(dY)*f32(x)*r).
// ----------------------------------------------------------------------------------------
template <typename F, typename B, int VPT>
__global__ void __launch_bounds__(bwd_w_max_threads(VPT))
rms_norm_bwd_w_partial_kernel(int n_rows, int n_cols, int group_threads, const float * __restrict__ fwd_rms_vals,
                              const void * __restrict__ X, const void * __restrict__ dY, float * __restrict__ partials) {
	extern __shared__ float group_sums[];      // [groups - 1][n_cols]
	pdl_prologue();                            // also lets stage 2 be scheduled: it waits for this grid in its own prologue
	const int n_chunks = n_cols / E;
	const int groups = blockDim.x / group_threads;
	const int g = threadIdx.x / group_threads;
	const int tid = threadIdx.x - g * group_threads;

	float acc[VPT][E];
	#pragma unroll
	for (int v = 0; v < VPT; v++)
		#pragma unroll
		for (int i = 0; i < E; i++) acc[v][i] = 0.0f;

	// Rows are visited from the LAST one backwards: this op usually follows rms_norm_bwd_x on the same X and dY, whose last rows are
	// the ones still in L2 (the two tensors exceed it), so the walk starts where the cache is warm. The sum does not depend on the order.
	const int row_stride = gridDim.x * groups;
	RawChunk<F> xr[VPT], xn[VPT];
	RawChunk<B> gr[VPT], gn[VPT];
	int row = blockIdx.x * groups + g;
	float r_next = 0.0f;                             // the row's rms value travels with its packets, one row ahead
	if (row < n_rows) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				const uint64_t off = (uint64_t) (n_rows - 1 - row) * n_cols + (uint64_t) c * E;
				ld_raw<F>(X, off, xr[v]);
				ld_raw<B>(dY, off, gr[v]);
			}
		}
		r_next = __ldg(fwd_rms_vals + (n_rows - 1 - row));
	}
	for (; row < n_rows; row += row_stride) {
		const int next_row = row + row_stride;
		const float r = r_next;
		if (next_row < n_rows) {                     // next row's packets are requested before this row is consumed
			r_next = __ldg(fwd_rms_vals + (n_rows - 1 - next_row));
			#pragma unroll
			for (int v = 0; v < VPT; v++) {
				const int c = tid + v * group_threads;
				if (c < n_chunks) {
					const uint64_t off = (uint64_t) (n_rows - 1 - next_row) * n_cols + (uint64_t) c * E;
					ld_raw<F>(X, off, xn[v]);
					ld_raw<B>(dY, off, gn[v]);
				}
			}
		}
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				float x[E], gy[E];
				to_f32<F>(xr[v], x); to_f32<B>(gr[v], gy);
				#pragma unroll
				for (int i = 0; i < E; i++) acc[v][i] += gy[i] * x[i] * r;
			}
		}
		#pragma unroll
		for (int v = 0; v < VPT; v++) { xr[v] = xn[v]; gr[v] = gn[v]; }
	}

	if (g > 0) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				float4 * dst = reinterpret_cast<float4 *>(group_sums + (size_t) (g - 1) * n_cols + (size_t) c * E);
				dst[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
				dst[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
			}
		}
	}
	__syncthreads();
	if (g == 0) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				for (int o = 0; o < groups - 1; o++) {
					const float4 * src = reinterpret_cast<const float4 *>(group_sums + (size_t) o * n_cols + (size_t) c * E);
					const float4 a = src[0], b = src[1];
					acc[v][0] += a.x; acc[v][1] += a.y; acc[v][2] += a.z; acc[v][3] += a.w;
					acc[v][4] += b.x; acc[v][5] += b.y; acc[v][6] += b.z; acc[v][7] += b.w;
				}
				float4 * dst = reinterpret_cast<float4 *>(partials + (size_t) blockIdx.x * n_cols + (size_t) c * E);
				dst[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
				dst[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
			}
		}
	}
}

// ----------------------------------------------------------------------------------------
// backward-x and backward-w stage 1 in ONE pass over X and dY (no reference counterpart: the reference launches the two kernels
// above one after the other, and the second reads X and dY again). Geometry of backward-w stage 1: one CTA per SM, GROUPS row
// groups of `group_threads` threads, group g taking rows blockIdx.x*GROUPS + g, + gridDim.x*GROUPS, ... . Per row a thread does
// what rms_norm_bwd_x_kernel does to its packets of dX (same arithmetic, same roundings: the dX it writes is bit-identical) and
// adds f32(dY)*f32(x)*r to its fp32 column sums, which leave the CTA the way rms_norm_bwd_w_partial_kernel's do. There is no
// barrier in the row loop, so the warps of a CTA drift apart and one warp's loads overlap another's arithmetic; all packets of a
// row are requested before the first is used (6*VPT 16-byte loads per thread in flight).
// ----------------------------------------------------------------------------------------
template <typename F, typename B, int VPT>
__global__ void __launch_bounds__(bwd_w_max_threads(VPT))
rms_norm_bwd_xw_partial_kernel(int n_rows, int n_cols, int group_threads, const float * __restrict__ fwd_weighted_sums,
                               const float * __restrict__ fwd_rms_vals, const void * __restrict__ weight, const void * __restrict__ X,
                               const void * __restrict__ dY, void * dX, float * __restrict__ partials) {
	constexpr int BEPW = Word<B>::EPW, BW = E / BEPW;
	extern __shared__ float group_sums[];      // [groups - 1][n_cols]
	pdl_prologue();                            // also lets stage 2 be scheduled: it waits for this grid in its own prologue
	const int n_chunks = n_cols / E;
	const int groups = blockDim.x / group_threads;
	const int g = threadIdx.x / group_threads;
	const int tid = threadIdx.x - g * group_threads;
	const float n_cols_f = (float) n_cols;

	float acc[VPT][E];
	RawChunk<F> wr[VPT];
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		#pragma unroll
		for (int i = 0; i < E; i++) acc[v][i] = 0.0f;
		const int c = tid + v * group_threads;
		if (c < n_chunks) ld_words<E / Word<F>::EPW, Hint::KEEP>(reinterpret_cast<const char *>(weight) + (size_t) c * E * (4 / Word<F>::EPW), wr[v].w);
	}

	const int row_stride = gridDim.x * groups;
	for (int row = blockIdx.x * groups + g; row < n_rows; row += row_stride) {
		RawChunk<F> xr[VPT];
		RawChunk<B> gr[VPT], dr[VPT];
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				const uint64_t off = (uint64_t) row * n_cols + (uint64_t) c * E;
				ld_raw<F>(X, off, xr[v]);
				ld_raw<B>(dY, off, gr[v]);
				ld_raw<B>(dX, off, dr[v]);
			}
		}
		const float r = __ldg(fwd_rms_vals + row);
		const float ws = __ldg(fwd_weighted_sums + row);
		const float r3 = r * r * r;
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				float x[E], w[E], gy[E], deriv[E];
				to_f32<F>(xr[v], x); to_f32<F>(wr[v], w); to_f32<B>(gr[v], gy);
				#pragma unroll
				for (int i = 0; i < E; i++) {
					deriv[i] = (w[i] * r) - (__fdividef(x[i] * r3, n_cols_f) * ws);
					acc[v][i] += gy[i] * x[i] * r;
				}
				uint32_t o[BW];
				#pragma unroll
				for (int k = 0; k < BW; k++) o[k] = FusedUpdate<B>::apply(dr[v].w[k], gr[v].w[k], &deriv[k * BEPW]);
				st_words<BW>(reinterpret_cast<char *>(dX) + ((uint64_t) row * n_cols + (uint64_t) c * E) * (4 / BEPW), o);
			}
		}
	}

	if (g > 0) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				float4 * dst = reinterpret_cast<float4 *>(group_sums + (size_t) (g - 1) * n_cols + (size_t) c * E);
				dst[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
				dst[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
			}
		}
	}
	__syncthreads();
	if (g == 0) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				for (int o = 0; o < groups - 1; o++) {
					const float4 * src = reinterpret_cast<const float4 *>(group_sums + (size_t) o * n_cols + (size_t) c * E);
					const float4 a = src[0], b = src[1];
					acc[v][0] += a.x; acc[v][1] += a.y; acc[v][2] += a.z; acc[v][3] += a.w;
					acc[v][4] += b.x; acc[v][5] += b.y; acc[v][6] += b.z; acc[v][7] += b.w;
				}
				float4 * dst = reinterpret_cast<float4 *>(partials + (size_t) blockIdx.x * n_cols + (size_t) c * E);
				dst[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
				dst[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
			}
		}
	}
}

// ----------------------------------------------------------------------------------------
// The same fused pass with the rows STAGED through shared memory by bulk asynchronous copies. A thread of the register kernel above
// has at most 6*VPT packets in flight and then stops requesting while it computes; what a whole SM keeps in flight (96 KB at 1024
// threads) is what limits it (5.0 TB/s at 8192 x 4096 bf16). Here each row group owns a ring of `stages` row slots [X | dY | dX] that
// its thread 0 refills with three bulk copies as soon as the group has consumed a slot, so an SM has up to 8 rows (192 KB at
// d = 4096 bf16) in flight whatever the threads are doing, and the registers hold only the weights and the column sums.
// Waits are bounded: a group whose copy does not arrive records it in *status, the CTA's partial sums become NaN (so does dW) and
// the rows it did not reach keep their dX.
// ----------------------------------------------------------------------------------------
constexpr int XW_STAGED_THREADS = 512, XW_MAX_STAGES = 4;
constexpr size_t XW_RING_BUDGET = 200 * 1024;

template <int NW> __device__ __forceinline__ void lds_words(const unsigned char * p, uint32_t (&w)[NW]) {
	static_assert(NW == 2 || NW == 4 || NW == 8, "a chunk of 8 elements is 8, 16 or 32 bytes");
	if constexpr (NW == 2) {
		const uint2 v = *reinterpret_cast<const uint2 *>(p);
		w[0] = v.x; w[1] = v.y;
	} else {
		#pragma unroll
		for (int q = 0; q < NW / 4; q++) {
			const uint4 v = reinterpret_cast<const uint4 *>(p)[q];
			w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
		}
	}
}

template <typename F, typename B, int VPT>
__global__ void __launch_bounds__(XW_STAGED_THREADS, 1)
rms_norm_bwd_xw_staged_kernel(int n_rows, int n_cols, int group_threads, int stages, const float * __restrict__ fwd_weighted_sums,
                              const float * __restrict__ fwd_rms_vals, const void * __restrict__ weight, const void * X, const void * dY, void * dX,
                              float * __restrict__ partials, unsigned int * status) {
	constexpr int FW = E / Word<F>::EPW, BEPW = Word<B>::EPW, BW = E / BEPW;
	constexpr uint32_t FSIZE = 4 / Word<F>::EPW, BSIZE = 4 / BEPW;
	extern __shared__ __align__(128) unsigned char xw_smem[];
	__shared__ int s_failed;
	const int n_chunks = n_cols / E;
	const int groups = blockDim.x / group_threads;
	const int g = threadIdx.x / group_threads;
	const int tid = threadIdx.x - g * group_threads;
	const float n_cols_f = (float) n_cols;
	const uint32_t xb = (uint32_t) n_cols * FSIZE, gb = (uint32_t) n_cols * BSIZE, stage_bytes = xb + 2 * gb;
	unsigned char * ring = xw_smem + (size_t) g * stages * stage_bytes;                                         // this group's [stages][X | dY | dX]
	uint64_t * full = reinterpret_cast<uint64_t *>(xw_smem + (size_t) groups * stages * stage_bytes) + g * stages;

	cudaTriggerProgrammaticLaunchCompletion();       // see pdl_prologue(): the set-up below needs no global memory
	if (threadIdx.x == 0) s_failed = 0;
	if (tid == 0) {
		// while the previous kernel of the stream drains: this group's first rows on their way to L2
		for (int k = 0; k < stages; k++) {
			const uint64_t row = (uint64_t) blockIdx.x * groups + g + (uint64_t) k * gridDim.x * groups;
			if (row >= (uint64_t) n_rows) break;
			bulk_prefetch_l2(reinterpret_cast<const unsigned char *>(X) + row * xb, xb);
			bulk_prefetch_l2(reinterpret_cast<const unsigned char *>(dY) + row * gb, gb);
			bulk_prefetch_l2(reinterpret_cast<const unsigned char *>(dX) + row * gb, gb);
		}
		for (int s = 0; s < stages; s++) mbar_init(&full[s], 1);
		mbar_fence_init();
	}
	float acc[VPT][E];
	#pragma unroll
	for (int v = 0; v < VPT; v++)
		#pragma unroll
		for (int i = 0; i < E; i++) acc[v][i] = 0.0f;
	__syncthreads();
	cudaGridDependencySynchronize();

	const int row_stride = gridDim.x * groups, first = blockIdx.x * groups + g;
	const int my_iters = first < n_rows ? (n_rows - first + row_stride - 1) / row_stride : 0;
	auto issue = [&](int k) {                        // thread 0 of the group only
		const int s = k % stages;
		const uint64_t row = (uint64_t) (first + k * row_stride);
		unsigned char * dst = ring + (size_t) s * stage_bytes;
		mbar_arrive_expect_tx(&full[s], stage_bytes);
		bulk_load(dst, reinterpret_cast<const unsigned char *>(X) + row * xb, xb, &full[s]);
		bulk_load(dst + xb, reinterpret_cast<const unsigned char *>(dY) + row * gb, gb, &full[s]);
		bulk_load(dst + xb + gb, reinterpret_cast<const unsigned char *>(dX) + row * gb, gb, &full[s]);
	};
	if (tid == 0)
		for (int k = 0; k < stages && k < my_iters; k++) issue(k);

	RawChunk<F> wr[VPT];
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * group_threads;
		if (c < n_chunks) ld_words<FW, Hint::KEEP>(reinterpret_cast<const char *>(weight) + (size_t) c * E * FSIZE, wr[v].w);
	}

	// the two statistics of a row are requested one row ahead: a scalar load issued when the row is due would put a trip to L2 on
	// every row's critical path
	float r_next = 0.0f, ws_next = 0.0f;
	if (my_iters > 0) { r_next = __ldg(fwd_rms_vals + first); ws_next = __ldg(fwd_weighted_sums + first); }
	for (int k = 0; k < my_iters; k++) {
		const int s = k % stages, row = first + k * row_stride;
		const float r = r_next, ws = ws_next;
		if (k + 1 < my_iters) { r_next = __ldg(fwd_rms_vals + row + row_stride); ws_next = __ldg(fwd_weighted_sums + row + row_stride); }
		const bool arrived = mbar_wait_bounded(&full[s], (uint32_t) (k / stages) & 1u, status, 0x300u + (unsigned) s);
		if (arrived) {
			const unsigned char * slot = ring + (size_t) s * stage_bytes;
			const float r3 = r * r * r;
			#pragma unroll
			for (int v = 0; v < VPT; v++) {
				const int c = tid + v * group_threads;
				if (c < n_chunks) {
					RawChunk<F> xr;
					RawChunk<B> gr, dr;
					lds_words<FW>(slot + (size_t) c * E * FSIZE, xr.w);
					lds_words<BW>(slot + xb + (size_t) c * E * BSIZE, gr.w);
					lds_words<BW>(slot + xb + gb + (size_t) c * E * BSIZE, dr.w);
					float x[E], w[E], gy[E], deriv[E];
					to_f32<F>(xr, x); to_f32<F>(wr[v], w); to_f32<B>(gr, gy);
					#pragma unroll
					for (int i = 0; i < E; i++) {
						deriv[i] = (w[i] * r) - (__fdividef(x[i] * r3, n_cols_f) * ws);
						acc[v][i] += gy[i] * x[i] * r;
					}
					uint32_t o[BW];
					#pragma unroll
					for (int q = 0; q < BW; q++) o[q] = FusedUpdate<B>::apply(dr.w[q], gr.w[q], &deriv[q * BEPW]);
					st_words<BW>(reinterpret_cast<char *>(dX) + ((uint64_t) row * n_cols + (uint64_t) c * E) * BSIZE, o);
				}
			}
		} else {
			*reinterpret_cast<volatile int *>(&s_failed) = 1;
		}
		// the group's own barrier (ids 1 .. groups): every thread of the group has read the slot, and a failure flag set above is visible
		asm volatile("bar.sync %0, %1;" :: "r"(1 + g), "r"(group_threads) : "memory");
		if (*reinterpret_cast<volatile int *>(&s_failed)) break;
		if (tid == 0 && k + stages < my_iters) issue(k + stages);
	}
	__syncthreads();                                 // every group has left its loop
	const bool failed = *reinterpret_cast<volatile int *>(&s_failed) != 0;
	if (failed) {
		// copies may still be in flight into the ring: leave it alone, and poison what this CTA contributes
		for (int c = threadIdx.x; c < n_cols; c += blockDim.x) partials[(size_t) blockIdx.x * n_cols + c] = CUDART_NAN_F;
		return;
	}
	// every copy that was issued has been waited for, so the ring can carry the groups' column sums now
	float * group_sums = reinterpret_cast<float *>(xw_smem);   // [groups - 1][n_cols]
	if (g > 0) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				float4 * dst = reinterpret_cast<float4 *>(group_sums + (size_t) (g - 1) * n_cols + (size_t) c * E);
				dst[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
				dst[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
			}
		}
	}
	__syncthreads();
	if (g == 0) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				for (int o = 0; o < groups - 1; o++) {
					const float4 * src = reinterpret_cast<const float4 *>(group_sums + (size_t) o * n_cols + (size_t) c * E);
					const float4 a = src[0], b = src[1];
					acc[v][0] += a.x; acc[v][1] += a.y; acc[v][2] += a.z; acc[v][3] += a.w;
					acc[v][4] += b.x; acc[v][5] += b.y; acc[v][6] += b.z; acc[v][7] += b.w;
				}
				float4 * dst = reinterpret_cast<float4 *>(partials + (size_t) blockIdx.x * n_cols + (size_t) c * E);
				dst[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
				dst[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
			}
		}
	}
}

// backward-w, stage 2: dW[c] = B( f32(dW[c]) + sum_p partials[p][c] ). A CTA covers 32
// columns with 32 slices of the partial rows (every thread a handful of independent loads);
// slices are combined in slice order. Launched as a programmatic dependent of stage 1: its CTAs
// are scheduled while stage 1 drains and block in cudaGridDependencySynchronize() until stage 1
// has completed and its partial sums are visible, which hides the launch latency.
// SUMS = true: dW is a float array that RECEIVES the column sums (fp32, overwritten, nothing read): the form a data-parallel
// caller wants, whose next step is an all-reduce of fp32 partial gradients (a slot of a packed exchange buffer).
template <typename B, bool SUMS>
__global__ void __launch_bounds__(1024)
rms_norm_bwd_w_final_kernel(int n_cols, int n_partials, const float * __restrict__ partials, void * dW) {
	__shared__ float slice_sum[32][33];
	const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
	const int col = blockIdx.x * 32 + lane;
	pdl_prologue();
	float s = 0.0f;
	if (col < n_cols) {
		#pragma unroll 4
		for (int p = slice; p < n_partials; p += 32) s += partials[(size_t) p * n_cols + col];
	}
	slice_sum[slice][lane] = s;
	__syncthreads();
	if (slice == 0 && col < n_cols) {
		float total = slice_sum[0][lane];
		#pragma unroll
		for (int k = 1; k < 32; k++) total += slice_sum[k][lane];
		// element-wise read-modify-write of dW in its own type
		if constexpr (SUMS) {
			reinterpret_cast<float *>(dW)[col] = total;
		} else if constexpr (Word<B>::EPW == 1) {
			float * p = reinterpret_cast<float *>(dW) + col;
			*p = *p + total;
		} else {
			static_assert(Word<B>::EPW == 2, "backward datatypes are fp32, fp16 or bf16");
			uint16_t * p = reinterpret_cast<uint16_t *>(dW) + col;
			float pair[2];
			Word<B>::unpack((uint32_t) *p, pair);
			pair[0] += total; pair[1] = 0.0f;
			*p = (uint16_t) (Word<B>::pack(pair) & 0xffffu);
		}
	}
}

// ----------------------------------------------------------------------------------------
// General shapes: any n_cols, tensors aligned to their element size only -- what the reference's thread-strided scalar loops
// accept (src/ops/nvidia/norm/rms_norm.cu:339-406, rms_norm_bwd_x.cu:243-252, rms_norm_bwd_w.cu:270-299). One 256-thread CTA per
// row at a time, one element per access; the arithmetic and the rounding points are those of the packet kernels above (the fp32
// summation order within a row differs, as it does between any two thread layouts).
// ----------------------------------------------------------------------------------------
constexpr int GENERAL_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(GENERAL_THREADS)
rms_norm_fwd_general_kernel(int n_rows, int n_cols, float eps, const void * __restrict__ weight, const void * __restrict__ X,
                            void * __restrict__ out, float * __restrict__ weighted_sums, float * __restrict__ rms_vals) {
	__shared__ float red[2][2][32];
	pdl_prologue();
	int slot = 0;
	for (int row = blockIdx.x; row < n_rows; row += gridDim.x, slot ^= 1) {
		const uint64_t base = (uint64_t) row * n_cols;
		float ss = 0.0f, ws = 0.0f;
		for (int i = threadIdx.x; i < n_cols; i += GENERAL_THREADS) {
			const float x = load_one<T>(X, base + i), w = load_one<T>(weight, i);
			ws = fmaf(w, x, ws); ss = fmaf(x, x, ss);
		}
		block_sum2(ss, ws, red, slot);
		const float r = rsqrtf(ss / (float) n_cols + eps);
		if (threadIdx.x == 0) {
			if (weighted_sums) weighted_sums[row] = ws;
			if (rms_vals) rms_vals[row] = r;
		}
		for (int i = threadIdx.x; i < n_cols; i += GENERAL_THREADS)
			store_one<T>(out, base + i, (load_one<T>(X, base + i) * r) * load_one<T>(weight, i));
	}
}

// dX + dY * B(deriv) as ONE fused multiply-add in B (see FusedUpdate), for a single element
template <typename B> __device__ __forceinline__ float fused_update_one(float dx, float dy, float deriv);
template <> __device__ __forceinline__ float fused_update_one<f32_t>(float dx, float dy, float deriv) { return fmaf(dy, deriv, dx); }
template <> __device__ __forceinline__ float fused_update_one<bf16_t>(float dx, float dy, float deriv) {
	return __bfloat162float(__hfma(__float2bfloat16_rn(dy), __float2bfloat16_rn(deriv), __float2bfloat16_rn(dx)));      // dy, dx are bf16 values: exact
}
template <> __device__ __forceinline__ float fused_update_one<f16_t>(float dx, float dy, float deriv) {
	return __half2float(__hfma(__float2half_rn(dy), __float2half_rn(deriv), __float2half_rn(dx)));
}

template <typename F, typename B>
__global__ void __launch_bounds__(GENERAL_THREADS)
rms_norm_bwd_x_general_kernel(int n_rows, int n_cols, const float * __restrict__ fwd_weighted_sums, const float * __restrict__ fwd_rms_vals,
                              const void * __restrict__ weight, const void * __restrict__ X, const void * __restrict__ dY, void * dX) {
	pdl_prologue();
	const float n_cols_f = (float) n_cols;
	for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
		const uint64_t base = (uint64_t) row * n_cols;
		const float r = __ldg(fwd_rms_vals + row), ws = __ldg(fwd_weighted_sums + row);
		const float r3 = r * r * r;
		for (int i = threadIdx.x; i < n_cols; i += GENERAL_THREADS) {
			const float deriv = (load_one<F>(weight, i) * r) - (__fdividef(load_one<F>(X, base + i) * r3, n_cols_f) * ws);
			store_one<B>(dX, base + i, fused_update_one<B>(load_one<B>(dX, base + i), load_one<B>(dY, base + i), deriv));
		}
	}
}

// stage 1 of backward-w: CTA b sums its rows b, b + gridDim.x, ... for every column; thread t owns columns t, t + 256, ...
template <typename F, typename B>
__global__ void __launch_bounds__(GENERAL_THREADS)
rms_norm_bwd_w_partial_general_kernel(int n_rows, int n_cols, const float * __restrict__ fwd_rms_vals, const void * __restrict__ X,
                                      const void * __restrict__ dY, float * __restrict__ partials) {
	pdl_prologue();
	for (int c = threadIdx.x; c < n_cols; c += GENERAL_THREADS) {
		float acc = 0.0f;
		for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
			const uint64_t i = (uint64_t) row * n_cols + c;
			acc += load_one<B>(dY, i) * load_one<F>(X, i) * __ldg(fwd_rms_vals + row);
		}
		partials[(size_t) blockIdx.x * n_cols + c] = acc;
	}
}

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------

struct RowGeometry { int vpt; int threads; };

static bool elem_aligned(const void * p, int dt) { return reinterpret_cast<uintptr_t>(p) % (uintptr_t) dtype_size(dt) == 0; }

// Pick the chunks-per-thread (1,2,4,8) and the CTA width (multiple of 32) for a row of
// n_chunks chunks: about `row_threads` threads per row, wider (up to 512) only once VPT has
// reached its maximum.
static bool row_geometry(int n_chunks, int row_threads, RowGeometry * geo) {
	int vpt = 1;
	while (vpt < MAX_VPT && (n_chunks + vpt - 1) / vpt > row_threads) vpt *= 2;
	int threads = (n_chunks + vpt - 1) / vpt;
	threads = (threads + 31) / 32 * 32;
	if (threads > (vpt < MAX_VPT ? row_threads : 512)) return false;
	geo->vpt = vpt; geo->threads = threads;
	return true;
}

// *packets = true: the row length is a multiple of 8 elements within the packet kernels' range (the caller still checks the 16-byte
// alignment of its tensors); false: the general kernels take the call.
static int check_rows(const char * op, int n_rows, int n_cols, int row_threads, RowGeometry * geo, bool * packets) {
	if (n_rows < 0 || n_cols <= 0) return set_error(DFB200_ERR_ARG, "%s: bad shape %d x %d", op, n_rows, n_cols);
	*packets = n_cols % E == 0 && row_geometry(n_cols / E, row_threads, geo);
	return DFB200_OK;
}

static int general_row_grid(int n_rows) {
	const long long cap = (long long) (sm_count() > 0 ? sm_count() : 1) * 8;
	return (int) (n_rows < cap ? (n_rows > 0 ? n_rows : 1) : cap);
}

#define DFB200_DISPATCH_VPT(vpt, VPT, ...)                  \
	switch (vpt) {                                          \
		case 1:  { constexpr int VPT = 1;  __VA_ARGS__; break; } \
		case 2:  { constexpr int VPT = 2;  __VA_ARGS__; break; } \
		case 4:  { constexpr int VPT = 4;  __VA_ARGS__; break; } \
		default: { constexpr int VPT = 8;  __VA_ARGS__; break; } \
	}

// Grid of a persistent row kernel: every SM filled to the occupancy the kernel reaches.
template <typename K> static int persistent_grid(K kernel, int n_rows, int threads) {
	const int per_sm = ctas_per_sm(reinterpret_cast<const void *>(kernel), threads, 0);
	long long g = (long long) sm_count() * per_sm;
	if (g > n_rows) g = n_rows;
	return g < 1 ? 1 : (int) g;
}

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_rms_norm(int fwd_dt, int n_rows, int n_cols, float eps, const void * rms_weight, const void * X, void * out,
                               float * weighted_sums, float * rms_vals, void * stream) {
	if (!dtype_size(fwd_dt)) return set_error(DFB200_ERR_DTYPE, "rms_norm: unsupported datatype %d", fwd_dt);
	RowGeometry geo;
	bool packets;
	int rc = check_rows("rms_norm", n_rows, n_cols, FWD_ROW_THREADS, &geo, &packets);
	if (rc) return rc;
	if (n_rows == 0) return DFB200_OK;
	if (!rms_weight || !X || !out) return set_error(DFB200_ERR_ARG, "rms_norm: NULL tensor argument");
	if (!elem_aligned(rms_weight, fwd_dt) || !elem_aligned(X, fwd_dt) || !elem_aligned(out, fwd_dt))
		return set_error(DFB200_ERR_ARG, "rms_norm: tensors must be aligned to their element size");
	if (!packets || !aligned16(rms_weight) || !aligned16(X) || !aligned16(out)) {
		DFB200_DISPATCH_DTYPE(fwd_dt, T,
			(launch_pdl(rms_norm_fwd_general_kernel<T>, dim3(general_row_grid(n_rows)), dim3(GENERAL_THREADS), 0, (cudaStream_t) stream, n_rows, n_cols, eps,
			            rms_weight, X, out, weighted_sums, rms_vals)));
		return check_launch("rms_norm (general shape)");
	}
	DFB200_DISPATCH_DTYPE(fwd_dt, T, DFB200_DISPATCH_VPT(geo.vpt, VPT, {
		auto kernel = rms_norm_fwd_kernel<T, VPT>;
		const int grid = persistent_grid(kernel, n_rows, geo.threads);
		launch_pdl(kernel, dim3(grid), dim3(geo.threads), 0, (cudaStream_t) stream, n_rows, n_cols, eps, rms_weight, X, out, weighted_sums, rms_vals);
	}));
	return check_launch("rms_norm");
}

extern "C" int dfb200_rms_norm_bwd_x(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_weighted_sums,
                                     const float * fwd_rms_vals, const void * rms_weight, const void * X_inp, const void * upstream_dX,
                                     void * dX, void * stream) {
	(void) eps;
	if (!valid_fwd_bwd_pair(fwd_dt, bwd_dt)) return set_error(DFB200_ERR_DTYPE, "rms_norm_bwd_x: unsupported datatype pair (%d, %d)", fwd_dt, bwd_dt);
	RowGeometry geo;
	bool packets;
	int rc = check_rows("rms_norm_bwd_x", n_rows, n_cols, BWD_X_ROW_THREADS, &geo, &packets);
	if (rc) return rc;
	if (n_rows == 0) return DFB200_OK;
	if (!fwd_weighted_sums || !fwd_rms_vals || !rms_weight || !X_inp || !upstream_dX || !dX)
		return set_error(DFB200_ERR_ARG, "rms_norm_bwd_x: NULL tensor argument");
	if (!elem_aligned(rms_weight, fwd_dt) || !elem_aligned(X_inp, fwd_dt) || !elem_aligned(upstream_dX, bwd_dt) || !elem_aligned(dX, bwd_dt))
		return set_error(DFB200_ERR_ARG, "rms_norm_bwd_x: tensors must be aligned to their element size");
	if (!packets || !aligned16(rms_weight) || !aligned16(X_inp) || !aligned16(upstream_dX) || !aligned16(dX)) {
		DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
			(launch_pdl(rms_norm_bwd_x_general_kernel<F, B>, dim3(general_row_grid(n_rows)), dim3(GENERAL_THREADS), 0, (cudaStream_t) stream, n_rows, n_cols,
			            fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX)));
		return check_launch("rms_norm_bwd_x (general shape)");
	}
	DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B, DFB200_DISPATCH_VPT(geo.vpt, VPT, {
		auto kernel = rms_norm_bwd_x_kernel<F, B, VPT>;
		const int grid = persistent_grid(kernel, n_rows, geo.threads);
		launch_pdl(kernel, dim3(grid), dim3(geo.threads), 0, (cudaStream_t) stream, n_rows, n_cols, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX);
	}));
	return check_launch("rms_norm_bwd_x");
}

// Stage-1 geometry of backward-w: one CTA per SM, split into row groups of geo.threads threads.
// The 8*VPT fp32 accumulators per thread limit the CTA to 1024 threads for VPT <= 2 and 512 beyond.
static void bwd_w_geometry(int n_rows, const RowGeometry & geo, int * groups, int * grid) {
	int g = bwd_w_max_threads(geo.vpt) / geo.threads;
	if (g < 1) g = 1;
	if (g > 8) g = 8;
	while (g > 1 && g > n_rows) g /= 2;
	long long ctas = sm_count();
	const long long needed = ((long long) n_rows + g - 1) / g;
	if (ctas > needed) ctas = needed;
	if (ctas < 1) ctas = 1;
	*groups = g;
	*grid = (int) ctas;
}

extern "C" uint64_t dfb200_rms_norm_bwd_w_workspace_bytes(int n_rows, int n_cols) {
	(void) n_rows;
	if (n_cols <= 0) return 0;
	int sms = sm_count();
	if (sms <= 0) sms = 148;
	return (uint64_t) sms * (uint64_t) n_cols * sizeof(float);
}

// Stage 2 of backward-w as a programmatic dependent of the stage-1 launch before it.
static int launch_bwd_w_final(const char * op, bool sums, int fwd_dt, int bwd_dt, int n_cols, int n_partials, const float * partials, void * dW, cudaStream_t s) {
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3((n_cols + 31) / 32, 1, 1);
	cfg.blockDim = dim3(1024, 1, 1);
	cfg.stream = s;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr; cfg.numAttrs = 1;
	cudaError_t e = cudaErrorInvalidValue;
	DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
		e = (sums ? cudaLaunchKernelEx(&cfg, rms_norm_bwd_w_final_kernel<B, true>, n_cols, n_partials, partials, dW)
		          : cudaLaunchKernelEx(&cfg, rms_norm_bwd_w_final_kernel<B, false>, n_cols, n_partials, partials, dW)));
	if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e)); }
	return DFB200_OK;
}

static int launch_rms_norm_bwd_w(bool sums, int fwd_dt, int bwd_dt, int n_rows, int n_cols, const float * fwd_rms_vals, const void * X_inp,
                                 const void * upstream_dX, void * dW, void * workspace, uint64_t workspace_bytes, void * stream) {
	if (!valid_fwd_bwd_pair(fwd_dt, bwd_dt)) return set_error(DFB200_ERR_DTYPE, "rms_norm_bwd_w: unsupported datatype pair (%d, %d)", fwd_dt, bwd_dt);
	RowGeometry geo;
	bool packets;
	int rc = check_rows("rms_norm_bwd_w", n_rows, n_cols, BWD_W_ROW_THREADS, &geo, &packets);
	if (rc) return rc;
	if (n_rows == 0) return DFB200_OK;
	if (!fwd_rms_vals || !X_inp || !upstream_dX || !dW) return set_error(DFB200_ERR_ARG, "rms_norm_bwd_w: NULL tensor argument");
	if (!elem_aligned(X_inp, fwd_dt) || !elem_aligned(upstream_dX, bwd_dt) || !elem_aligned(dW, sums ? DATAFLOW_FP32 : bwd_dt))
		return set_error(DFB200_ERR_ARG, "rms_norm_bwd_w: tensors must be aligned to their element size");
	packets = packets && aligned16(X_inp) && aligned16(upstream_dX);
	int groups = 1, grid;
	if (packets) {
		bwd_w_geometry(n_rows, geo, &groups, &grid);
	} else {
		grid = sm_count() > 0 ? sm_count() : 1;
		if (grid > n_rows) grid = n_rows;
	}
	const uint64_t need = (uint64_t) grid * (uint64_t) n_cols * sizeof(float);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "rms_norm_bwd_w: needs %llu bytes of 16-byte aligned workspace, got %llu",
		                 (unsigned long long) need, (unsigned long long) workspace_bytes);
	const size_t smem = (size_t) (groups - 1) * n_cols * sizeof(float);
	if (smem > 200 * 1024) return set_error(DFB200_ERR_ARG, "rms_norm_bwd_w: n_cols = %d too large", n_cols);
	cudaStream_t s = (cudaStream_t) stream;
	float * partials = reinterpret_cast<float *>(workspace);
	if (packets) {
		DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B, DFB200_DISPATCH_VPT(geo.vpt, VPT, {
			auto kernel = rms_norm_bwd_w_partial_kernel<F, B, VPT>;
			allow_dyn_smem(reinterpret_cast<const void *>(kernel), smem);
			launch_pdl(kernel, dim3(grid), dim3(groups * geo.threads), smem, s, n_rows, n_cols, geo.threads, fwd_rms_vals, X_inp, upstream_dX, partials);
		}));
	} else {
		DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
			(launch_pdl(rms_norm_bwd_w_partial_general_kernel<F, B>, dim3(grid), dim3(GENERAL_THREADS), 0, s, n_rows, n_cols, fwd_rms_vals, X_inp, upstream_dX, partials)));
	}
	rc = check_launch("rms_norm_bwd_w (partial sums)");
	if (rc) return rc;
	return launch_bwd_w_final("rms_norm_bwd_w (final sum)", sums, fwd_dt, bwd_dt, n_cols, grid, partials, dW, s);
}

// rms_norm_bwd_x and rms_norm_bwd_w in one call: one pass over X and dY (rms_norm_bwd_xw_partial_kernel) where the row length and
// the alignment allow the packet kernels, the two separate general-shape paths otherwise. dX is what rms_norm_bwd_x gives, bit for
// bit; dW differs from rms_norm_bwd_w's only by the order of the fp32 additions (rows are dealt to the row groups in another order).
static int launch_rms_norm_bwd_xw(bool sums, int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_weighted_sums,
                                  const float * fwd_rms_vals, const void * rms_weight, const void * X_inp, const void * upstream_dX, void * dX,
                                  void * dW, void * workspace, uint64_t workspace_bytes, void * stream) {
	const char * op = sums ? "rms_norm_bwd_x_w_sums" : "rms_norm_bwd_x_w";
	if (!valid_fwd_bwd_pair(fwd_dt, bwd_dt)) return set_error(DFB200_ERR_DTYPE, "%s: unsupported datatype pair (%d, %d)", op, fwd_dt, bwd_dt);
	RowGeometry geo;
	bool packets;
	int rc = check_rows(op, n_rows, n_cols, BWD_W_ROW_THREADS, &geo, &packets);
	if (rc) return rc;
	if (n_rows == 0 && !sums) return DFB200_OK;
	packets = packets && n_rows > 0 && aligned16(rms_weight) && aligned16(X_inp) && aligned16(upstream_dX) && aligned16(dX);
	int groups = 1, grid = 1;
	if (packets) bwd_w_geometry(n_rows, geo, &groups, &grid);
	const size_t smem = (size_t) (groups - 1) * n_cols * sizeof(float);
	if (!packets || smem > 200 * 1024) {
		rc = dfb200_rms_norm_bwd_x(fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, stream);
		if (rc) return rc;
		return sums ? dfb200_rms_norm_bwd_w_sums(fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, static_cast<float *>(dW), workspace, workspace_bytes, stream)
		            : dfb200_rms_norm_bwd_w(fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, dW, workspace, workspace_bytes, stream);
	}
	if (!fwd_weighted_sums || !fwd_rms_vals || !rms_weight || !X_inp || !upstream_dX || !dX || !dW) return set_error(DFB200_ERR_ARG, "%s: NULL tensor argument", op);
	if (!elem_aligned(dW, sums ? DATAFLOW_FP32 : bwd_dt)) return set_error(DFB200_ERR_ARG, "%s: tensors must be aligned to their element size", op);
	// one fp32 row of partial sums per CTA, and neither form launches more CTAs than SMs or rows
	const uint64_t need = (uint64_t) (sm_count() < n_rows ? (sm_count() > 0 ? sm_count() : 1) : n_rows) * (uint64_t) n_cols * sizeof(float);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "%s: needs %llu bytes of 16-byte aligned workspace, got %llu", op, (unsigned long long) need,
		                 (unsigned long long) workspace_bytes);
	cudaStream_t s = (cudaStream_t) stream;
	float * partials = reinterpret_cast<float *>(workspace);
	// Staged form: rows are multiples of 16 bytes in both types (bulk copies), the row group fits 512 threads, and at least two row
	// slots per group fit the ring.
	{
		const size_t stage_bytes = (size_t) n_cols * (dtype_size(fwd_dt) + 2 * dtype_size(bwd_dt));
		unsigned int * status = kernel_status_word(STATUS_RMS);
		int sgroups = XW_STAGED_THREADS / geo.threads;
		if (sgroups > 8) sgroups = 8;                            // the groups synchronise on named barriers 1 .. groups
		while (sgroups > 1 && (sgroups > n_rows || XW_RING_BUDGET / (sgroups * stage_bytes) < 2)) sgroups /= 2;
		int stages = sgroups >= 1 ? (int) (XW_RING_BUDGET / ((size_t) sgroups * stage_bytes)) : 0;
		if (stages > XW_MAX_STAGES) stages = XW_MAX_STAGES;
		if (status && sgroups >= 1 && stages >= 2 && ((size_t) n_cols * dtype_size(fwd_dt)) % 16 == 0 && ((size_t) n_cols * dtype_size(bwd_dt)) % 16 == 0 &&
		    geo.threads <= XW_STAGED_THREADS && aligned16(X_inp) && aligned16(upstream_dX) && aligned16(dX)) {
			long long sgrid = sm_count();
			const long long needed = ((long long) n_rows + sgroups - 1) / sgroups;
			if (sgrid > needed) sgrid = needed;
			if (sgrid < 1) sgrid = 1;
			const size_t ssmem = (size_t) sgroups * stages * stage_bytes + (size_t) sgroups * stages * sizeof(uint64_t);
			DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B, DFB200_DISPATCH_VPT(geo.vpt, VPT, {
				auto kernel = rms_norm_bwd_xw_staged_kernel<F, B, VPT>;
				allow_dyn_smem(reinterpret_cast<const void *>(kernel), ssmem);
				launch_pdl(kernel, dim3((unsigned) sgrid), dim3(sgroups * geo.threads), ssmem, s, n_rows, n_cols, geo.threads, stages, fwd_weighted_sums, fwd_rms_vals,
				           rms_weight, X_inp, upstream_dX, dX, partials, status);
			}));
			rc = check_launch(op);
			if (rc) return rc;
			return launch_bwd_w_final(op, sums, fwd_dt, bwd_dt, n_cols, (int) sgrid, partials, dW, s);
		}
	}
	DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B, DFB200_DISPATCH_VPT(geo.vpt, VPT, {
		auto kernel = rms_norm_bwd_xw_partial_kernel<F, B, VPT>;
		allow_dyn_smem(reinterpret_cast<const void *>(kernel), smem);
		launch_pdl(kernel, dim3(grid), dim3(groups * geo.threads), smem, s, n_rows, n_cols, geo.threads, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp,
		           upstream_dX, dX, partials);
	}));
	rc = check_launch(op);
	if (rc) return rc;
	return launch_bwd_w_final(op, sums, fwd_dt, bwd_dt, n_cols, grid, partials, dW, s);
}

extern "C" int dfb200_rms_norm_bwd_x_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_weighted_sums,
                                       const float * fwd_rms_vals, const void * rms_weight, const void * X_inp, const void * upstream_dX,
                                       void * dX, void * dW, void * workspace, uint64_t workspace_bytes, void * stream) {
	return launch_rms_norm_bwd_xw(false, fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, dW, workspace,
	                              workspace_bytes, stream);
}

extern "C" int dfb200_rms_norm_bwd_x_w_sums(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_weighted_sums,
                                            const float * fwd_rms_vals, const void * rms_weight, const void * X_inp, const void * upstream_dX,
                                            void * dX, float * column_sums, void * workspace, uint64_t workspace_bytes, void * stream) {
	return launch_rms_norm_bwd_xw(true, fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, column_sums,
	                              workspace, workspace_bytes, stream);
}

extern "C" int dfb200_rms_norm_bwd_w(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_rms_vals,
                                     const void * X_inp, const void * upstream_dX, void * dW, void * workspace, uint64_t workspace_bytes,
                                     void * stream) {
	(void) eps;
	return launch_rms_norm_bwd_w(false, fwd_dt, bwd_dt, n_rows, n_cols, fwd_rms_vals, X_inp, upstream_dX, dW, workspace, workspace_bytes, stream);
}

extern "C" int dfb200_rms_norm_bwd_w_sums(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_rms_vals,
                                          const void * X_inp, const void * upstream_dX, float * column_sums, void * workspace,
                                          uint64_t workspace_bytes, void * stream) {
	(void) eps;
	if (reinterpret_cast<uintptr_t>(column_sums) & 3u) return set_error(DFB200_ERR_ARG, "rms_norm_bwd_w_sums: column_sums must be 4-byte aligned");
	if (n_rows == 0 && n_cols > 0 && column_sums) {          // no rows: the sums are zero (the accumulating form leaves dW alone instead)
		cudaError_t e = cudaMemsetAsync(column_sums, 0, (size_t) n_cols * sizeof(float), (cudaStream_t) stream);
		if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "rms_norm_bwd_w_sums: %s", cudaGetErrorString(e)); }
		return DFB200_OK;
	}
	return launch_rms_norm_bwd_w(true, fwd_dt, bwd_dt, n_rows, n_cols, fwd_rms_vals, X_inp, upstream_dX, column_sums, workspace, workspace_bytes, stream);
}

// ----------------------------------------------------------------------------------------
// rms_norm_bwd_w for callers that must not allocate
// ----------------------------------------------------------------------------------------
// Some callers cannot give this op a workspace: programs that handed the whole device to their own arena with
// one bulk alloc_mem() at start-up (the memory model the handle interface is built around) and have nothing left
// to carve scratch from, and code running where cudaMalloc is off limits because it synchronises the whole device
// (a latency-critical step loop, other streams mid-flight). For them the partial column sums live in this
// fixed array, which every GPU that loads the library holds from load until exit.
constexpr int STATIC_SCRATCH_FLOATS = 160 * 8192;      // 5 MiB: n_SM * n_cols must fit, e.g. 8192 columns on up to 160 SMs
static __device__ __align__(256) float g_bwd_w_static_scratch[STATIC_SCRATCH_FLOATS];

// Same arithmetic, kernels and results as dfb200_rms_norm_bwd_w, with the scratch taken from the array above instead
// of a caller workspace. It calls no cudaMalloc, cudaFree or allocating library routine.
//  * The first call on each device (more exactly: in each CUDA context, for programs that make contexts of their own) looks up
//    the array's device address (cudaGetSymbolAddress, with that device current) and remembers it; make that first call
//    outside any stream capture.
//  * Limit: n_SM * n_cols <= 1,310,720 floats (n_cols <= 8192 on a 148-SM B200); larger shapes are rejected
//    with DFB200_ERR_WORKSPACE and a message, never truncated.
//  * All calls on a device share the one array and it keeps the previous call's contents. Nothing in it has to
//    start at zero (stage 1 overwrites every partial row that stage 2 reads), but two calls that overlap on the
//    GPU (different streams, no dependency between them) race on it: order them.
extern "C" int dfb200_rms_norm_bwd_w_static(int fwd_dt, int bwd_dt, int n_rows, int n_cols, float eps, const float * fwd_rms_vals,
                                            const void * X_inp, const void * upstream_dX, void * dW, void * stream) {
	int dev = -1;
	cudaError_t e = cudaGetDevice(&dev);
	if (e != cudaSuccess || dev < 0) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "rms_norm_bwd_w_static: no current device (%s)", cudaGetErrorString(e)); }
	// in host code the array's name is only a handle for the runtime, not a device address: symbol_address asks the runtime
	// (cudaGetSymbolAddress, return code checked) once per context and remembers the answer
	float * scratch = static_cast<float *>(symbol_address(g_bwd_w_static_scratch));
	if (!scratch) return set_error(DFB200_ERR_CUDA, "rms_norm_bwd_w_static: cudaGetSymbolAddress failed for the built-in scratch array");
	const uint64_t capacity = (uint64_t) STATIC_SCRATCH_FLOATS * sizeof(float);
	const uint64_t need = dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols);
	if (need > capacity)
		return set_error(DFB200_ERR_WORKSPACE, "rms_norm_bwd_w_static: n_cols = %d needs %llu bytes of scratch on this device, the built-in array holds %llu "
		                 "(n_SM * n_cols <= %d); use dfb200_rms_norm_bwd_w with a caller workspace", n_cols, (unsigned long long) need,
		                 (unsigned long long) capacity, STATIC_SCRATCH_FLOATS);
	return dfb200_rms_norm_bwd_w(fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, dW, scratch, capacity, stream);
}
