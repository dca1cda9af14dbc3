// SwiGLU forward and backward: pure streaming kernels (3 resp. 5 tensors, each touched once).
// Every thread owns UNROLL chunks of 8 consecutive elements and issues all its loads before the
// first use. Measured on B200 (8192 x 14336 bf16): one chunk per thread with 2048 resident
// threads per SM reaches ~7.0 TB/s, while unrolling to 4 chunks per thread costs occupancy and
// drops to 4.8 TB/s -- bytes in flight come from resident warps, not from per-thread unrolling.
// The row structure is irrelevant (tensors are contiguous), so the kernels index the flat
// element range.
#include "common.cuh"

namespace dfb200 {

constexpr int E = 8;                       // elements per chunk
// launch shapes chosen by measurement on B200 (threads per CTA, chunks per thread)
constexpr int SWIGLU_FWD_THREADS = 512, SWIGLU_FWD_UNROLL = 1;
constexpr int SWIGLU_BWD_THREADS = 512, SWIGLU_BWD_UNROLL = 1;

// exp and divide are the approximate hardware forms (ex2.approx / rcp.approx based), the same
// ones the reference build selects with --use_fast_math (src/ops/nvidia/Makefile:3-5).
__device__ __forceinline__ float silu_and_e(float x, float & e) {
	e = __expf(-x);
	return __fdividef(x, 1.0f + e);
}

template <typename F, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
swiglu_fwd_kernel(uint64_t n_chunks, const void * __restrict__ x_w1, const void * __restrict__ x_w3, void * __restrict__ out) {
	pdl_prologue();
	const uint64_t first = (uint64_t) blockIdx.x * (THREADS * UNROLL) + threadIdx.x;
	float a[UNROLL][E], b[UNROLL][E];
	#pragma unroll
	for (int u = 0; u < UNROLL; u++) {
		const uint64_t c = first + (uint64_t) u * THREADS;
		if (c < n_chunks) {
			load_elems<F, E, Hint::KEEP>(x_w1, c * E, a[u]);     // no evict-first hint: the backward op reads these again (from their end)
			load_elems<F, E, Hint::KEEP>(x_w3, c * E, b[u]);
		}
	}
	#pragma unroll
	for (int u = 0; u < UNROLL; u++) {
		const uint64_t c = first + (uint64_t) u * THREADS;
		if (c < n_chunks) {
			float o[E];
			#pragma unroll
			for (int i = 0; i < E; i++) { float e; o[i] = silu_and_e(a[u][i], e) * b[u][i]; }
			store_elems<F, E>(out, c * E, o);
		}
	}
}

// Reference arithmetic (src/ops/nvidia/activations/swiglu_bwd_x.cu:68-77), kept term for term:
//   dX_w3 = dY * silu(x1);   dX_w1 = dY * ( (x3 * (1 + e + x1*e)) / ((1+e)*(1+e)) ),  e = exp(-x1)
template <typename F, typename B, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
swiglu_bwd_x_kernel(uint64_t n_chunks, const void * __restrict__ x_w1, const void * __restrict__ x_w3,
                    const void * __restrict__ upstream_dX, void * __restrict__ dX_w1, void * __restrict__ dX_w3) {
	// The tensors are walked from their END: in a layer's forward-then-backward sequence the tail of x_w1 and x_w3 is what the forward
	// kernel left in L2.
	const uint64_t first = (uint64_t) blockIdx.x * (THREADS * UNROLL) + threadIdx.x, last = n_chunks - 1;
	cudaTriggerProgrammaticLaunchCompletion();
	#pragma unroll
	for (int u = 0; u < UNROLL; u++) {                 // while the previous kernel of the stream drains: this thread's lines on their way to L2
		const uint64_t c = last - (first + (uint64_t) u * THREADS);
		if (c < n_chunks) {
			prefetch_l2(reinterpret_cast<const char *>(x_w1) + c * (E * (4 / Word<F>::EPW)));
			prefetch_l2(reinterpret_cast<const char *>(x_w3) + c * (E * (4 / Word<F>::EPW)));
			prefetch_l2(reinterpret_cast<const char *>(upstream_dX) + c * (E * (4 / Word<B>::EPW)));
		}
	}
	cudaGridDependencySynchronize();
	float a[UNROLL][E], b[UNROLL][E], g[UNROLL][E];
	#pragma unroll
	for (int u = 0; u < UNROLL; u++) {
		const uint64_t c = last - (first + (uint64_t) u * THREADS);        // c < n_chunks also rejects the wrapped values
		if (c < n_chunks) {
			load_elems<F, E>(x_w1, c * E, a[u]);
			load_elems<F, E>(x_w3, c * E, b[u]);
			load_elems<B, E>(upstream_dX, c * E, g[u]);
		}
	}
	#pragma unroll
	for (int u = 0; u < UNROLL; u++) {
		const uint64_t c = last - (first + (uint64_t) u * THREADS);        // c < n_chunks also rejects the wrapped values
		if (c < n_chunks) {
			float d1[E], d3[E];
			#pragma unroll
			for (int i = 0; i < E; i++) {
				float e;
				const float x1 = a[u][i];
				const float s = silu_and_e(x1, e);
				const float ope = 1.0f + e;
				d3[i] = g[u][i] * s;
				d1[i] = g[u][i] * __fdividef(b[u][i] * (ope + x1 * e), ope * ope);
			}
			store_elems<B, E>(dX_w1, c * E, d1);
			store_elems<B, E>(dX_w3, c * E, d3);
		}
	}
}

// General shapes: any element count, tensors aligned to their element size only (what the reference's element-per-thread kernels
// accept, src/ops/nvidia/activations/swiglu.cu:48-68). One element per thread, same arithmetic as the packet kernels.
constexpr int GENERAL_THREADS = 256;

template <typename F>
__global__ void __launch_bounds__(GENERAL_THREADS)
swiglu_fwd_general_kernel(uint64_t n, const void * __restrict__ x_w1, const void * __restrict__ x_w3, void * __restrict__ out) {
	pdl_prologue();
	for (uint64_t i = (uint64_t) blockIdx.x * GENERAL_THREADS + threadIdx.x; i < n; i += (uint64_t) gridDim.x * GENERAL_THREADS) {
		float e;
		store_one<F>(out, i, silu_and_e(load_one<F>(x_w1, i), e) * load_one<F>(x_w3, i));
	}
}

template <typename F, typename B>
__global__ void __launch_bounds__(GENERAL_THREADS)
swiglu_bwd_x_general_kernel(uint64_t n, const void * __restrict__ x_w1, const void * __restrict__ x_w3, const void * __restrict__ upstream_dX,
                            void * __restrict__ dX_w1, void * __restrict__ dX_w3) {
	pdl_prologue();
	for (uint64_t i = (uint64_t) blockIdx.x * GENERAL_THREADS + threadIdx.x; i < n; i += (uint64_t) gridDim.x * GENERAL_THREADS) {
		float e;
		const float x1 = load_one<F>(x_w1, i), x3 = load_one<F>(x_w3, i), g = load_one<B>(upstream_dX, i);
		const float s = silu_and_e(x1, e), ope = 1.0f + e;
		store_one<B>(dX_w3, i, g * s);
		store_one<B>(dX_w1, i, g * __fdividef(x3 * (ope + x1 * e), ope * ope));
	}
}

static unsigned general_grid(uint64_t n) {
	const uint64_t blocks = (n + GENERAL_THREADS - 1) / GENERAL_THREADS, cap = (uint64_t) (sm_count() > 0 ? sm_count() : 1) * 32;
	return (unsigned) (blocks < cap ? (blocks ? blocks : 1) : cap);
}

// *packets = true: every tensor is 16-byte aligned and the element count is a multiple of 8 (the packet kernels); false: the general kernels.
static int check_elementwise(const char * op, int num_rows, int num_cols, uint64_t * n_elems, bool * packets, int n_ptrs, const void * const * ptrs,
                             const int * elem_sizes) {
	if (num_rows < 0 || num_cols < 0) return set_error(DFB200_ERR_ARG, "%s: negative shape %d x %d", op, num_rows, num_cols);
	const uint64_t n = (uint64_t) num_rows * (uint64_t) num_cols;
	*packets = n % E == 0;
	for (int i = 0; i < n_ptrs; i++) {
		if (n && !ptrs[i]) return set_error(DFB200_ERR_ARG, "%s: NULL tensor argument %d", op, i);
		if (reinterpret_cast<uintptr_t>(ptrs[i]) % (uintptr_t) elem_sizes[i])
			return set_error(DFB200_ERR_ARG, "%s: tensor argument %d is not aligned to its element size", op, i);
		if (!aligned16(ptrs[i])) *packets = false;
	}
	*n_elems = n;
	return DFB200_OK;
}

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_swiglu(int fwd_dt, int num_rows, int num_cols, const void * x_w1, const void * x_w3, void * out, void * stream) {
	const int es = dtype_size(fwd_dt);
	if (!es) return set_error(DFB200_ERR_DTYPE, "swiglu: unsupported datatype %d", fwd_dt);
	uint64_t n;
	bool packets;
	const void * ptrs[3] = {x_w1, x_w3, out};
	const int sizes[3] = {es, es, es};
	int rc = check_elementwise("swiglu", num_rows, num_cols, &n, &packets, 3, ptrs, sizes);
	if (rc || n == 0) return rc;
	if (!packets) {
		DFB200_DISPATCH_DTYPE(fwd_dt, F,
			(launch_pdl(swiglu_fwd_general_kernel<F>, dim3(general_grid(n)), dim3(GENERAL_THREADS), 0, (cudaStream_t) stream, n, x_w1, x_w3, out)));
		return check_launch("swiglu (general shape)");
	}
	const uint64_t n_chunks = n / E;
	constexpr int THREADS = SWIGLU_FWD_THREADS, UNROLL = SWIGLU_FWD_UNROLL;
	const uint64_t blocks = (n_chunks + THREADS * UNROLL - 1) / (THREADS * UNROLL);
	if (blocks > 0x7fffffffull) return set_error(DFB200_ERR_ARG, "swiglu: tensor too large");
	DFB200_DISPATCH_DTYPE(fwd_dt, F,
		(launch_pdl(swiglu_fwd_kernel<F, THREADS, UNROLL>, dim3((unsigned) blocks), dim3(THREADS), 0, (cudaStream_t) stream, n_chunks, x_w1, x_w3, out)));
	return check_launch("swiglu");
}

extern "C" int dfb200_swiglu_bwd_x(int fwd_dt, int bwd_dt, int num_rows, int num_cols, const void * x_w1, const void * x_w3,
                                   const void * upstream_dX, void * dX_w1, void * dX_w3, void * stream) {
	if (!valid_fwd_bwd_pair(fwd_dt, bwd_dt)) return set_error(DFB200_ERR_DTYPE, "swiglu_bwd_x: unsupported datatype pair (%d, %d)", fwd_dt, bwd_dt);
	uint64_t n;
	bool packets;
	const void * ptrs[5] = {x_w1, x_w3, upstream_dX, dX_w1, dX_w3};
	const int fs = dtype_size(fwd_dt), bs = dtype_size(bwd_dt);
	const int sizes[5] = {fs, fs, bs, bs, bs};
	int rc = check_elementwise("swiglu_bwd_x", num_rows, num_cols, &n, &packets, 5, ptrs, sizes);
	if (rc || n == 0) return rc;
	if (!packets) {
		DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
			(launch_pdl(swiglu_bwd_x_general_kernel<F, B>, dim3(general_grid(n)), dim3(GENERAL_THREADS), 0, (cudaStream_t) stream, n, x_w1, x_w3, upstream_dX, dX_w1, dX_w3)));
		return check_launch("swiglu_bwd_x (general shape)");
	}
	const uint64_t n_chunks = n / E;
	constexpr int THREADS = SWIGLU_BWD_THREADS, UNROLL = SWIGLU_BWD_UNROLL;
	const uint64_t blocks = (n_chunks + THREADS * UNROLL - 1) / (THREADS * UNROLL);
	if (blocks > 0x7fffffffull) return set_error(DFB200_ERR_ARG, "swiglu_bwd_x: tensor too large");
	DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
		(launch_pdl(swiglu_bwd_x_kernel<F, B, THREADS, UNROLL>, dim3((unsigned) blocks), dim3(THREADS), 0, (cudaStream_t) stream, n_chunks, x_w1, x_w3, upstream_dX, dX_w1, dX_w3)));
	return check_launch("swiglu_bwd_x");
}
