// Mixture-of-experts router: per token, sigmoid scores of the router logits, the top-k experts, their normalised
// weights, and the per-expert token counts with their inclusive prefix sum.
//
// Semantics follow the reference kernel (src/ops/nvidia/moe/select_experts.cu:3-239) exactly where they are
// observable:
//   * score_e = 1 / (1 + exp(-x_e)), computed as fp32 add, then a double-precision division rounded to fp32 (the
//     reference writes `1.0 / (1 + expf(..))`, :112);
//   * k slots start at (-inf, id 0xFFFF); experts are scanned in index order and expert e replaces the slot that
//     currently holds the minimum iff score_e > that minimum (strict: on equal scores the earlier expert stays);
//     after a replacement the minimum is searched again from slot 0 with a strict `<` (the earliest slot among
//     equal minima). The order of a token's experts in the output is therefore the slot order, not sorted (:131-153);
//   * the sum of the selected scores is maintained incrementally in fp32 (subtract the evicted score, add the new
//     one, :131-137) and weight_j = score_j / sum, rounded to the tensor's datatype (:164);
//   * expert_counts[e] += tokens routed to e (the caller zeroes it, as with the reference's atomicAdd, :185),
//     expert_counts_cumsum = inclusive prefix sum of expert_counts, num_routed_by_expert[e] = 0 (:226-236);
//     expert_counts has n_experts + 1 entries, the last one is the kernel's block counter and is left at 0.
//
// Differences: (1) exp is a fixed sequence of IEEE fp32 operations (Cody-Waite reduction + degree-5 polynomial,
// below) instead of the hardware approximation the reference's fast-math build uses, and the final division is
// IEEE, so that the CPU oracle reproduces every score bit for bit and the chosen expert ids are bit-exact
// against it; against the reference binary the scores differ by a few units in the last place.
// (2) The reference's block 0 spins, unbounded, until every block has added its counts (:198-202), which
// deadlocks when the grid exceeds what is resident. Here the LAST block to finish (a ticket from the same
// counter) computes the prefix sum: nothing waits.
// (3) One thread owns one token (slots in registers for k <= 8); the reference gives a warp to a token and lets
// lane 0 do the scan.
#include "common.cuh"

#include <math_constants.h>

namespace dfb200 {

constexpr int SELECT_THREADS = 128;

// exp(x) from IEEE operations only (no contraction: every operation is an explicit round-to-nearest intrinsic).
__device__ __forceinline__ float det_expf(float x) {
	x = fminf(fmaxf(x, -87.0f), 88.0f);
	const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
	float r = __fmaf_rn(n, -0.693359375f, x);
	r = __fmaf_rn(n, 2.12194440e-4f, r);
	float p = 1.9875691500e-4f;
	p = __fmaf_rn(p, r, 1.3981999507e-3f);
	p = __fmaf_rn(p, r, 8.3334519073e-3f);
	p = __fmaf_rn(p, r, 4.1665795894e-2f);
	p = __fmaf_rn(p, r, 1.6666665459e-1f);
	p = __fmaf_rn(p, r, 5.0000001201e-1f);
	const float r2 = __fmul_rn(r, r);
	const float e = __fadd_rn(__fmaf_rn(p, r2, r), 1.0f);
	return __fmul_rn(e, __int_as_float(((int) n + 127) << 23));
}

__device__ __forceinline__ float sigmoid_score(float x) {
	const float denom = __fadd_rn(1.0f, det_expf(-x));
	return (float) __ddiv_rn(1.0, (double) denom);
}

template <typename T> __device__ __forceinline__ float load_one(const void * p, uint64_t i);
template <> __device__ __forceinline__ float load_one<f32_t>(const void * p, uint64_t i) { return static_cast<const float *>(p)[i]; }
template <> __device__ __forceinline__ float load_one<f16_t>(const void * p, uint64_t i) { return __half2float(static_cast<const __half *>(p)[i]); }
template <> __device__ __forceinline__ float load_one<bf16_t>(const void * p, uint64_t i) { return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]); }
template <> __device__ __forceinline__ float load_one<e4m3_t>(const void * p, uint64_t i) {
	float f[4]; Word<e4m3_t>::unpack(static_cast<const uint8_t *>(p)[i], f); return f[0];
}
template <> __device__ __forceinline__ float load_one<e5m2_t>(const void * p, uint64_t i) {
	float f[4]; Word<e5m2_t>::unpack(static_cast<const uint8_t *>(p)[i], f); return f[0];
}
template <typename T> __device__ __forceinline__ void store_one(void * p, uint64_t i, float v);
template <> __device__ __forceinline__ void store_one<f32_t>(void * p, uint64_t i, float v) { static_cast<float *>(p)[i] = v; }
template <> __device__ __forceinline__ void store_one<f16_t>(void * p, uint64_t i, float v) { static_cast<__half *>(p)[i] = __float2half_rn(v); }
template <> __device__ __forceinline__ void store_one<bf16_t>(void * p, uint64_t i, float v) { static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store_one<e4m3_t>(void * p, uint64_t i, float v) {
	static_cast<uint8_t *>(p)[i] = (uint8_t) __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
template <> __device__ __forceinline__ void store_one<e5m2_t>(void * p, uint64_t i, float v) {
	static_cast<uint8_t *>(p)[i] = (uint8_t) __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2);
}

// K = compile-time slot capacity (top_k <= K). Slots are registers: every access is an unrolled select.
template <typename T, int K>
__global__ void __launch_bounds__(SELECT_THREADS)
select_experts_kernel(int total_tokens, int n_experts, int top_k, const void * __restrict__ X_routed, void * __restrict__ token_expert_weights,
                      uint16_t * __restrict__ chosen_experts, int * expert_counts, int * __restrict__ expert_counts_cumsum,
                      int * __restrict__ num_routed_by_expert) {
	extern __shared__ int s_counts[];          // n_experts block-local counts
	__shared__ int s_last;
	for (int e = threadIdx.x; e < n_experts; e += SELECT_THREADS) s_counts[e] = 0;
	__syncthreads();

	const int tok = blockIdx.x * SELECT_THREADS + threadIdx.x;
	if (tok < total_tokens) {
		float vals[K];
		int ids[K];
		#pragma unroll
		for (int k = 0; k < K; k++) { vals[k] = -CUDART_INF_F; ids[k] = 0xFFFF; }
		float min_val = -CUDART_INF_F, sum = 0.0f;
		int min_slot = 0;
		const uint64_t base = (uint64_t) tok * (uint64_t) n_experts;
		for (int e = 0; e < n_experts; e++) {
			const float score = sigmoid_score(load_one<T>(X_routed, base + e));
			if (score > min_val) {
				float evicted = 0.0f;
				#pragma unroll
				for (int k = 0; k < K; k++)
					if (k == min_slot) { evicted = vals[k]; vals[k] = score; ids[k] = e; }
				if (evicted != -CUDART_INF_F) sum = __fsub_rn(sum, evicted);
				sum = __fadd_rn(sum, score);
				min_val = CUDART_INF_F;
				#pragma unroll
				for (int k = 0; k < K; k++)
					if (k < top_k && vals[k] < min_val) { min_val = vals[k]; min_slot = k; }
			}
		}
		const uint64_t out = (uint64_t) tok * (uint64_t) top_k;
		#pragma unroll
		for (int k = 0; k < K; k++) {
			if (k < top_k) {
				store_one<T>(token_expert_weights, out + k, __fdiv_rn(vals[k], sum));
				chosen_experts[out + k] = (uint16_t) ids[k];
				if (ids[k] < n_experts) atomicAdd(&s_counts[ids[k]], 1);
			}
		}
	}
	__syncthreads();

	for (int e = threadIdx.x; e < n_experts; e += SELECT_THREADS)
		if (s_counts[e]) atomicAdd(&expert_counts[e], s_counts[e]);
	__threadfence();
	__syncthreads();
	if (threadIdx.x == 0) s_last = atomicAdd(&expert_counts[n_experts], 1) == (int) gridDim.x - 1;
	__syncthreads();
	if (!s_last) return;

	// last block: every other block's counts are visible (their fence precedes their ticket)
	__threadfence();
	if (threadIdx.x < 32) {
		const int lane = threadIdx.x;
		int carry = 0;
		for (int e0 = 0; e0 < n_experts; e0 += 32) {
			const int e = e0 + lane;
			int c = e < n_experts ? __ldcg(expert_counts + e) : 0;
			#pragma unroll
			for (int off = 1; off < 32; off <<= 1) {
				const int t = __shfl_up_sync(0xffffffffu, c, off);
				if (lane >= off) c += t;
			}
			if (e < n_experts) { expert_counts_cumsum[e] = carry + c; num_routed_by_expert[e] = 0; }
			carry += __shfl_sync(0xffffffffu, c, 31);
		}
		if (lane == 0) expert_counts[n_experts] = 0;
	}
}

template <typename T>
static int launch_select(int total_tokens, int n_experts, int top_k, const void * X, void * w, uint16_t * ids, int * counts, int * cumsum, int * routed,
                         cudaStream_t s) {
	const unsigned grid = (unsigned) ((total_tokens + SELECT_THREADS - 1) / SELECT_THREADS);
	const size_t smem = (size_t) n_experts * sizeof(int);
	if (top_k <= 2)       select_experts_kernel<T, 2><<<grid, SELECT_THREADS, smem, s>>>(total_tokens, n_experts, top_k, X, w, ids, counts, cumsum, routed);
	else if (top_k <= 4)  select_experts_kernel<T, 4><<<grid, SELECT_THREADS, smem, s>>>(total_tokens, n_experts, top_k, X, w, ids, counts, cumsum, routed);
	else if (top_k <= 8)  select_experts_kernel<T, 8><<<grid, SELECT_THREADS, smem, s>>>(total_tokens, n_experts, top_k, X, w, ids, counts, cumsum, routed);
	else if (top_k <= 16) select_experts_kernel<T, 16><<<grid, SELECT_THREADS, smem, s>>>(total_tokens, n_experts, top_k, X, w, ids, counts, cumsum, routed);
	else                  select_experts_kernel<T, 32><<<grid, SELECT_THREADS, smem, s>>>(total_tokens, n_experts, top_k, X, w, ids, counts, cumsum, routed);
	return check_launch("select_experts");
}

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_select_experts(int dt, int total_tokens, int n_experts, int top_k_experts, const void * X_routed, void * token_expert_weights,
                                     uint16_t * chosen_experts, int * expert_counts, int * expert_counts_cumsum, int * num_routed_by_expert, void * stream) {
	if (total_tokens <= 0 || n_experts <= 0 || n_experts > 8192 || top_k_experts <= 0 || top_k_experts > 32 || top_k_experts > n_experts)
		return set_error(DFB200_ERR_ARG, "select_experts: bad shape (%d tokens, %d experts, top %d); 1 <= top_k <= min(32, n_experts), n_experts <= 8192",
		                 total_tokens, n_experts, top_k_experts);
	if (!X_routed || !token_expert_weights || !chosen_experts || !expert_counts || !expert_counts_cumsum || !num_routed_by_expert)
		return set_error(DFB200_ERR_ARG, "select_experts: NULL pointer");
	const int es = dtype_size(dt);
	if (!es) return set_error(DFB200_ERR_DTYPE, "select_experts: unsupported datatype %d", dt);
	if ((reinterpret_cast<uintptr_t>(X_routed) & (es - 1)) || (reinterpret_cast<uintptr_t>(token_expert_weights) & (es - 1)) ||
	    (reinterpret_cast<uintptr_t>(chosen_experts) & 1u) || (reinterpret_cast<uintptr_t>(expert_counts) & 3u) ||
	    (reinterpret_cast<uintptr_t>(expert_counts_cumsum) & 3u) || (reinterpret_cast<uintptr_t>(num_routed_by_expert) & 3u))
		return set_error(DFB200_ERR_ARG, "select_experts: misaligned pointer");
	cudaStream_t s = (cudaStream_t) stream;
	switch (dt) {
		case DATAFLOW_FP32:    return launch_select<f32_t>(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum, num_routed_by_expert, s);
		case DATAFLOW_FP16:    return launch_select<f16_t>(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum, num_routed_by_expert, s);
		case DATAFLOW_BF16:    return launch_select<bf16_t>(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum, num_routed_by_expert, s);
		case DATAFLOW_FP8E4M3: return launch_select<e4m3_t>(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum, num_routed_by_expert, s);
		default:               return launch_select<e5m2_t>(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum, num_routed_by_expert, s);
	}
}
