// Rotary position embedding, forward and backward, in place on Q [tokens, model_dim] and
// K [tokens, kv_dim] (interleaved pairs; src/ops/nvidia/attention/rope.cu:137-171,
// rope_bwd_x.cu:144-172).
//
// The reference evaluates powf + sinf + cosf once per PAIR (and again for K): 40 times per
// (token, frequency) for 32+8 heads. Here a CTA keeps the head_dim/2 inverse frequencies in
// shared memory for its whole life, builds the (cos, sin) table of TOK tokens per iteration
// (one sincosf per (token, frequency)), and then streams the TOK rows of Q and K through
// registers in 128-bit packets, 4 packets in flight per thread. HBM traffic is one read and
// one write of Q and K plus the positions.
#include "common.cuh"

namespace dfb200 {

constexpr int E = 8;
constexpr int ROPE_THREADS = 256;
constexpr int ROPE_UNROLL = 4;
constexpr int ROPE_MAX_TABLE = 2048;       // (cos, sin) entries per buffer: TOK * head_dim / 2

template <typename T, bool BWD>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kernel(int tokens, int model_dim, int kv_dim, int head_dim, int tok_per_iter, float theta,
            const int * __restrict__ seq_positions, void * X_q, void * X_k) {
	extern __shared__ float smem_f[];
	const int half = head_dim >> 1;
	float * inv_freq = smem_f;                                              // [half]
	float2 * table = reinterpret_cast<float2 *>(smem_f + ((half + 3) & ~3)); // [2][tok_per_iter * half]
	const int table_len = tok_per_iter * half;
	const int tid = threadIdx.x;

	// angle_j = theta^(-(2j)/head_dim). The exponent is formed in fp32 as the reference does;
	// the power is taken in fp64 and rounded once, which gives the correctly rounded fp32 powf.
	for (int j = tid; j < half; j += ROPE_THREADS) {
		const float expo = -1.0f * ((float) (2 * j) / (float) head_dim);
		inv_freq[j] = (float) pow((double) theta, (double) expo);
	}
	__syncthreads();

	const int q_chunks = model_dim / E, k_chunks = kv_dim / E;
	const int row_chunks = q_chunks + k_chunks;
	const int chunks_per_head = head_dim / E;

	int buf = 0;
	for (int tok0 = blockIdx.x * tok_per_iter; tok0 < tokens; tok0 += gridDim.x * tok_per_iter, buf ^= 1) {
		const int n_tok = min(tok_per_iter, tokens - tok0);
		float2 * tab = table + buf * table_len;
		for (int e = tid; e < n_tok * half; e += ROPE_THREADS) {
			const int t = e / half, j = e - t * half;
			const float ang = (float) __ldg(seq_positions + tok0 + t) * inv_freq[j];
			float s, c;
			sincosf(ang, &s, &c);
			tab[e] = make_float2(c, BWD ? -s : s);
		}
		__syncthreads();     // one barrier per iteration: the other buffer is only rewritten after the next one

		const int work = n_tok * row_chunks;
		for (int i0 = tid; i0 < work; i0 += ROPE_THREADS * ROPE_UNROLL) {
			uint32_t raw[ROPE_UNROLL][E / Word<T>::EPW];
			char * addr[ROPE_UNROLL];
			int tab_off[ROPE_UNROLL];
			#pragma unroll
			for (int u = 0; u < ROPE_UNROLL; u++) {
				const int i = i0 + u * ROPE_THREADS;
				if (i < work) {
					const int t = i / row_chunks, c = i - t * row_chunks;
					const bool is_q = c < q_chunks;
					const int cc = is_q ? c : c - q_chunks;
					char * base = reinterpret_cast<char *>(is_q ? X_q : X_k);
					const uint64_t elem = (uint64_t) (tok0 + t) * (is_q ? model_dim : kv_dim) + (uint64_t) cc * E;
					addr[u] = base + elem * (4 / Word<T>::EPW);
					tab_off[u] = t * half + (cc % chunks_per_head) * (E / 2);
					ld_words<E / Word<T>::EPW, Hint::STREAM>(addr[u], raw[u]);
				}
			}
			#pragma unroll
			for (int u = 0; u < ROPE_UNROLL; u++) {
				const int i = i0 + u * ROPE_THREADS;
				if (i < work) {
					float x[E], o[E];
					#pragma unroll
					for (int k = 0; k < E / Word<T>::EPW; k++) Word<T>::unpack(raw[u][k], &x[k * Word<T>::EPW]);
					const float4 * cs = reinterpret_cast<const float4 *>(tab + tab_off[u]);
					const float4 cs01 = cs[0], cs23 = cs[1];
					const float cv[4] = {cs01.x, cs01.z, cs23.x, cs23.z};
					const float sv[4] = {cs01.y, cs01.w, cs23.y, cs23.w};
					#pragma unroll
					for (int p = 0; p < 4; p++) {
						// products are rounded separately (no fma contraction), as in the reference expression
						o[2 * p]     = __fsub_rn(__fmul_rn(cv[p], x[2 * p]),     __fmul_rn(sv[p], x[2 * p + 1]));
						o[2 * p + 1] = __fadd_rn(__fmul_rn(cv[p], x[2 * p + 1]), __fmul_rn(sv[p], x[2 * p]));
					}
					uint32_t w[E / Word<T>::EPW];
					#pragma unroll
					for (int k = 0; k < E / Word<T>::EPW; k++) w[k] = Word<T>::pack(&o[k * Word<T>::EPW]);
					st_words<E / Word<T>::EPW>(addr[u], w);
				}
			}
		}
	}
}

template <bool BWD>
static int launch_rope(const char * op, int dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                       const int * seq_positions, void * X_q, void * X_k, void * stream) {
	if (BWD ? !(dt == DATAFLOW_FP32 || dt == DATAFLOW_FP16 || dt == DATAFLOW_BF16) : !dtype_size(dt))
		return set_error(DFB200_ERR_DTYPE, "%s: unsupported datatype %d", op, dt);
	if (model_dim <= 0 || head_dim <= 0 || num_kv_heads < 0 || theta <= 0)
		return set_error(DFB200_ERR_ARG, "%s: bad dimensions (model_dim %d, head_dim %d, num_kv_heads %d, theta %d)", op, model_dim, head_dim, num_kv_heads, theta);
	if (head_dim % E || model_dim % head_dim)
		return set_error(DFB200_ERR_ARG, "%s: head_dim (%d) must be a multiple of %d and divide model_dim (%d)", op, head_dim, E, model_dim);
	if (N % (uint64_t) model_dim) return set_error(DFB200_ERR_ARG, "%s: N is not a multiple of model_dim", op);
	const uint64_t tokens64 = N / (uint64_t) model_dim;
	if (tokens64 > 0x7fffffffull) return set_error(DFB200_ERR_ARG, "%s: too many tokens", op);
	const int tokens = (int) tokens64;
	if (tokens == 0) return DFB200_OK;
	const int kv_dim = num_kv_heads * head_dim;
	if (!seq_positions || !X_q || (kv_dim && !X_k)) return set_error(DFB200_ERR_ARG, "%s: NULL tensor argument", op);
	if (!aligned16(X_q) || !aligned16(X_k)) return set_error(DFB200_ERR_ARG, "%s: tensors must be 16-byte aligned", op);
	const int half = head_dim / 2;
	if (half > ROPE_MAX_TABLE) return set_error(DFB200_ERR_ARG, "%s: head_dim %d too large", op, head_dim);
	int tok_per_iter = ROPE_THREADS / half;
	if (tok_per_iter < 1) tok_per_iter = 1;
	if (tok_per_iter > 8) tok_per_iter = 8;
	const size_t smem = (((size_t) half + 3) & ~(size_t) 3) * sizeof(float) + 2 * (size_t) tok_per_iter * half * sizeof(float2);
	int grid = 0;
	DFB200_DISPATCH_DTYPE(dt, T, {
		auto kernel = rope_kernel<T, BWD>;
		int per_sm = 0;
		if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, ROPE_THREADS, smem) != cudaSuccess || per_sm < 1) { cudaGetLastError(); per_sm = 1; }
		long long g = (long long) sm_count() * per_sm;
		const long long iters = ((long long) tokens + tok_per_iter - 1) / tok_per_iter;
		if (g > iters) g = iters;
		grid = g < 1 ? 1 : (int) g;
		kernel<<<grid, ROPE_THREADS, smem, (cudaStream_t) stream>>>(tokens, model_dim, kv_dim, head_dim, tok_per_iter, (float) theta, seq_positions, X_q, X_k);
	});
	return check_launch(op);
}

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_rope(int fwd_dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                           const int * seq_positions, void * X_q, void * X_k, void * stream) {
	return launch_rope<false>("rope", fwd_dt, N, model_dim, head_dim, num_kv_heads, theta, seq_positions, X_q, X_k, stream);
}

extern "C" int dfb200_rope_bwd_x(int bwd_dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                                 const int * seq_positions, void * dX_q, void * dX_k, void * stream) {
	return launch_rope<true>("rope_bwd_x", bwd_dt, N, model_dim, head_dim, num_kv_heads, theta, seq_positions, dX_q, dX_k, stream);
}
