// Rotary position embedding, forward and backward, in place on Q [tokens, model_dim] and
// K [tokens, kv_dim] (interleaved pairs; src/ops/nvidia/attention/rope.cu:137-171,
// rope_bwd_x.cu:144-172).
//
// The reference evaluates powf + sinf + cosf once per PAIR (and again for K): 40 times per
// (token, frequency) for 32+8 heads. Here a CTA keeps the head_dim/2 inverse frequencies in
// shared memory for its whole life, builds the (cos, sin) table of TOK tokens per iteration
// (one sincosf per (token, frequency)), and then streams the TOK rows of Q and K through
// registers in 128-bit packets. HBM traffic is one read and one write of Q and K plus the positions.
//
// Two kernels share that scheme:
//   rope_staged_kernel  rows are staged through shared memory by bulk asynchronous copies (TMA
//                       unit): the Q rows of TOK consecutive tokens are one contiguous block, so a
//                       stage is two copies (Q block, K block) into a 4-deep ring; threads rotate
//                       the pairs in place in shared memory and one thread writes the stage back
//                       with a bulk store. Two to three stages (40-60 KB) are in flight per CTA
//                       whatever the register budget, which an in-place register kernel cannot
//                       reach (it cannot hoist a load above the previous store to the same tensor).
//   rope_kernel         the register path, for shapes whose rows are not 16-byte multiples or do
//                       not fit the ring.
#include "common.cuh"
#include "tma.cuh"

namespace dfb200 {

constexpr int E = 8;
#ifndef DFB200_ROPE_THREADS
#define DFB200_ROPE_THREADS 512      /* measured on B200, 8192 tokens x (4096 + 1024): 512 x 1 = 5.7 TB/s, 256 x 4 = 5.1 TB/s */
#define DFB200_ROPE_UNROLL 1
#define DFB200_ROPE_MAX_TOK 8
#endif
constexpr int ROPE_THREADS = DFB200_ROPE_THREADS;
constexpr int ROPE_UNROLL = DFB200_ROPE_UNROLL;
constexpr int ROPE_MAX_TOK = DFB200_ROPE_MAX_TOK;       // tokens whose (cos, sin) table a CTA builds per iteration
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
	cudaTriggerProgrammaticLaunchCompletion();       // see pdl_prologue(): the frequencies below need no global memory,

	// angle_j = theta^(-(2j)/head_dim). The exponent is formed in fp32 as the reference does;
	// the power is taken in fp64 and rounded once, which gives the correctly rounded fp32 powf.
	for (int j = tid; j < half; j += ROPE_THREADS) {
		const float expo = -1.0f * ((float) (2 * j) / (float) head_dim);
		inv_freq[j] = (float) pow((double) theta, (double) expo);
	}
	__syncthreads();
	cudaGridDependencySynchronize();                 // so the wait for the previous kernel of the stream comes after them

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

// ----------------------------------------------------------------------------------------
// staged kernel
// ----------------------------------------------------------------------------------------
// Ring geometry, measured on B200 at 8192 / 16384 tokens x (4096 + 1024) bf16 (10 KB per token, 320 threads per CTA), launches back to
// back, and as the step of the Llama-3-8B layer chain that holds two RoPE launches (bench.py): 3 tokens x 3 stages 25.3 / 56.0 us,
// step 0.407 ms; 2 x 3: 24.0 / 56.5, 0.408; 2 x 4: 26.3 / 56.3, 0.412; 1 x 4: 30.4 / 58.9, 0.413; 3 x 2: 30.5 / 59.9, 0.415;
// 4 x 2: 32.9 / 65.7, 0.422. Geometries that leave one CTA per SM (3 x 4, 4 x 3, 2 x 6, 1 x 8) take 70 - 90 us at 16384 tokens.
#ifndef DFB200_ROPE_STAGES
#define DFB200_ROPE_STAGES 3
#endif
#ifndef DFB200_ROPE_STAGE_BUDGET
#define DFB200_ROPE_STAGE_BUDGET 32768
#endif
constexpr int ROPE_STAGED_THREADS = 512;

template <typename T, bool BWD>
__global__ void __launch_bounds__(ROPE_STAGED_THREADS)
rope_staged_kernel(int tokens, int model_dim, int kv_dim, int head_dim, int tok_per_stage, int stages, float theta,
                   const int * __restrict__ seq_positions, void * X_q, void * X_k, unsigned int * status) {
	constexpr int ESIZE = 4 / Word<T>::EPW;              // bytes per element
	constexpr int CW = E / Word<T>::EPW;                 // 32-bit words per chunk
	extern __shared__ __align__(128) unsigned char smem[];
	const int half = head_dim >> 1;
	const uint32_t q_stage_bytes = (uint32_t) tok_per_stage * model_dim * ESIZE;
	const uint32_t k_stage_bytes = (uint32_t) tok_per_stage * kv_dim * ESIZE;
	const uint32_t stage_bytes = (q_stage_bytes + k_stage_bytes + 127u) & ~127u;
	unsigned char * ring = smem;                                                        // [STAGES][stage_bytes]
	// cos and sin in separate arrays: a thread reads 4 consecutive cos and 4 consecutive sin (two 16-byte loads),
	// and consecutive threads read consecutive 16-byte slots, which is free of bank conflicts
	// Two table buffers: the table of stage it + 1 is built while stage it is rotated, so one CTA barrier per stage serves both
	// "rotated rows ready for the write-back" and "next table ready".
	const int table_len = tok_per_stage * half;
	float * tab_cos = reinterpret_cast<float *>(smem + stages * stage_bytes);      // [2][tok_per_stage * half]
	float * tab_sin = tab_cos + 2 * table_len;                                          // [2][tok_per_stage * half]
	float * inv_freq = tab_sin + 2 * table_len;                                         // [half]
	uint64_t * full = reinterpret_cast<uint64_t *>(inv_freq + ((half + 3) & ~3));       // [STAGES]
	const int tid = threadIdx.x, nthr = blockDim.x;

	cudaTriggerProgrammaticLaunchCompletion();       // see pdl_prologue(): barrier setup and the frequencies need no global memory,
	if (tid == 0) {
		// while the previous kernel of the stream drains: this CTA's first stages on their way to L2
		const int n_blocks0 = (tokens + tok_per_stage - 1) / tok_per_stage;
		for (int it = 0; it < stages - 1; it++) {
			const int blk = (int) blockIdx.x + it * (int) gridDim.x;
			if (blk >= n_blocks0) break;
			const int tok0 = blk * tok_per_stage, n_tok = min(tok_per_stage, tokens - tok0);
			bulk_prefetch_l2(reinterpret_cast<const unsigned char *>(X_q) + (size_t) tok0 * model_dim * ESIZE, (uint32_t) n_tok * model_dim * ESIZE);
			if (kv_dim) bulk_prefetch_l2(reinterpret_cast<const unsigned char *>(X_k) + (size_t) tok0 * kv_dim * ESIZE, (uint32_t) n_tok * kv_dim * ESIZE);
		}
		for (int s = 0; s < stages; s++) mbar_init(&full[s], 1);
		mbar_fence_init();
	}
	for (int j = tid; j < half; j += nthr) {
		const float expo = -1.0f * ((float) (2 * j) / (float) head_dim);
		inv_freq[j] = (float) pow((double) theta, (double) expo);
	}
	__syncthreads();
	cudaGridDependencySynchronize();                 // so the wait for the previous kernel of the stream comes after them

	// this CTA's iterations: token blocks blockIdx.x, + gridDim.x, ...
	const int n_blocks = (tokens + tok_per_stage - 1) / tok_per_stage;
	const int my_iters = blockIdx.x < n_blocks ? (n_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
	auto tok0_of = [&](int it) { return (blockIdx.x + it * (int) gridDim.x) * tok_per_stage; };
	auto issue_load = [&](int it) {          // thread 0 only
		const int s = it % stages, tok0 = tok0_of(it), n_tok = min(tok_per_stage, tokens - tok0);
		const uint32_t qb = (uint32_t) n_tok * model_dim * ESIZE, kb = (uint32_t) n_tok * kv_dim * ESIZE;
		unsigned char * dst = ring + (size_t) s * stage_bytes;
		mbar_arrive_expect_tx(&full[s], qb + kb);
		bulk_load(dst, reinterpret_cast<const unsigned char *>(X_q) + (size_t) tok0 * model_dim * ESIZE, qb, &full[s]);
		if (kb) bulk_load(dst + q_stage_bytes, reinterpret_cast<const unsigned char *>(X_k) + (size_t) tok0 * kv_dim * ESIZE, kb, &full[s]);
	};
	if (tid == 0)
		for (int it = 0; it < stages - 1 && it < my_iters; it++) issue_load(it);
	// (cos, sin) of one stage's tokens into table buffer it & 1
	auto build_table = [&](int it) {
		if (it >= my_iters) return;
		const int tok0 = tok0_of(it), n_tok = min(tok_per_stage, tokens - tok0);
		float * tc = tab_cos + (it & 1) * table_len, * ts = tab_sin + (it & 1) * table_len;
		for (int e = tid; e < n_tok * half; e += nthr) {
			const int t = e / half, j = e - t * half;
			float sn, cs;
			sincosf((float) __ldg(seq_positions + tok0 + t) * inv_freq[j], &sn, &cs);
			tc[e] = cs;
			ts[e] = BWD ? -sn : sn;
		}
	};
	build_table(0);
	__syncthreads();

	const int q_chunks = model_dim / E, k_chunks = kv_dim / E, row_chunks = q_chunks + k_chunks;
	const int chunks_per_head = head_dim / E;
	const int head_mask = (chunks_per_head & (chunks_per_head - 1)) == 0 ? chunks_per_head - 1 : -1;
	bool ok = true;
	for (int it = 0; it < my_iters && ok; it++) {
		const int s = it % stages, tok0 = tok0_of(it), n_tok = min(tok_per_stage, tokens - tok0);
		// every thread waits for the stage's copy itself; a thread whose wait gave up skips the rotation, and the barrier below tells all
		const bool arrived = mbar_wait_bounded(&full[s], (uint32_t) (it / stages) & 1u, status, 0x100u + (unsigned) s);

		// Rotate in place in shared memory. Token-major outer loop, chunk-strided inner loop: a chunk's slot in the (cos, sin) table
		// depends only on its position inside its head, which for Q and K alike is (c mod chunks_per_head) because both sections hold
		// whole heads -- no division in the inner loop when chunks_per_head is a power of two. The launcher sizes the CTA so that a
		// row's chunks divide evenly among the threads (640 chunks: 320 threads x 2), or else most warps would idle through the
		// second pass over every token's chunks.
		unsigned char * stage = ring + (size_t) s * stage_bytes;
		for (int t = 0; t < n_tok && arrived; t++) {
			unsigned char * q_row = stage + (size_t) t * model_dim * ESIZE;
			unsigned char * k_row = stage + q_stage_bytes + (size_t) t * kv_dim * ESIZE - (size_t) q_chunks * E * ESIZE;
			const float * cos_t = tab_cos + (it & 1) * table_len + t * half, * sin_t = tab_sin + (it & 1) * table_len + t * half;
			for (int c = tid; c < row_chunks; c += nthr) {
				uint32_t * p = reinterpret_cast<uint32_t *>((c < q_chunks ? q_row : k_row) + (size_t) c * E * ESIZE);
				const int in_head = head_mask >= 0 ? (c & head_mask) : (c % chunks_per_head);
				uint32_t w[CW];
				if constexpr (CW == 2) { const uint2 v = *reinterpret_cast<const uint2 *>(p); w[0] = v.x; w[1] = v.y; }
				else {
					#pragma unroll
					for (int k = 0; k < CW; k += 4) { const uint4 v = *reinterpret_cast<const uint4 *>(p + k); w[k] = v.x; w[k + 1] = v.y; w[k + 2] = v.z; w[k + 3] = v.w; }
				}
				float x[E], o[E];
				#pragma unroll
				for (int k = 0; k < CW; k++) Word<T>::unpack(w[k], &x[k * Word<T>::EPW]);
				const float4 c4 = *reinterpret_cast<const float4 *>(cos_t + in_head * (E / 2));
				const float4 s4 = *reinterpret_cast<const float4 *>(sin_t + in_head * (E / 2));
				const float cv[4] = {c4.x, c4.y, c4.z, c4.w};
				const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
				#pragma unroll
				for (int q = 0; q < 4; q++) {
					// one product rounded, the other fused into the sum: the contraction nvcc applies to the
					// reference's `c*e - s*o` and `c*o + s*e`
					o[2 * q]     = fmaf(cv[q], x[2 * q],     -__fmul_rn(sv[q], x[2 * q + 1]));
					o[2 * q + 1] = fmaf(cv[q], x[2 * q + 1],  __fmul_rn(sv[q], x[2 * q]));
				}
				#pragma unroll
				for (int k = 0; k < CW; k++) w[k] = Word<T>::pack(&o[k * Word<T>::EPW]);
				if constexpr (CW == 2) *reinterpret_cast<uint2 *>(p) = make_uint2(w[0], w[1]);
				else {
					#pragma unroll
					for (int k = 0; k < CW; k += 4) *reinterpret_cast<uint4 *>(p + k) = make_uint4(w[k], w[k + 1], w[k + 2], w[k + 3]);
				}
			}
		}
		build_table(it + 1);                   // the other buffer: its last readers passed the previous iteration's barrier
		fence_async_smem();                    // rotated values must be visible to the bulk store
		ok = __syncthreads_and(arrived);       // rows rotated, next table visible; everyone agrees on whether to go on
		if (!ok) break;
		if (tid == 0) {
			const uint32_t qb = (uint32_t) n_tok * model_dim * ESIZE, kb = (uint32_t) n_tok * kv_dim * ESIZE;
			bulk_store(reinterpret_cast<unsigned char *>(X_q) + (size_t) tok0 * model_dim * ESIZE, stage, qb);
			if (kb) bulk_store(reinterpret_cast<unsigned char *>(X_k) + (size_t) tok0 * kv_dim * ESIZE, stage + q_stage_bytes, kb);
			bulk_commit();
			const int next = it + stages - 1;            // refills the stage written back in the previous iteration
			if (next < my_iters) {
				bulk_wait_read<1>();                     // ... once that write-back no longer reads it
				issue_load(next);
			}
		}
	}
	if (tid == 0) bulk_wait_all<0>();          // shared memory must outlive the write-backs
}

// General shapes: any even head_dim, tensors aligned to their element size only (the reference rotates one pair per thread with no
// other demand, src/ops/nvidia/attention/rope.cu:137-171). One pair per thread; frequency, angle and rotation exactly as in the
// kernels above (fp64 power rounded once, fp32 angle, sincosf, separately rounded products), recomputed per pair.
constexpr int ROPE_GENERAL_THREADS = 256;

template <typename T, bool BWD>
__global__ void __launch_bounds__(ROPE_GENERAL_THREADS)
rope_general_kernel(int tokens, int model_dim, int kv_dim, int head_dim, float theta, const int * __restrict__ seq_positions, void * X_q, void * X_k) {
	pdl_prologue();
	const uint64_t pairs_per_token = (uint64_t) (model_dim + kv_dim) / 2, n_pairs = (uint64_t) tokens * pairs_per_token;
	for (uint64_t p = (uint64_t) blockIdx.x * ROPE_GENERAL_THREADS + threadIdx.x; p < n_pairs; p += (uint64_t) gridDim.x * ROPE_GENERAL_THREADS) {
		const int t = (int) (p / pairs_per_token);
		int e = 2 * (int) (p - (uint64_t) t * pairs_per_token);               // even element index within the token's Q | K row
		const bool is_q = e < model_dim;
		if (!is_q) e -= model_dim;
		void * base = is_q ? X_q : X_k;
		const uint64_t idx = (uint64_t) t * (is_q ? model_dim : kv_dim) + e;
		const int j = (e % head_dim) >> 1;
		const float expo = -1.0f * ((float) (2 * j) / (float) head_dim);
		const float ang = (float) __ldg(seq_positions + t) * (float) pow((double) theta, (double) expo);
		float sn, cs;
		sincosf(ang, &sn, &cs);
		if (BWD) sn = -sn;
		const float x0 = load_one<T>(base, idx), x1 = load_one<T>(base, idx + 1);
		store_one<T>(base, idx, __fsub_rn(__fmul_rn(cs, x0), __fmul_rn(sn, x1)));
		store_one<T>(base, idx + 1, __fadd_rn(__fmul_rn(cs, x1), __fmul_rn(sn, x0)));
	}
}

template <bool BWD>
static int launch_rope(const char * op, int dt, uint64_t N, int model_dim, int head_dim, int num_kv_heads, int theta,
                       const int * seq_positions, void * X_q, void * X_k, void * stream) {
	if (BWD ? !(dt == DATAFLOW_FP32 || dt == DATAFLOW_FP16 || dt == DATAFLOW_BF16) : !dtype_size(dt))
		return set_error(DFB200_ERR_DTYPE, "%s: unsupported datatype %d", op, dt);
	if (model_dim <= 0 || head_dim <= 0 || num_kv_heads < 0 || theta <= 0)
		return set_error(DFB200_ERR_ARG, "%s: bad dimensions (model_dim %d, head_dim %d, num_kv_heads %d, theta %d)", op, model_dim, head_dim, num_kv_heads, theta);
	if (head_dim % 2 || model_dim % head_dim)
		return set_error(DFB200_ERR_ARG, "%s: head_dim (%d) must be even and divide model_dim (%d)", op, head_dim, model_dim);
	if (N % (uint64_t) model_dim) return set_error(DFB200_ERR_ARG, "%s: N is not a multiple of model_dim", op);
	const uint64_t tokens64 = N / (uint64_t) model_dim;
	if (tokens64 > 0x7fffffffull) return set_error(DFB200_ERR_ARG, "%s: too many tokens", op);
	const int tokens = (int) tokens64;
	if (tokens == 0) return DFB200_OK;
	const int kv_dim = num_kv_heads * head_dim;
	if (!seq_positions || !X_q || (kv_dim && !X_k)) return set_error(DFB200_ERR_ARG, "%s: NULL tensor argument", op);
	const uintptr_t esz = (uintptr_t) dtype_size(dt);
	if (reinterpret_cast<uintptr_t>(X_q) % esz || reinterpret_cast<uintptr_t>(X_k) % esz || (reinterpret_cast<uintptr_t>(seq_positions) & 3u))
		return set_error(DFB200_ERR_ARG, "%s: tensors must be aligned to their element size", op);
	const int half = head_dim / 2;
	if (head_dim % E || !aligned16(X_q) || !aligned16(X_k) || half > ROPE_MAX_TABLE) {
		const uint64_t n_pairs = (uint64_t) tokens * (uint64_t) (model_dim + kv_dim) / 2;
		const uint64_t blocks = (n_pairs + ROPE_GENERAL_THREADS - 1) / ROPE_GENERAL_THREADS, cap = (uint64_t) (sm_count() > 0 ? sm_count() : 1) * 32;
		DFB200_DISPATCH_DTYPE(dt, T,
			(launch_pdl(rope_general_kernel<T, BWD>, dim3((unsigned) (blocks < cap ? blocks : cap)), dim3(ROPE_GENERAL_THREADS), 0, (cudaStream_t) stream, tokens,
			            model_dim, kv_dim, head_dim, (float) theta, seq_positions, X_q, X_k)));
		return check_launch(op);
	}

	// staged path: rows must be 16-byte multiples (bulk copies) and four stages of at least one token must fit
	{
		const size_t esize = (size_t) dtype_size(dt);
		const size_t row_bytes = ((size_t) model_dim + kv_dim) * esize;
		const bool copyable = (model_dim * esize) % 16 == 0 && (kv_dim * esize) % 16 == 0;
		int tok = (int) (DFB200_ROPE_STAGE_BUDGET / row_bytes);
		int stages = DFB200_ROPE_STAGES;
		// threads per CTA: the fewest passes over a row's chunks that 512 threads allow, then as few threads as do it in that many
		// passes (a multiple of 32), so that every thread has the same number of chunks per token
		const int row_chunks = (model_dim + kv_dim) / E, passes = (row_chunks + ROPE_STAGED_THREADS - 1) / ROPE_STAGED_THREADS;
		int sthreads = ((row_chunks + passes - 1) / passes + 31) / 32 * 32;
		if (sthreads < 64) sthreads = 64;
		if (tok > 8) tok = 8;
		if (tok > tokens) tok = tokens;
		unsigned int * status = kernel_status_word(STATUS_ROPE);
		if (copyable && tok >= 1 && status) {
			const size_t stage_bytes = ((size_t) tok * row_bytes + 127) & ~(size_t) 127;
			const size_t smem = stages * stage_bytes + 2 * (size_t) tok * half * sizeof(float2) + (((size_t) half + 3) & ~(size_t) 3) * sizeof(float)
			                    + stages * sizeof(uint64_t);
			int rc = DFB200_ERR_DTYPE;
			DFB200_DISPATCH_DTYPE(dt, T, {
				auto kernel = rope_staged_kernel<T, BWD>;
				allow_dyn_smem(reinterpret_cast<const void *>(kernel), smem);
				const int per_sm = ctas_per_sm(reinterpret_cast<const void *>(kernel), sthreads, smem);
				long long g = (long long) sm_count() * per_sm;
				const long long blocks = ((long long) tokens + tok - 1) / tok;
				if (g > blocks) g = blocks;
				launch_pdl(kernel, dim3((unsigned) (g < 1 ? 1 : g)), dim3(sthreads), smem, (cudaStream_t) stream, tokens, model_dim, kv_dim, head_dim, tok,
				           stages, (float) theta, seq_positions, X_q, X_k, status);
				rc = check_launch(op);
			});
			return rc;
		}
	}

	int tok_per_iter = ROPE_THREADS / half;
	if (tok_per_iter < 1) tok_per_iter = 1;
	if (tok_per_iter > ROPE_MAX_TOK) tok_per_iter = ROPE_MAX_TOK;
	const size_t smem = (((size_t) half + 3) & ~(size_t) 3) * sizeof(float) + 2 * (size_t) tok_per_iter * half * sizeof(float2);
	int grid = 0;
	DFB200_DISPATCH_DTYPE(dt, T, {
		auto kernel = rope_kernel<T, BWD>;
		const int per_sm = ctas_per_sm(reinterpret_cast<const void *>(kernel), ROPE_THREADS, smem);
		long long g = (long long) sm_count() * per_sm;
		const long long iters = ((long long) tokens + tok_per_iter - 1) / tok_per_iter;
		if (g > iters) g = iters;
		grid = g < 1 ? 1 : (int) g;
		launch_pdl(kernel, dim3(grid), dim3(ROPE_THREADS), smem, (cudaStream_t) stream, tokens, model_dim, kv_dim, head_dim, tok_per_iter, (float) theta,
		           seq_positions, X_q, X_k);
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
