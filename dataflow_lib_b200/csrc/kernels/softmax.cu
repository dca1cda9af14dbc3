// Row softmax, the cross-entropy gradient step, and the two fused into one pass.
//
// A row lives ON CHIP: a thread-block cluster of 1, 2, 4 or 8 CTAs owns one row, every
// thread requests its packets up front (up to 8 into registers; for long rows of 16- and 32-bit
// elements half of them into shared-memory slots of its own), and the three phases of the
// reference kernel (max, sum of exponentials, normalise; src/ops/nvidia/loss/softmax.cu:311-405)
// run on that copy. The row is read from HBM once and written once; the reference
// reads it three times. The CTAs of a cluster exchange their maxima and partial sums by
// pushing them into each other's shared memory (asynchronous stores counted on a barrier in
// the receiver's shared memory; every wait is bounded).
//
// Rounding points kept from the reference (W = the output/"backward" datatype, which is also
// the type the reference holds its shared-memory scratch in):
//   * max is taken over W values (exact), x - max is rounded to W before the exponential,
//   * the row is split into 32 interleaved partial sums: element j belongs to partial
//     (j / 32) % 32 -- the reference's 32 warps striding over 32-element groups -- each
//     accumulated in fp32 and rounded to W; the 32 rounded values are added in fp32 in the
//     shuffle-tree order and the total is rounded to W again,
//   * out = W( exp(W(x - max)) / total ).
// Within a partial sum the fp32 addition order differs from the reference's (it cannot be
// reproduced by a different thread layout); that changes a partial by a few fp32 ulps before
// its rounding to W.
//
// Measured history at 16384 x 128256 bf16. A persistent variant that staged row slices through shared memory with bulk
// asynchronous copies (3-deep ring, one 1024-thread CTA per SM): 3.4 ms. Register-only CTAs in clusters of four with cluster
// barriers: 1.9 ms -- per row the chain max -> exchange -> sums -> exchange -> normalise is latency however the data arrives, so
// what matters is how many independent rows an SM has in flight and how cheap the exchange is. The current form (two resident
// CTAs per SM, half of each thread's packets in shared memory, pushed exchange): 1.5 ms.
//
// Keeping the exponentials of phase 2 in registers for phase 3 (possible at <= 4 packets per thread, which for long rows
// means a cluster twice as large) was measured too and was slower everywhere: 32768 columns 5.8 -> 3.6 TB/s, 65536 columns
// 4.6 -> 3.3 TB/s, 128256 columns 4.3 -> 3.0 TB/s. Evaluating exp twice is cheaper than the larger clusters and the store
// bursts of a compute-free phase 3. CTAs of 1024 threads (a cluster half as large) were slower as well (128256 columns: 3.5 TB/s).
#include "common.cuh"
#include "tma.cuh"

#include <cooperative_groups.h>
#include <math_constants.h>

namespace cg = cooperative_groups;

namespace dfb200 {

constexpr int E = 8;                       // elements per chunk
constexpr int SLICE_ALIGN_CHUNKS = 128;    // slices start on a multiple of 1024 elements so that a thread's partial index is fixed
constexpr int SOFTMAX_MAX_CLUSTER = 8;
#ifndef DFB200_SOFTMAX_MAX_THREADS
#define DFB200_SOFTMAX_MAX_THREADS 512
#endif
constexpr int SOFTMAX_MAX_THREADS = DFB200_SOFTMAX_MAX_THREADS;
#ifndef DFB200_SOFTMAX_MAX_CPT
#define DFB200_SOFTMAX_MAX_CPT 8
#endif
constexpr int SOFTMAX_MAX_CPT = DFB200_SOFTMAX_MAX_CPT;

// ---- exchange between the CTAs of a cluster: every CTA PUSHES its value into the shared memory of each peer with an asynchronous
// store that counts its bytes on a barrier in the peer's shared memory, and waits (bounded) on its own barrier. Against
// barrier.cluster + remote loads this takes the memory fence of the cluster barrier's release and one round trip out of each of the
// two exchanges of a row.
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ uint32_t peer_smem_addr(const void * p, unsigned cta_rank) {
	uint32_t r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(cta_rank));
	return r;
}
__device__ __forceinline__ void push_f32(uint32_t peer_dst, float v, uint32_t peer_bar) {
	asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
	             :: "r"(peer_dst), "r"(__float_as_uint(v)), "r"(peer_bar) : "memory");
}
// Waits for phase 0 of `bar` (its expected bytes have arrived from the peers). Gives up after WAIT_LIMIT_NS and records `where`
// in the family's status word. Once any wait of THIS launch has given up, the launch's other waits give up at their next look at the
// abort word, so a broken exchange costs the launch one time limit and not one per row. The abort word (STATUS_SLOTS words after the
// status word) holds the number of the launch that gave up, not a flag: a value left by an earlier launch never shortens a later one.
// A caller that gets `false` must poison what it computes from the exchange (NaN), so that the failure shows in the data too.
__device__ __forceinline__ bool wait_pushed(uint64_t * bar, unsigned int * status, unsigned int where, unsigned int epoch) {
	auto done = [&]() {
		uint32_t ok;
		asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
		             : "=r"(ok) : "r"(smem_u32(bar)) : "memory");
		return ok != 0;
	};
	if (done()) return true;
	const unsigned long long t0 = global_timer_ns();
	for (;;) {
		for (int i = 0; i < 1024; i++)
			if (done()) return true;
		if (global_timer_ns() - t0 > WAIT_LIMIT_NS) break;
		if (status && *reinterpret_cast<volatile unsigned int *>(status + STATUS_SLOTS) == epoch) break;
	}
	if (status) { atomicMax(status, where); atomicExch(status + STATUS_SLOTS, epoch); }
	return false;
}

// Per-chunk arithmetic. The softmax is instruction-bound before it is memory-bound (two exponentials per element
// plus the rounding of x - max to the working type): at 6.5 TB/s an SM has about 22 issue slots per element, and
// the conversion/transcendental pipe only 4 per element. The same-type 16-bit cases therefore work on PACKED pairs:
// the maximum with max.bf16x2 / max.f16x2 and x - max with sub.bf16x2 / sub.f16x2 -- which is also literally the
// reference's operation (one rounding of the exact difference, src/ops/nvidia/loss/softmax.cu:359) -- so that no
// float->bf16 conversion is left in the inner loops. Other type pairs take the generic fp32 path.
template <typename F, typename B> struct RowMath {
	static constexpr int FW = E / Word<F>::EPW;
	struct Max { float m; };
	static __device__ __forceinline__ Max max_init() { return Max{-CUDART_INF_F}; }
	static __device__ __forceinline__ void max_chunk(Max & acc, const uint32_t (&raw)[FW]) {
		float x[E];
		#pragma unroll
		for (int i = 0; i < FW; i++) Word<F>::unpack(raw[i], &x[i * Word<F>::EPW]);
		#pragma unroll
		for (int i = 0; i < E; i++) acc.m = fmaxf(acc.m, x[i]);
	}
	static __device__ __forceinline__ float max_value(const Max & acc) { return acc.m; }
	struct Shift { float m; };
	static __device__ __forceinline__ Shift shift_of(float row_max) { return Shift{row_max}; }
	// d[i] = W(x[i] - max) as fp32
	static __device__ __forceinline__ void shifted(const Shift & sh, const uint32_t (&raw)[FW], float (&d)[E]) {
		float x[E];
		#pragma unroll
		for (int i = 0; i < FW; i++) Word<F>::unpack(raw[i], &x[i * Word<F>::EPW]);
		#pragma unroll
		for (int i = 0; i < E; i++) d[i] = round_to<B>(x[i] - sh.m);
	}
};

template <> struct RowMath<bf16_t, bf16_t> {
	static constexpr int FW = 4;
	struct Max { __nv_bfloat162 m; };
	static __device__ __forceinline__ Max max_init() { Max a; a.m = __float2bfloat162_rn(-CUDART_INF_F); return a; }
	static __device__ __forceinline__ void max_chunk(Max & acc, const uint32_t (&raw)[FW]) {
		#pragma unroll
		for (int i = 0; i < FW; i++) acc.m = __hmax2(acc.m, *reinterpret_cast<const __nv_bfloat162 *>(&raw[i]));
	}
	static __device__ __forceinline__ float max_value(const Max & acc) { return fmaxf(__low2float(acc.m), __high2float(acc.m)); }
	struct Shift { __nv_bfloat162 m; };
	static __device__ __forceinline__ Shift shift_of(float row_max) { Shift s; s.m = __float2bfloat162_rn(row_max); return s; }   // exact: the max is a bf16 value
	static __device__ __forceinline__ void shifted(const Shift & sh, const uint32_t (&raw)[FW], float (&d)[E]) {
		#pragma unroll
		for (int i = 0; i < FW; i++) {
			const __nv_bfloat162 v = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[i]), sh.m);
			Word<bf16_t>::unpack(*reinterpret_cast<const uint32_t *>(&v), &d[2 * i]);
		}
	}
};

template <> struct RowMath<f16_t, f16_t> {
	static constexpr int FW = 4;
	struct Max { __half2 m; };
	static __device__ __forceinline__ Max max_init() { Max a; a.m = __float2half2_rn(-CUDART_INF_F); return a; }
	static __device__ __forceinline__ void max_chunk(Max & acc, const uint32_t (&raw)[FW]) {
		#pragma unroll
		for (int i = 0; i < FW; i++) acc.m = __hmax2(acc.m, *reinterpret_cast<const __half2 *>(&raw[i]));
	}
	static __device__ __forceinline__ float max_value(const Max & acc) { return fmaxf(__low2float(acc.m), __high2float(acc.m)); }
	struct Shift { __half2 m; };
	static __device__ __forceinline__ Shift shift_of(float row_max) { Shift s; s.m = __float2half2_rn(row_max); return s; }
	static __device__ __forceinline__ void shifted(const Shift & sh, const uint32_t (&raw)[FW], float (&d)[E]) {
		#pragma unroll
		for (int i = 0; i < FW; i++) {
			const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&raw[i]), sh.m);
			Word<f16_t>::unpack(*reinterpret_cast<const uint32_t *>(&v), &d[2 * i]);
		}
	}
};

// OUT = the type the probabilities are stored in: B for the registered ops; f32_t (with B = F) for the reference's
// softmax_<f16|bf16>_fp32 kernels (src/ops/nvidia/loss/softmax.cu:965-1249), which keep their scratch in the input type and
// store exp(..) / total unrounded. ARGMAX additionally writes the smallest index holding the row maximum to arg_maxs[row]
// (the reference lets whichever thread sees the maximum last win, :1057-1059).
// SPT > 0 (16- and 32-bit inputs): a thread owns SPT more packets of the row in SHARED memory (slots [k][quarter][tid], fetched with
// per-thread asynchronous 16-byte copies and read back only by the thread that requested them, so no barrier guards them).
// A 512-thread CTA then covers (CPT + SPT) x 512 packets (8 + 8 of 16 bytes, or 4 + 4 of 32 bytes for fp32) with 64 KB of shared memory and 64 registers per thread, so two
// CTAs stay resident per SM and one computes exponentials while the other waits for memory. Rows of up to 65536 elements take one
// such CTA, rows of up to 131072 elements a cluster of two, up to 262144 a cluster of four. Measured at 16384 x 128256 bf16: cluster of 4 register-only CTAs
// 1.93 ms; one 1024-thread CTA with 128 KB of shared memory (no cluster, but one CTA per SM) 1.76 ms; the cluster of two 1.64 ms with
// cluster barriers and remote reads, 1.50 ms with the pushed exchange above.
// Resident CTAs per SM the compiler is asked to make room for, by the registers the row copy takes (32-bit words per thread): up to
// 16 words leave room for four 512-thread CTAs (32 registers per thread), up to 32 words for two (64 registers); beyond that
// (fp32 rows at 8 packets per thread) the compiler is left alone.
constexpr int softmax_min_ctas(int row_words_per_thread, int spt) { return spt > 0 ? 2 : row_words_per_thread <= 16 ? 4 : row_words_per_thread <= 32 ? 2 : 0; }

template <typename F, typename B, int CPT, bool FUSE_CE, typename OUT = B, bool ARGMAX = false, int SPT = 0, bool MULTI = false>
__global__ void __launch_bounds__(SOFTMAX_MAX_THREADS, softmax_min_ctas(CPT * (E / Word<F>::EPW), SPT))
softmax_rows_kernel(int n_rows, int n_cols, int slice_chunks, const void * __restrict__ X, void * __restrict__ out,
                    const uint32_t * __restrict__ labels, float * __restrict__ row_loss, uint32_t * __restrict__ arg_maxs, unsigned int * status,
                    unsigned int epoch) {
	static_assert(!FUSE_CE || sizeof(OUT) == sizeof(B), "the fused cross-entropy step works in the output type");
	constexpr int FW = E / Word<F>::EPW;
	static_assert(SPT == 0 || FW % 4 == 0, "shared-memory packets are made of 16-byte quarters");
	constexpr int QW = FW / 4;                             // 16-byte quarters per packet: 1 for 16-bit elements, 2 for fp32
	constexpr int NPK = CPT + SPT;                         // packets per thread: the first CPT in registers, the rest in shared memory
	extern __shared__ uint4 s_pack[];                      // [SPT][QW][blockDim.x]
	__shared__ float s_warp_max[32];
	__shared__ float s_warp_part[SOFTMAX_MAX_THREADS / 32][8];
	__shared__ float s_peer_max[SOFTMAX_MAX_CLUSTER];      // [r] pushed here by CTA r of the cluster
	__shared__ float s_peer_part[SOFTMAX_MAX_CLUSTER][32];
	__shared__ uint64_t s_pushed[2];                       // byte-counting barriers of the two exchanges
	__shared__ float s_row[3];              // row max, row total (rounded to W), row total in fp32 (fused cross entropy: the loss)
	__shared__ uint32_t s_label[3];         // label, owning thread, packet index (fused cross entropy)

	// MULTI = the row is shared by a cluster of more than one CTA (only rows that need 8 packets per thread are); without it the
	// cluster code compiles away.
	unsigned csize = 1, crank = 0;
	if constexpr (MULTI) { csize = cg::this_cluster().num_blocks(); crank = cg::this_cluster().block_rank(); }
	const int row = blockIdx.x / csize;
	const int tid = threadIdx.x, nthr = blockDim.x;
	const int warp = tid >> 5, lane = tid & 31, n_warps = nthr >> 5;

	const int n_chunks = n_cols / E;
	const int c_begin = crank * slice_chunks;
	const int c_end = min(n_chunks, c_begin + slice_chunks);
	const uint64_t row_elem = (uint64_t) row * (uint64_t) n_cols;

	if constexpr (ARGMAX) {
		// ordered before every atomicMin below: by the release / acquire of the cluster barrier for the peers, by __syncthreads here
		if (crank == 0 && tid == 0) arg_maxs[row] = 0xffffffffu;
	}
	// ---- cluster set-up, before any load is in flight so that the release of the arrive has nothing to wait for: the two barriers
	// expect the peers' bytes (4 per peer for the maximum, 128 per peer for the partial sums); peers push only after their wait.
	if constexpr (MULTI) {
		if (tid == 0) {
			mbar_init(&s_pushed[0], 1);
			mbar_init(&s_pushed[1], 1);
			mbar_fence_init();
			mbar_arrive_expect_tx(&s_pushed[0], (csize - 1) * 4u);
			mbar_arrive_expect_tx(&s_pushed[1], (csize - 1) * 128u);
		}
		__syncwarp();
		// fence.mbarrier_init has published the barriers; only the arg-max form has a store (above) that the arrive must release
		if constexpr (ARGMAX) cluster_arrive_release(); else cluster_arrive_relaxed();
	}

	// ---- load: every packet of the slice is requested before anything is consumed
	uint32_t raw[CPT][FW];
	#pragma unroll
	for (int k = 0; k < CPT; k++) {
		const int c = c_begin + tid + k * nthr;
		if (c < c_end) ld_words<FW, Hint::STREAM>(reinterpret_cast<const char *>(X) + (row_elem + (uint64_t) c * E) * (4 / Word<F>::EPW), raw[k]);
	}
	if constexpr (SPT > 0) {
		#pragma unroll
		for (int k = 0; k < SPT; k++) {
			const int c = c_begin + tid + (CPT + k) * nthr;
			if (c < c_end) {
				const char * src = reinterpret_cast<const char *>(X) + (row_elem + (uint64_t) c * E) * (4 / Word<F>::EPW);
				#pragma unroll
				for (int q = 0; q < QW; q++) {
					const uint32_t dst = (uint32_t) __cvta_generic_to_shared(&s_pack[(k * QW + q) * nthr + tid]);
					asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src + 16 * q) : "memory");
				}
			}
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	}
	if constexpr (FUSE_CE) {
		// Requested after the packets. Thread 0 also works out which thread of the cluster holds the label's packet and as which of
		// its packets, so that the other threads pay one shared-memory read and a compare for the cross-entropy step.
		if (tid == 0) {
			const uint32_t label = labels ? __ldg(labels + row) : 0xffffffffu;      // no labels: no row has one (the plain softmax through this form)
			const int rel = (int) (label / E) - c_begin;
			const bool mine = label < (uint32_t) n_cols && rel >= 0 && (int) (label / E) < c_end;
			s_label[0] = label;
			s_label[1] = mine ? (uint32_t) (rel % nthr) : 0xffffffffu;   // owning thread of this CTA, if any
			s_label[2] = mine ? (uint32_t) (rel / nthr) : 0u;            // index of the packet in that thread
		}
	}
	auto shared_packet = [&](int ks, uint32_t (&w)[FW]) {   // shared-memory packet ks of this thread
		if constexpr (SPT > 0) {
			#pragma unroll
			for (int q = 0; q < QW; q++) {
				const uint4 v = s_pack[(ks * QW + q) * nthr + tid];
				w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
			}
		}
	};
	// packet k of this thread: registers for k < CPT, its own shared-memory slot otherwise (k is a compile-time constant after unrolling)
	auto packet = [&](int k, uint32_t (&w)[FW]) {
		if (k < CPT) {
			#pragma unroll
			for (int i = 0; i < FW; i++) w[i] = raw[k < CPT ? k : 0][i];
		} else if constexpr (SPT > 0) {
			shared_packet(k - CPT, w);
		}
	};

	// ---- phase 1: row maximum
	using Math = RowMath<F, B>;
	typename Math::Max macc = Math::max_init();
	#pragma unroll
	for (int k = 0; k < CPT; k++) {
		const int c = c_begin + tid + k * nthr;
		if (c < c_end) Math::max_chunk(macc, raw[k]);
	}
	if constexpr (SPT > 0) {
		asm volatile("cp.async.wait_group 0;" ::: "memory");       // this thread's own copies have landed
		#pragma unroll
		for (int k = CPT; k < NPK; k++) {
			const int c = c_begin + tid + k * nthr;
			if (c < c_end) { uint32_t w[FW]; packet(k, w); Math::max_chunk(macc, w); }
		}
	}
	float m = warp_max(Math::max_value(macc));
	if (lane == 0) s_warp_max[warp] = m;
	if constexpr (MULTI) cluster_wait_acquire();  // every CTA of the cluster runs and has its barriers set up (long since: the loads came between)
	__syncthreads();
	if (warp == 0) {
		float v = lane < n_warps ? s_warp_max[lane] : -CUDART_INF_F;
		v = warp_max(v);
		if constexpr (MULTI) {
			if ((unsigned) lane == crank) s_peer_max[crank] = v;
			else if ((unsigned) lane < csize) push_f32(peer_smem_addr(&s_peer_max[crank], lane), v, peer_smem_addr(&s_pushed[0], lane));
			const bool arrived = wait_pushed(&s_pushed[0], status, 0x50000001u, epoch);
			__syncwarp();
			v = (unsigned) lane < csize ? s_peer_max[lane] : -CUDART_INF_F;
			v = warp_max(v);
			if (!__all_sync(0xffffffffu, arrived)) v = CUDART_NAN_F;   // a peer's maximum never came: the row's outputs become NaN
		}
		if (lane == 0) s_row[0] = v;
	}
	__syncthreads();
	const float row_max = s_row[0];
	const typename Math::Shift shift = Math::shift_of(row_max);
	// ---- the fused cross-entropy step needs W(x[label] - max) after the last phase: the one thread of the row whose packet holds the
	// label takes it aside now (one register through the hot loops; the label itself waits in shared memory), so that the row copy can
	// be given up packet by packet in phase 3.
	constexpr float NO_LABEL = 1.0f;                       // shifted logits are <= 0 (or NaN)
	float label_logit = NO_LABEL;                          // W(x[label] - max): what the stored probability is made from
	float label_diff = 0.0f;                               // x[label] - max in fp32, not rounded to W: what the loss is made from
	if constexpr (FUSE_CE) {
		if ((uint32_t) tid == s_label[1]) {               // written by thread 0 before the barriers of phase 1
			const int kl = (int) s_label[2], j = (int) (s_label[0] % E);
			uint32_t w[FW];
			if (kl >= CPT) {
				shared_packet(kl - CPT, w);
			} else {
				#pragma unroll
				for (int k = 0; k < CPT; k++) {
					if (k == kl) {
						#pragma unroll
						for (int i = 0; i < FW; i++) w[i] = raw[k][i];
					}
				}
			}
			float d[E], x[E];
			Math::shifted(shift, w, d);
			#pragma unroll
			for (int i = 0; i < FW; i++) Word<F>::unpack(w[i], &x[i * Word<F>::EPW]);
			#pragma unroll
			for (int i = 0; i < E; i++) if (i == j) { label_logit = d[i]; label_diff = x[i] - row_max; }
		}
	}
	if constexpr (ARGMAX) {
		uint32_t first = 0xffffffffu;
		#pragma unroll
		for (int k = NPK - 1; k >= 0; k--) {
			const int c = c_begin + tid + k * nthr;
			if (c < c_end) {
				float x[E];
				uint32_t w[FW];
				packet(k, w);
				#pragma unroll
				for (int i = 0; i < FW; i++) Word<F>::unpack(w[i], &x[i * Word<F>::EPW]);
				#pragma unroll
				for (int i = E - 1; i >= 0; i--) if (x[i] == row_max) first = (uint32_t) (c * E + i);
			}
		}
		if (first != 0xffffffffu) atomicMin(arg_maxs + row, first);
	}

	// ---- phase 2: 32 interleaved partial sums of exp(W(x - max))
	float part4[4] = {0.0f, 0.0f, 0.0f, 0.0f};            // four independent chains: the adds are not the critical path
	#pragma unroll
	for (int k = 0; k < NPK; k++) {
		const int c = c_begin + tid + k * nthr;
		if (c < c_end) {
			float d[E];
			uint32_t w[FW];
			packet(k, w);
			Math::shifted(shift, w, d);
			#pragma unroll
			for (int i = 0; i < E; i++) part4[i & 3] += fast_exp(d[i]);
		}
	}
	float part = (part4[0] + part4[1]) + (part4[2] + part4[3]);
	// chunk c covers elements 8c..8c+7, so its partial index is (c / 4) % 32; c = tid + k*nthr with
	// nthr % 128 == 0 and c_begin % 128 == 0 makes that (tid / 4) % 32 for every k.
	part += __shfl_xor_sync(0xffffffffu, part, 1);
	part += __shfl_xor_sync(0xffffffffu, part, 2);
	if ((lane & 3) == 0) s_warp_part[warp][lane >> 2] = part;
	__syncthreads();
	if (warp == 0) {
		// partial `lane` was produced by warps w with w % 4 == lane / 8 (8 partials per warp)
		float v = 0.0f;
		for (int w = lane >> 3; w < n_warps; w += 4) v += s_warp_part[w][lane & 7];
		if constexpr (MULTI) {
			s_peer_part[crank][lane] = v;
			for (unsigned r = 0; r < csize; r++)
				if (r != crank) push_f32(peer_smem_addr(&s_peer_part[crank][lane], r), v, peer_smem_addr(&s_pushed[1], r));
			const bool arrived = wait_pushed(&s_pushed[1], status, 0x50000002u, epoch);
			v = 0.0f;
			for (unsigned r = 0; r < csize; r++) v += s_peer_part[r][lane];   // the same order in every CTA of the cluster
			if (!arrived) v = CUDART_NAN_F;                                    // a peer's sums never came: the row's outputs become NaN
		}
		// The loss is not one of the reference's outputs and keeps none of its roundings: its row total is the fp32 sum of the 32
		// partial sums BEFORE they are rounded to W.
		float total32 = 0.0f;
		if constexpr (FUSE_CE) total32 = warp_sum(v);
		v = round_to<B>(v);
		v = warp_sum(v);
		if (lane == 0) { s_row[1] = round_to<B>(v); if constexpr (FUSE_CE) s_row[2] = total32; }
	}
	// A CTA has received everything its peers will ever write into its shared memory once both waits have returned, so it may leave
	// without a closing barrier; the arrive / wait pair below only covers a wait that gave up (the status word then says so).
	if constexpr (MULTI) cluster_arrive_relaxed();
	__syncthreads();
	const float total = s_row[1];

	// ---- phase 3: normalise and store. exp(d) / total is the approximate division of the reference build, i.e. a
	// multiplication by rcp.approx(total); the reciprocal is taken once per thread.
	const float inv_total = fast_rcp(total);
	#pragma unroll
	for (int k = 0; k < NPK; k++) {
		const int c = c_begin + tid + k * nthr;
		if (c < c_end) {
			float d[E], o[E];
			uint32_t w[FW];
			packet(k, w);
			Math::shifted(shift, w, d);
			#pragma unroll
			for (int i = 0; i < E; i++) o[i] = fast_exp(d[i]) * inv_total;
			store_elems<OUT, E>(out, row_elem + (uint64_t) c * E, o);
		}
	}
	// ---- cross-entropy step, by the one thread of the row that holds the label: the probability is recomputed from the logit taken
	// aside above (nothing is read back from memory), rounded to the working type, one is subtracted and the difference rounded again
	// -- what the separate kernel does to the stored value -- and stored over it. The row's loss is log(sum_j exp(W(x_j - max))) -
	// (x_label - max) with the sum and the difference in fp32: the only rounding to W left in it is the one inside the exponentials,
	// which moves the mean loss of N(0, 2) logits over 128256 columns by 5e-6 of its value against an fp64 cross entropy.
	if constexpr (FUSE_CE) {
		if (label_logit != NO_LABEL) {
			store_one<OUT>(out, row_elem + s_label[0], round_to<B>(fast_exp(label_logit) * inv_total) - 1.0f);
			if (row_loss) row_loss[row] = logf(s_row[2]) - label_diff;
		} else if (row_loss && crank == 0 && tid == 0 && s_label[0] >= (uint32_t) n_cols) {
			row_loss[row] = 0.0f;
		}
	}
	if constexpr (MULTI) cluster_wait_acquire();
}

// General shapes: any n_cols, tensors aligned to their element size only, rows of any length. The reference's structure itself
// (src/ops/nvidia/loss/softmax.cu:273-407): one 1024-thread block per row, three passes over the row in global memory; warp w takes the
// 32-element groups w, w + 32, ... (so thread t holds elements t, t + 1024, ...), its sum is rounded to the working type, the 32
// rounded sums are added in the shuffle-tree order and the total rounded again. A ragged last group contributes what it has.
template <typename F, typename B>
__global__ void __launch_bounds__(1024)
softmax_general_kernel(int n_rows, int n_cols, const void * __restrict__ X, void * __restrict__ out) {
	__shared__ float s_warp[32];
	__shared__ float s_row[2];
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
		const uint64_t base = (uint64_t) row * (uint64_t) n_cols;
		float m = -CUDART_INF_F;
		for (int i = tid; i < n_cols; i += 1024) m = fmaxf(m, load_one<F>(X, base + i));
		m = warp_max(m);
		if (lane == 0) s_warp[warp] = m;
		__syncthreads();
		if (warp == 0) { const float v = warp_max(s_warp[lane]); if (lane == 0) s_row[0] = v; }
		__syncthreads();
		const float row_max = s_row[0];
		float part = 0.0f;
		for (int i = tid; i < n_cols; i += 1024) part += fast_exp(round_to<B>(load_one<F>(X, base + i) - row_max));
		part = warp_sum(part);
		if (lane == 0) s_warp[warp] = round_to<B>(part);
		__syncthreads();
		if (warp == 0) { const float v = warp_sum(s_warp[lane]); if (lane == 0) s_row[1] = round_to<B>(v); }
		__syncthreads();
		const float inv_total = fast_rcp(s_row[1]);
		for (int i = tid; i < n_cols; i += 1024) store_one<B>(out, base + i, fast_exp(round_to<B>(load_one<F>(X, base + i) - row_max)) * inv_total);
		__syncthreads();                      // s_warp and s_row are reused by the next row
	}
}

// pred[r, labels[r]] -= 1 in the tensor's own type (intended semantics of
// src/ops/nvidia/loss/cross_entropy.cu:33-44, whose row index is always 0 as written).
template <typename B>
__global__ void cross_entropy_step_kernel(int n_rows, int n_cols, void * pred, const uint32_t * __restrict__ labels) {
	const int row = blockIdx.x * blockDim.x + threadIdx.x;
	if (row >= n_rows) return;
	const uint32_t label = labels[row];
	if (label >= (uint32_t) n_cols) return;
	const uint64_t idx = (uint64_t) row * (uint64_t) n_cols + label;
	if constexpr (Word<B>::EPW == 1) {
		float * p = reinterpret_cast<float *>(pred) + idx;
		*p = *p - 1.0f;
	} else {
		uint16_t * p = reinterpret_cast<uint16_t *>(pred) + idx;
		float pair[2];
		Word<B>::unpack((uint32_t) *p, pair);
		pair[0] -= 1.0f; pair[1] = 0.0f;
		*p = (uint16_t) (Word<B>::pack(pair) & 0xffffu);
	}
}

// loss_sum[0] = sum of row_loss over rows with a valid label (fp64, fixed order), loss_sum[1] = their count.
__global__ void __launch_bounds__(1024)
loss_sum_kernel(int n_rows, int n_cols, const float * __restrict__ row_loss, const uint32_t * __restrict__ labels, float * loss_sum) {
	__shared__ double s_sum[1024];
	__shared__ unsigned s_cnt[1024];
	double acc = 0.0;
	unsigned cnt = 0;
	// eight rows per thread in flight; the additions keep the order r, r + 1024, r + 2048, ...
	int r = threadIdx.x;
	for (; r + 7 * 1024 < n_rows; r += 8 * 1024) {
		uint32_t l[8];
		float v[8];
		#pragma unroll
		for (int i = 0; i < 8; i++) { l[i] = __ldg(labels + r + i * 1024); v[i] = row_loss[r + i * 1024]; }
		#pragma unroll
		for (int i = 0; i < 8; i++)
			if (l[i] < (uint32_t) n_cols) { acc += (double) v[i]; cnt++; }
	}
	for (; r < n_rows; r += 1024) {
		if (labels[r] < (uint32_t) n_cols) { acc += (double) row_loss[r]; cnt++; }
	}
	s_sum[threadIdx.x] = acc; s_cnt[threadIdx.x] = cnt;
	__syncthreads();
	for (int o = 512; o > 0; o >>= 1) {
		if (threadIdx.x < o) { s_sum[threadIdx.x] += s_sum[threadIdx.x + o]; s_cnt[threadIdx.x] += s_cnt[threadIdx.x + o]; }
		__syncthreads();
	}
	if (threadIdx.x == 0) { loss_sum[0] = (float) s_sum[0]; loss_sum[1] = (float) s_cnt[0]; }
}

// Number of this launch for the abort word of wait_pushed: 1, 2, ... (0, the word's initial value, is never used).
static unsigned int next_launch_epoch() {
	static unsigned int counter = 0;
	unsigned int e = __atomic_add_fetch(&counter, 1u, __ATOMIC_RELAXED);
	if (e == 0) e = __atomic_add_fetch(&counter, 1u, __ATOMIC_RELAXED);
	return e;
}

struct SoftmaxGeometry { int cluster, threads, cpt, slice_chunks, spt; };      // spt > 0: packets per thread kept in shared memory

// The form with shared-memory packets: per thread 8 + 8 packets of 16 bytes (16-bit elements) or 4 + 4 packets of 32 bytes (fp32), i.e.
// 32 words of the row in registers and 64 KB of shared memory per 512-thread CTA in both cases.
constexpr int SOFTMAX_SPT_16BIT = 8, SOFTMAX_SPT_FP32 = 4;

// packet_bytes = bytes of one 8-element chunk in the input type (8 for fp8, 16 for fp16 / bf16, 32 for fp32)
static bool softmax_geometry(int n_chunks, int packet_bytes, SoftmaxGeometry * g) {
	g->spt = 0;
	// Long rows of 16- and 32-bit elements: CTAs of up to 512 threads with half of their packets in registers and half in shared memory.
	// The smallest cluster that holds the row -- 16-bit: one CTA for rows of up to 65536 elements, two up to 131072, four up to 262144;
	// fp32: one CTA up to 32768 elements, clusters of two, four and eight up to 262144 -- is then widened to more, smaller CTAs (below).
	// Shorter rows (<= 32 words per thread) stay in registers.
	const int half = packet_bytes == 16 ? SOFTMAX_SPT_16BIT : packet_bytes == 32 ? SOFTMAX_SPT_FP32 : 0;
	if (half && n_chunks > SOFTMAX_MAX_THREADS * half && n_chunks <= SOFTMAX_MAX_CLUSTER * SOFTMAX_MAX_THREADS * 2 * half &&
	    SOFTMAX_MAX_CPT == 8 && SOFTMAX_MAX_THREADS == 512) {
		const int per_cta = SOFTMAX_MAX_THREADS * 2 * half;
		int cluster = 1;
		while (cluster * per_cta < n_chunks) cluster *= 2;
		auto shape_of = [&](int cl, int * slice_out, int * threads_out) {
			int sl = (n_chunks + cl - 1) / cl;
			sl = (sl + SLICE_ALIGN_CHUNKS - 1) / SLICE_ALIGN_CHUNKS * SLICE_ALIGN_CHUNKS;
			int th = (sl + 2 * half - 1) / (2 * half);
			th = (th + 127) / 128 * 128;
			*slice_out = sl; *threads_out = th;
		};
		int slice, threads;
		shape_of(cluster, &slice, &threads);
		// More, smaller CTAs per row: eight 128-thread CTAs on an SM interleave their load / exponential / store phases more finely than
		// two of 512 threads (16384 x 128256 bf16, fused cross entropy: clusters of 2 x 512 threads 1468 us, 4 x 256 1403 us, 8 x 128
		// 1391 us). The cluster is widened while the CTAs keep at least 128 threads and the thread slots that the 128-thread
		// granularity leaves empty do not grow beyond a tenth of the row.
		while (cluster * 2 <= SOFTMAX_MAX_CLUSTER && threads > 128) {
			int slice2, threads2;
			shape_of(cluster * 2, &slice2, &threads2);
			const double slots = (double) cluster * threads * 2 * half / n_chunks, slots2 = (double) cluster * 2 * threads2 * 2 * half / n_chunks;
			if (slots2 > (slots > 1.1 ? slots : 1.1)) break;
			cluster *= 2; slice = slice2; threads = threads2;
		}
		if (cluster <= SOFTMAX_MAX_CLUSTER && threads <= SOFTMAX_MAX_THREADS) {
			g->cluster = cluster; g->threads = threads; g->cpt = half; g->slice_chunks = slice;
			g->spt = half;
			return true;
		}
	}
	// smallest cluster whose CTAs (<= 512 threads, <= 8 packets per thread) cover the row
	int cluster = 1;
	while (cluster < SOFTMAX_MAX_CLUSTER && (long long) cluster * SOFTMAX_MAX_THREADS * SOFTMAX_MAX_CPT < n_chunks) cluster *= 2;
	int slice = (n_chunks + cluster - 1) / cluster;
	slice = (slice + SLICE_ALIGN_CHUNKS - 1) / SLICE_ALIGN_CHUNKS * SLICE_ALIGN_CHUNKS;
	if (slice > SOFTMAX_MAX_THREADS * SOFTMAX_MAX_CPT) return false;
	// (cluster > 1 implies slices of more than 2048 chunks, so the 128-chunk alignment never leaves a CTA without work)
	// threads: multiple of 128; packets per thread: power of two, as few as keep the CTA <= 512 threads
	int cpt = 1;
	while (cpt < SOFTMAX_MAX_CPT && (slice + cpt - 1) / cpt > SOFTMAX_MAX_THREADS) cpt *= 2;
	// prefer >= 4 packets in flight per thread once the row is long enough to fill 128 threads with them
	while (cpt < 4 && slice / (cpt * 2) >= 128) cpt *= 2;
	int threads = (slice + cpt - 1) / cpt;
	threads = (threads + 127) / 128 * 128;
	if (threads > SOFTMAX_MAX_THREADS) return false;
	if (cluster > 1 && cpt != 8) return false;     // the cluster forms of the kernel exist for 8 packets per thread only (never taken: see above)
	g->cluster = cluster; g->threads = threads; g->cpt = cpt; g->slice_chunks = slice;
	return true;
}

// The form with shared-memory packets (16-bit inputs, long rows).
template <typename F, typename B, bool FUSE_CE, typename OUT, bool ARGMAX>
static int launch_softmax_long_rows(const SoftmaxGeometry & g, int n_rows, int n_cols, const void * X, void * out, const uint32_t * labels, float * row_loss,
                                    uint32_t * arg_maxs, cudaStream_t stream) {
	if constexpr (Word<F>::EPW > 2) {
		return set_error(DFB200_ERR_DTYPE, "softmax: internal geometry error");
	} else {
		constexpr int HALF = Word<F>::EPW == 2 ? SOFTMAX_SPT_16BIT : SOFTMAX_SPT_FP32;       // packets per thread in registers = in shared memory
		constexpr int QW = (E / Word<F>::EPW) / 4;
		if (g.spt != HALF || g.cpt != HALF) return set_error(DFB200_ERR_DTYPE, "softmax: internal geometry error");
		const size_t smem = (size_t) HALF * QW * g.threads * sizeof(uint4);
		unsigned int * status = kernel_status_word(STATUS_SOFTMAX);
		const unsigned int epoch = next_launch_epoch();
		cudaLaunchConfig_t cfg = {};
		cfg.gridDim = dim3((unsigned) n_rows * g.cluster, 1, 1);
		cfg.blockDim = dim3(g.threads, 1, 1);
		cfg.dynamicSmemBytes = smem;
		cfg.stream = stream;
		cudaLaunchAttribute attr[1];
		attr[0].id = cudaLaunchAttributeClusterDimension;
		attr[0].val.clusterDim.x = g.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
		cfg.attrs = attr; cfg.numAttrs = 1;
		auto kernel = g.cluster > 1 ? softmax_rows_kernel<F, B, HALF, FUSE_CE, OUT, ARGMAX, HALF, true>
		                            : softmax_rows_kernel<F, B, HALF, FUSE_CE, OUT, ARGMAX, HALF, false>;
		allow_dyn_smem(reinterpret_cast<const void *>(kernel), smem);
		const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, n_rows, n_cols, g.slice_chunks, X, out, labels, row_loss, arg_maxs, status, epoch);
		if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "softmax launch: %s", cudaGetErrorString(e)); }
		return DFB200_OK;
	}
}

template <typename F, typename B, bool FUSE_CE>
static int launch_softmax_rows(const SoftmaxGeometry & g, int n_rows, int n_cols, const void * X, void * out, const uint32_t * labels,
                               float * row_loss, cudaStream_t stream) {
	if (g.spt) return launch_softmax_long_rows<F, B, FUSE_CE, B, false>(g, n_rows, n_cols, X, out, labels, row_loss, nullptr, stream);
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3((unsigned) n_rows * g.cluster, 1, 1);
	cfg.blockDim = dim3(g.threads, 1, 1);
	cfg.dynamicSmemBytes = 0;
	cfg.stream = stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = g.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
	cfg.attrs = attr; cfg.numAttrs = 1;
	uint32_t * no_argmax = nullptr;
	unsigned int * status = kernel_status_word(STATUS_SOFTMAX);
	const unsigned int epoch = next_launch_epoch();
	cudaError_t e;
	switch (g.cpt) {
		case 1:  e = cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, B, 1, FUSE_CE>, n_rows, n_cols, g.slice_chunks, X, out, labels, row_loss, no_argmax, status, epoch); break;
		case 2:  e = cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, B, 2, FUSE_CE>, n_rows, n_cols, g.slice_chunks, X, out, labels, row_loss, no_argmax, status, epoch); break;
		case 4:  e = cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, B, 4, FUSE_CE>, n_rows, n_cols, g.slice_chunks, X, out, labels, row_loss, no_argmax, status, epoch); break;
		default: e = g.cluster > 1 ? cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, B, 8, FUSE_CE, B, false, 0, true>, n_rows, n_cols, g.slice_chunks, X, out, labels, row_loss, no_argmax, status, epoch)
		                           : cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, B, 8, FUSE_CE>, n_rows, n_cols, g.slice_chunks, X, out, labels, row_loss, no_argmax, status, epoch);
		         break;
	}
	if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "softmax launch: %s", cudaGetErrorString(e)); }
	return DFB200_OK;
}

template <typename F>
static int launch_softmax_fp32_out(const SoftmaxGeometry & g, int n_rows, int n_cols, const void * X, float * out, uint32_t * arg_maxs, cudaStream_t stream) {
	if (g.spt) {
		return arg_maxs ? launch_softmax_long_rows<F, F, false, f32_t, true>(g, n_rows, n_cols, X, out, nullptr, nullptr, arg_maxs, stream)
		                : launch_softmax_long_rows<F, F, false, f32_t, false>(g, n_rows, n_cols, X, out, nullptr, nullptr, nullptr, stream);
	}
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3((unsigned) n_rows * g.cluster, 1, 1);
	cfg.blockDim = dim3(g.threads, 1, 1);
	cfg.stream = stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = g.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
	cfg.attrs = attr; cfg.numAttrs = 1;
	const uint32_t * no_labels = nullptr;
	unsigned int * status = kernel_status_word(STATUS_SOFTMAX);
	const unsigned int epoch = next_launch_epoch();
	float * no_loss = nullptr;
	void * o = out;
	cudaError_t e;
#define DFB200_SOFTMAX_F32_CASE(CPT_, MULTI_) \
	(arg_maxs ? cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, F, CPT_, false, f32_t, true, 0, MULTI_>, n_rows, n_cols, g.slice_chunks, X, o, no_labels, no_loss, arg_maxs, status, epoch) \
	          : cudaLaunchKernelEx(&cfg, softmax_rows_kernel<F, F, CPT_, false, f32_t, false, 0, MULTI_>, n_rows, n_cols, g.slice_chunks, X, o, no_labels, no_loss, arg_maxs, status, epoch))
	switch (g.cpt) {
		case 1:  e = DFB200_SOFTMAX_F32_CASE(1, false); break;
		case 2:  e = DFB200_SOFTMAX_F32_CASE(2, false); break;
		case 4:  e = DFB200_SOFTMAX_F32_CASE(4, false); break;
		default: e = g.cluster > 1 ? DFB200_SOFTMAX_F32_CASE(8, true) : DFB200_SOFTMAX_F32_CASE(8, false); break;
	}
#undef DFB200_SOFTMAX_F32_CASE
	if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "softmax (fp32 out) launch: %s", cudaGetErrorString(e)); }
	return DFB200_OK;
}

static int check_softmax(const char * op, int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void * X, const void * out, SoftmaxGeometry * g) {
	if (!valid_fwd_bwd_pair(fwd_dt, bwd_dt)) return set_error(DFB200_ERR_DTYPE, "%s: unsupported datatype pair (%d, %d)", op, fwd_dt, bwd_dt);
	if (n_rows < 0 || n_cols <= 0) return set_error(DFB200_ERR_ARG, "%s: bad shape %d x %d", op, n_rows, n_cols);
	if (n_cols % E) return set_error(DFB200_ERR_ARG, "%s: n_cols = %d is not a multiple of %d", op, n_cols, E);
	if ((long long) n_rows * SOFTMAX_MAX_CLUSTER > 0x7fffffffLL) return set_error(DFB200_ERR_ARG, "%s: too many rows", op);
	const int packet_bytes = fwd_dt == DATAFLOW_FP32 ? 32 : (fwd_dt == DATAFLOW_FP16 || fwd_dt == DATAFLOW_BF16) ? 16 : 8;
	if (n_cols > SOFTMAX_MAX_CLUSTER * SOFTMAX_MAX_THREADS * SOFTMAX_MAX_CPT * E || !softmax_geometry(n_cols / E, packet_bytes, g))
		return set_error(DFB200_ERR_ARG, "%s: n_cols = %d exceeds the supported maximum of %d", op, n_cols,
		                 SOFTMAX_MAX_CLUSTER * SOFTMAX_MAX_THREADS * SOFTMAX_MAX_CPT * E);
	if (n_rows && (!X || !out)) return set_error(DFB200_ERR_ARG, "%s: NULL tensor argument", op);
	if (!aligned16(X) || !aligned16(out)) return set_error(DFB200_ERR_ARG, "%s: tensors must be 16-byte aligned", op);
	return DFB200_OK;
}

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_softmax(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void * X, void * out, void * stream) {
	SoftmaxGeometry g;
	// rows that are not multiples of 8 elements, rows beyond the on-chip forms and tensors that are only element-aligned: the general kernel
	if (valid_fwd_bwd_pair(fwd_dt, bwd_dt) && n_rows > 0 && n_cols > 0 && X && out &&
	    (n_cols % E || !aligned16(X) || !aligned16(out) || n_cols > SOFTMAX_MAX_CLUSTER * SOFTMAX_MAX_THREADS * SOFTMAX_MAX_CPT * E)) {
		if (reinterpret_cast<uintptr_t>(X) % (uintptr_t) dtype_size(fwd_dt) || reinterpret_cast<uintptr_t>(out) % (uintptr_t) dtype_size(bwd_dt))
			return set_error(DFB200_ERR_ARG, "softmax: tensors must be aligned to their element size");
		const long long cap = (long long) (sm_count() > 0 ? sm_count() : 1) * 2;
		const unsigned grid = (unsigned) (n_rows < cap ? n_rows : cap);
		DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B, (softmax_general_kernel<F, B><<<grid, 1024, 0, (cudaStream_t) stream>>>(n_rows, n_cols, X, out)));
		return check_launch("softmax (general shape)");
	}
	int rc = check_softmax("softmax", fwd_dt, bwd_dt, n_rows, n_cols, X, out, &g);
	if (rc || n_rows == 0) return rc;
	rc = DFB200_ERR_DTYPE;
	if (g.spt && dtype_size(fwd_dt) == 2) {
		// Long rows of 16-bit elements (the form with shared-memory packets): the instantiation with the cross-entropy step compiled in, given no labels,
		// so that no row has one. Measured, bf16: 16384 x 128256 1452 -> 1370 us, 32768 x 65536 1394 -> 1351 us (same registers, same
		// bytes; the compiler's schedule of the two instantiations differs). The register-only forms of shorter rows are the other
		// way round (262144 x 4096: 712 against 743 us), and so are fp32 rows (8192 x 128256: 1776 against 1814 us): they keep their own.
		DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
			rc = (launch_softmax_rows<F, B, true>(g, n_rows, n_cols, X, out, nullptr, nullptr, (cudaStream_t) stream)));
		return rc;
	}
	DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
		rc = (launch_softmax_rows<F, B, false>(g, n_rows, n_cols, X, out, nullptr, nullptr, (cudaStream_t) stream)));
	return rc;
}

extern "C" int dfb200_softmax_fp32_out(int fwd_dt, int n_rows, int n_cols, const void * X, float * out, uint32_t * arg_maxs, void * stream) {
	if (fwd_dt != DATAFLOW_FP16 && fwd_dt != DATAFLOW_BF16)
		return set_error(DFB200_ERR_DTYPE, "softmax_fp32_out: input must be fp16 or bf16 (got %d)", fwd_dt);
	SoftmaxGeometry g;
	int rc = check_softmax("softmax_fp32_out", fwd_dt, fwd_dt, n_rows, n_cols, X, out, &g);
	if (rc || n_rows == 0) return rc;
	if (arg_maxs && (reinterpret_cast<uintptr_t>(arg_maxs) & 3u)) return set_error(DFB200_ERR_ARG, "softmax_fp32_out: arg_maxs must be 4-byte aligned");
	return fwd_dt == DATAFLOW_FP16 ? launch_softmax_fp32_out<f16_t>(g, n_rows, n_cols, X, out, arg_maxs, (cudaStream_t) stream)
	                               : launch_softmax_fp32_out<bf16_t>(g, n_rows, n_cols, X, out, arg_maxs, (cudaStream_t) stream);
}

extern "C" int dfb200_cross_entropy_loss(int bwd_dt, int n_rows, int n_cols, void * pred_logits, const uint32_t * labels, void * stream) {
	if (!(bwd_dt == DATAFLOW_FP32 || bwd_dt == DATAFLOW_FP16 || bwd_dt == DATAFLOW_BF16))
		return set_error(DFB200_ERR_DTYPE, "cross_entropy_loss: unsupported datatype %d", bwd_dt);
	if (n_rows < 0 || n_cols <= 0) return set_error(DFB200_ERR_ARG, "cross_entropy_loss: bad shape %d x %d", n_rows, n_cols);
	if (n_rows == 0) return DFB200_OK;
	if (!pred_logits || !labels) return set_error(DFB200_ERR_ARG, "cross_entropy_loss: NULL tensor argument");
	const int blocks = (n_rows + 255) / 256;
	DFB200_DISPATCH_PAIR(bwd_dt, bwd_dt, F, B,
		(cross_entropy_step_kernel<B><<<blocks, 256, 0, (cudaStream_t) stream>>>(n_rows, n_cols, pred_logits, labels)));
	return check_launch("cross_entropy_loss");
}

extern "C" uint64_t dfb200_softmax_cross_entropy_workspace_bytes(int n_rows, int n_cols) {
	(void) n_cols;
	return n_rows > 0 ? (uint64_t) n_rows * sizeof(float) : 0;
}

extern "C" int dfb200_softmax_cross_entropy(int fwd_dt, int bwd_dt, int n_rows, int n_cols, const void * logits, const uint32_t * labels,
                                            void * dlogits, float * row_loss, float * loss_sum, void * workspace, uint64_t workspace_bytes,
                                            void * stream) {
	SoftmaxGeometry g;
	int rc = check_softmax("softmax_cross_entropy", fwd_dt, bwd_dt, n_rows, n_cols, logits, dlogits, &g);
	if (rc || n_rows == 0) return rc;
	if (!labels) return set_error(DFB200_ERR_ARG, "softmax_cross_entropy: NULL labels");
	float * losses = row_loss;
	if (!losses && loss_sum) {
		if (!workspace || workspace_bytes < (uint64_t) n_rows * sizeof(float))
			return set_error(DFB200_ERR_WORKSPACE, "softmax_cross_entropy: needs %llu bytes of workspace, got %llu",
			                 (unsigned long long) n_rows * sizeof(float), (unsigned long long) workspace_bytes);
		losses = reinterpret_cast<float *>(workspace);
	}
	rc = DFB200_ERR_DTYPE;
	DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B,
		rc = (launch_softmax_rows<F, B, true>(g, n_rows, n_cols, logits, dlogits, labels, losses, (cudaStream_t) stream)));
	if (rc) return rc;
	if (loss_sum) {
		loss_sum_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(n_rows, n_cols, losses, labels, loss_sum);
		return check_launch("softmax_cross_entropy (loss sum)");
	}
	return DFB200_OK;
}
