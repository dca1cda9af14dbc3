// FP8-weight SwiGLU FFN, forward and input gradient, on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
//   forward   Aq, sa = quantise_rows(A);  g = (Aq Wg^T) sa sg;  u = (Aq Wu^T) sa su            [T, f] bf16 each
//             Hq, sh = quantise_rows( bf16(silu(g) u) );  Out = (Hq Wd^T) sh sd (+ residual)    [T, d] bf16
//   backward  dOq, s1 = quantise_rows(dOut * sd);  dH = (dOq Wd) s1;  dGUq, s2 = quantise_rows( swiglu_bwd_x(g, u, dH) * [sg | su] );
//             dA = (dGUq [Wg | Wu]) s2
//
// Weights are e4m3 with one fp32 scale per OUTPUT channel and are stored [out_features, in_features] (reduction
// dimension contiguous). tcgen05.mma kind::f8f6f4 needs both operands in 8 bits, so activations are quantised to e4m3
// with one fp32 scale per ROW (token); both scales leave the contraction and are applied to the fp32 accumulator in the
// epilogue. Scales that sit on a contraction index (backward) are folded into the activations before quantisation.
// The reference has no such op (its only GEMM is a cuBLASLt call without scale pointers,
// src/ops/nvidia/external/matmul_helper/src/matmul_helper.c:379-416); the arithmetic contract is the one restated by the
// CPU oracle (oracle_quantize_rows_e4m3, oracle_gemm_e4m3*, and the reference's own swiglu / swiglu_bwd_x arithmetic).
//
// GEMM kernel: persistent, warp-specialised, two accumulator stages in tensor memory (2 x 256 of the 512 columns) so that the
// epilogue of one tile overlaps the MMAs of the next:
//   warp 0      one thread issues TMA tile loads (cp.async.bulk.tensor, 128-byte swizzle) into a shared-memory ring,
//               completion on mbarriers;
//   warp 1      allocates the tensor memory; one thread issues tcgen05.mma (fp32 accumulation in TMEM) and tcgen05.commit,
//               which releases ring stages and finally signals the epilogue;
//   warps 2-9   read the accumulator with tcgen05.ld (two warps per 32-lane quarter, half of the columns each), apply the
//               scales (and, in the fused modes, SwiGLU or its backward), convert to bf16 and store.
// Two forms: CTA PAIRS on 256 x 256 tiles (tcgen05 cta_group::2; see gemm_e4m3_kernel) and one CTA per 128 x 256 tile.
// Every mbarrier wait is bounded and reports through the kernel status word.
#include "common.cuh"
#include "tma.cuh"

#include <cuda.h>

namespace dfb200 {

constexpr int GEMM_BM = 128, GEMM_BK = 128;            // BK in elements = bytes (e4m3)
constexpr int GEMM_BN_HALF = 128;                        // columns per accumulator half
constexpr int GEMM_EPI_WARPS = 8;                         // two per 32-lane quarter of the accumulator: each takes half of the column chunks
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;
constexpr uint32_t TMEM_COLS = 512;                      // two 256-column accumulator stages
constexpr uint32_t A_STAGE_BYTES = GEMM_BM * GEMM_BK;                   // 16 KB: 128 rows of A
constexpr uint32_t B_HALF_BYTES = GEMM_BN_HALF * GEMM_BK;               // 16 KB: 128 rows of B
// One CTA per tile: a stage holds A and both B halves (48 KB, 4 stages). CTA pair per tile: each CTA holds its own 128 rows
// of A and ONE B half (32 KB, 6 stages); the pair's tensor cores read the other half from the peer's shared memory.
template <bool PAIR> struct GemmShape {
#ifndef DFB200_PAIR_STAGES
#define DFB200_PAIR_STAGES 6
#endif
	static constexpr int STAGES = PAIR ? DFB200_PAIR_STAGES : 4;
	static constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + (PAIR ? 1 : 2) * B_HALF_BYTES;
	static constexpr int TILE_M = PAIR ? 2 * GEMM_BM : GEMM_BM;
	static constexpr size_t SMEM = 1024 + (size_t) STAGES * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 2 * sizeof(uint32_t) + 4 * GEMM_BN_HALF * sizeof(float);
};

// ---------------------------------------------------------------------------------------------------------------
// PTX wrappers (tensor-map TMA, tcgen05)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void * smem_dst, const CUtensorMap * map, int x, int y, uint64_t * bar) {
	asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
	             :: "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// The same load issued by a CTA of a pair: the completion may be counted on a barrier of the other CTA (`bar_cluster_addr`
// is a shared::cluster address, see mapa_u32).
__device__ __forceinline__ void tma_load_2d_pair(void * smem_dst, const CUtensorMap * map, int x, int y, uint32_t bar_cluster_addr) {
	asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
	             :: "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// shared::cluster address of the variable at this CTA's shared address `local` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
	uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t tx_bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" :: "r"(bar_cluster_addr), "r"(tx_bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
	asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(bar_cluster_addr) : "memory");
}
// mbar_wait_bounded with cluster-scope acquire, for barriers that CTAs of the pair arrive on remotely
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t * bar, uint32_t parity, unsigned int * status, unsigned int where) {
	auto try_wait = [&]() {
		uint32_t done;
		asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
		             : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
		return done != 0;
	};
	if (try_wait()) return true;
	const unsigned long long t0 = global_timer_ns();
	for (;;) {
		for (int i = 0; i < 1024; i++)
			if (try_wait()) return true;
		if (global_timer_ns() - t0 > WAIT_LIMIT_NS) break;
	}
	atomicMax(status, where);
	return false;
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap * map) {
	asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t * smem_slot, uint32_t cols) {
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(smem_slot)), "r"(cols) : "memory");
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
// Pair forms: one warp of EACH CTA of the pair executes them; the columns are allocated in both CTAs' tensor memory.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t * smem_slot, uint32_t cols) {
	asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(smem_slot)), "r"(cols) : "memory");
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
	asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// All tcgen05.mma issued so far by this thread arrive on `bar` when they have completed (and no longer read shared memory).
__device__ __forceinline__ void tc_commit(uint64_t * bar) {
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
	asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
	             "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
	             :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Pair forms, issued by one thread of the leader CTA only: the MMA spans both CTAs' tensor cores (M = 256: rows 0..127 accumulate in
// the leader's tensor memory, rows 128..255 in the peer's; each CTA's shared memory supplies its 128 rows of A and its half of B at
// the same offsets), and the commit arrives on the barrier at the same shared-memory offset in every CTA of `cta_mask`.
__device__ __forceinline__ void tc_commit_pair(uint64_t * bar, uint16_t cta_mask) {
	asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
	             :: "r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
	asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
	             "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
	             :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive fp32 columns of this warp's 32 lanes (thread i gets lane base+i).
__device__ __forceinline__ void tmem_ld_32cols(uint32_t taddr, float (&v)[32]) {
	uint32_t r[32];
	asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
	             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
	               "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
	               "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
	             : "r"(taddr) : "memory");
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
	#pragma unroll
	for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major operand tile stored with the 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows (1024 bytes) stacked along M/N. Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30)
// (not used by swizzled K-major layouts; 1), stride byte offset >> 4 [32,46) = 1024 B between 8-row groups,
// descriptor version 1 [46,48), layout type SWIZZLE_128B = 2 [61,64).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(const void * smem_tile) {
	uint64_t d = (uint64_t) ((smem_u32(smem_tile) & 0x3ffffu) >> 4);
	d |= (uint64_t) 1 << 16;
	d |= (uint64_t) (1024 >> 4) << 32;
	d |= (uint64_t) 1 << 46;
	d |= (uint64_t) 2 << 61;
	return d;
}
// Instruction descriptor of kind::f8f6f4: D fp32 [4,6) = 1, A and B e4m3 (0), both K-major (0), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int m, int n) { return (1u << 4) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (m >> 4) << 24); }

// ---------------------------------------------------------------------------------------------------------------
// row quantisation: q[r, :] = e4m3( x[r, :] * (448 / amax_r) ),  scale[r] = amax_r / 448  (1 when the row is all zero)
// ---------------------------------------------------------------------------------------------------------------
// One CTA per row; the row stays PACKED in registers (4 words per 8 elements) between the two passes, so a thread holds few
// registers and an SM keeps 1800-2048 threads resident: bytes in flight come from occupancy. The optional per-column factors
// are re-read through the read-only cache in both passes (they are shared by every row, so they stay in L1/L2).
template <int VPT, bool HAS_MULT>
__global__ void __launch_bounds__(1024)
quantize_rows_e4m3_kernel(int n_rows, int n_cols, const void * __restrict__ X, const float * __restrict__ col_mult, void * __restrict__ Q,
                          float * __restrict__ scales) {
	__shared__ float red[32];
	const int n_chunks = n_cols / 8, tid = threadIdx.x, nthr = blockDim.x;
	const int row = blockIdx.x;
	const uint64_t row_elem = (uint64_t) row * (uint64_t) n_cols;
	uint32_t raw[VPT][4];
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		if (c < n_chunks) ld_words<4, Hint::STREAM>(reinterpret_cast<const char *>(X) + (row_elem + (uint64_t) c * 8) * 2, raw[v]);
	}
	auto scaled = [&](int v, int c, float (&x)[8]) {          // x = bf16 value * column factor (one fp32 rounding)
		#pragma unroll
		for (int i = 0; i < 4; i++) Word<bf16_t>::unpack(raw[v][i], &x[2 * i]);
		if constexpr (HAS_MULT) {
			const float4 m0 = __ldg(reinterpret_cast<const float4 *>(col_mult + (size_t) c * 8));
			const float4 m1 = __ldg(reinterpret_cast<const float4 *>(col_mult + (size_t) c * 8 + 4));
			x[0] = __fmul_rn(x[0], m0.x); x[1] = __fmul_rn(x[1], m0.y); x[2] = __fmul_rn(x[2], m0.z); x[3] = __fmul_rn(x[3], m0.w);
			x[4] = __fmul_rn(x[4], m1.x); x[5] = __fmul_rn(x[5], m1.y); x[6] = __fmul_rn(x[6], m1.z); x[7] = __fmul_rn(x[7], m1.w);
		}
	};
	float amax = 0.0f;
	if constexpr (HAS_MULT) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				float x[8];
				scaled(v, c, x);
				#pragma unroll
				for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(x[i]));
			}
		}
	} else {                                               // the maximum of the bf16 values themselves, on packed pairs
		__nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			if (tid + v * nthr < n_chunks) {
				#pragma unroll
				for (int i = 0; i < 4; i++) m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[v][i])));
			}
		}
		amax = fmaxf(__low2float(m2), __high2float(m2));
	}
	amax = warp_max(amax);
	if ((tid & 31) == 0) red[tid >> 5] = amax;
	__syncthreads();
	amax = red[0];
	for (int w = 1; w < (nthr >> 5); w++) amax = fmaxf(amax, red[w]);
	const float inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 1.0f;
	if (tid == 0) scales[row] = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		if (c < n_chunks) {
			float x[8], q[8];
			scaled(v, c, x);
			#pragma unroll
			for (int i = 0; i < 8; i++) q[i] = __fmul_rn(x[i], inv);
			store_elems<e4m3_t, 8>(Q, row_elem + (uint64_t) c * 8, q);
		}
	}
}

// Row quantisation fused with the elementwise op that produces the row, so that the bf16 intermediate never reaches memory:
//   FWD: h = bf16( silu(g) * u )                       -> codes [n_rows, f]   (the hidden activation of the FFN)
//   BWD: dg, du = swiglu_bwd_x(g, u, dh) in bf16, times the per-column factors -> codes [n_rows, 2f] = [dg | du]
// Arithmetic of the elementwise part is that of swiglu_fwd_kernel / swiglu_bwd_x_kernel (reference:
// src/ops/nvidia/activations/swiglu.cu:58-65, swiglu_bwd_x.cu:68-77), rounded to bf16 exactly where those kernels round; the
// quantisation is quantize_rows_e4m3_kernel's. One CTA per row, the bf16 results stay packed in registers between the passes.
template <int VPT, bool BWD, bool HAS_MULT>
__global__ void __launch_bounds__(1024, VPT <= 2 ? 2 : 1)
swiglu_quantize_rows_kernel(int n_rows, int f, const void * __restrict__ G, const void * __restrict__ U, const void * __restrict__ dH,
                            const float * __restrict__ col_mult, void * __restrict__ Q, float * __restrict__ scales, void * __restrict__ bf16_out) {
	__shared__ float red[32];
	const int n_chunks = f / 8, tid = threadIdx.x, nthr = blockDim.x;
	const int row = blockIdx.x;
	const uint64_t in_elem = (uint64_t) row * (uint64_t) f;
	constexpr int PARTS = BWD ? 2 : 1;                     // packed results per chunk: (dg, du) or h
	uint32_t res[VPT][PARTS][4];
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		if (c < n_chunks) {
			float g[8], u[8];
			load_elems<bf16_t, 8, Hint::STREAM>(G, in_elem + (uint64_t) c * 8, g);
			load_elems<bf16_t, 8, Hint::STREAM>(U, in_elem + (uint64_t) c * 8, u);
			if constexpr (BWD) {
				float dh[8], d1[8], d3[8];
				load_elems<bf16_t, 8, Hint::STREAM>(dH, in_elem + (uint64_t) c * 8, dh);
				#pragma unroll
				for (int i = 0; i < 8; i++) {                       // one reciprocal serves silu(g) and its derivative
					const float e = __expf(-g[i]), ope = 1.0f + e, r = fast_rcp(ope);
					d3[i] = dh[i] * (g[i] * r);
					d1[i] = dh[i] * ((u[i] * (ope + g[i] * e)) * (r * r));
				}
				#pragma unroll
				for (int i = 0; i < 4; i++) { res[v][0][i] = Word<bf16_t>::pack(&d1[2 * i]); res[v][1][i] = Word<bf16_t>::pack(&d3[2 * i]); }
			} else {
				float h[8];
				#pragma unroll
				for (int i = 0; i < 8; i++) h[i] = __fdividef(g[i], 1.0f + __expf(-g[i])) * u[i];
				#pragma unroll
				for (int i = 0; i < 4; i++) res[v][0][i] = Word<bf16_t>::pack(&h[2 * i]);
			}
		}
	}
	auto scaled = [&](int v, int part, int c, float (&x)[8]) {          // bf16 result * column factor (one fp32 rounding)
		#pragma unroll
		for (int i = 0; i < 4; i++) Word<bf16_t>::unpack(res[v][part][i], &x[2 * i]);
		if constexpr (HAS_MULT) {
			const float * m = col_mult + (size_t) part * f + (size_t) c * 8;
			const float4 m0 = __ldg(reinterpret_cast<const float4 *>(m)), m1 = __ldg(reinterpret_cast<const float4 *>(m + 4));
			x[0] = __fmul_rn(x[0], m0.x); x[1] = __fmul_rn(x[1], m0.y); x[2] = __fmul_rn(x[2], m0.z); x[3] = __fmul_rn(x[3], m0.w);
			x[4] = __fmul_rn(x[4], m1.x); x[5] = __fmul_rn(x[5], m1.y); x[6] = __fmul_rn(x[6], m1.z); x[7] = __fmul_rn(x[7], m1.w);
		}
	};
	float amax = 0.0f;
	if constexpr (HAS_MULT) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				#pragma unroll
				for (int part = 0; part < PARTS; part++) {
					float x[8];
					scaled(v, part, c, x);
					#pragma unroll
					for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(x[i]));
				}
			}
		}
	} else {                                               // no factors: the maximum of the bf16 values themselves, on packed pairs
		__nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				#pragma unroll
				for (int part = 0; part < PARTS; part++)
					#pragma unroll
					for (int i = 0; i < 4; i++) m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&res[v][part][i])));
			}
		}
		amax = fmaxf(__low2float(m2), __high2float(m2));
	}
	amax = warp_max(amax);
	if ((tid & 31) == 0) red[tid >> 5] = amax;
	__syncthreads();
	amax = red[0];
	for (int w = 1; w < (nthr >> 5); w++) amax = fmaxf(amax, red[w]);
	const float inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 1.0f;
	if (tid == 0) scales[row] = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
	const uint64_t out_elem = (uint64_t) row * (uint64_t) (PARTS * f);
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		if (c < n_chunks) {
			#pragma unroll
			for (int part = 0; part < PARTS; part++) {
				float x[8], q[8];
				scaled(v, part, c, x);
				#pragma unroll
				for (int i = 0; i < 8; i++) q[i] = __fmul_rn(x[i], inv);
				store_elems<e4m3_t, 8>(Q, out_elem + (uint64_t) part * f + (uint64_t) c * 8, q);
				// the bf16 values themselves (before the column factors), for the weight-gradient pass
				if (bf16_out) st_words<4>(reinterpret_cast<char *>(bf16_out) + (out_elem + (uint64_t) part * f + (uint64_t) c * 8) * 2, res[v][part]);
			}
		}
	}
}

// Weight gradients contract over the TOKENS, so their operands are the transposes of activation matrices, quantised with one scale
// per row of the transpose (= per column of the activation matrix; no scale sits on the contraction index):
//   col_amax_kernel          amax[c] = max_r |X[r, c]|           (persistent CTAs keep packed running maxima per column chunk in registers
//                                                                 and merge them with one integer atomicMax per column: order-independent)
//   transpose_quantize_kernel Qt[c, r] = e4m3( X[r, c] * (448 / amax[c]) ), scale[c] = amax[c] / 448 (1 for an all-zero column);
//                            128-token x 64-column tiles through shared memory, 128-byte rows of the transpose per store group
template <int VPT>
__global__ void __launch_bounds__(1024)
col_amax_kernel(int n_rows, int n_cols, int group_threads, const void * __restrict__ X, float * amax) {
	extern __shared__ unsigned int s_max[];                // [n_cols] maxima of this CTA (bit patterns of non-negative floats order like the floats)
	const int n_chunks = n_cols / 8;
	const int groups = blockDim.x / group_threads, g = threadIdx.x / group_threads, tid = threadIdx.x - g * group_threads;
	for (int c = threadIdx.x; c < n_cols; c += blockDim.x) s_max[c] = 0u;
	__nv_bfloat162 m[VPT][4];
	#pragma unroll
	for (int v = 0; v < VPT; v++)
		#pragma unroll
		for (int i = 0; i < 4; i++) m[v][i] = __float2bfloat162_rn(0.0f);
	// one CTA per SM; its row groups take interleaved rows, ROWS of them per iteration so that a thread has several loads in flight
	constexpr int ROWS = VPT == 1 ? 4 : 2;
	const int stride = gridDim.x * groups;
	for (int row0 = blockIdx.x * groups + g; row0 < n_rows && g < groups; row0 += ROWS * stride) {
		uint32_t raw[ROWS][VPT][4];
		#pragma unroll
		for (int r = 0; r < ROWS; r++) {
			const int row = row0 + r * stride;
			#pragma unroll
			for (int v = 0; v < VPT; v++) {
				const int c = tid + v * group_threads;
				if (row < n_rows && c < n_chunks) ld_words<4, Hint::STREAM>(reinterpret_cast<const char *>(X) + ((uint64_t) row * n_cols + (uint64_t) c * 8) * 2, raw[r][v]);
			}
		}
		#pragma unroll
		for (int r = 0; r < ROWS; r++) {
			if (row0 + r * stride >= n_rows) continue;
			#pragma unroll
			for (int v = 0; v < VPT; v++) {
				if (tid + v * group_threads < n_chunks) {
					#pragma unroll
					for (int i = 0; i < 4; i++) m[v][i] = __hmax2(m[v][i], __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[r][v][i])));
				}
			}
		}
	}
	__syncthreads();                                       // s_max cleared
	if (g < groups) {
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * group_threads;
			if (c < n_chunks) {
				#pragma unroll
				for (int i = 0; i < 4; i++) {
					atomicMax(&s_max[c * 8 + 2 * i], __float_as_uint(__low2float(m[v][i])));
					atomicMax(&s_max[c * 8 + 2 * i + 1], __float_as_uint(__high2float(m[v][i])));
				}
			}
		}
	}
	__syncthreads();
	for (int c = threadIdx.x; c < n_cols; c += blockDim.x)
		if (s_max[c]) atomicMax(reinterpret_cast<unsigned int *>(amax) + c, s_max[c]);
}

constexpr int TQ_TOKENS = 128, TQ_COLS = 64, TQ_PITCH = TQ_TOKENS + 4;
__global__ void __launch_bounds__(256)
transpose_quantize_kernel(int n_rows, int n_cols, const void * __restrict__ X, const float * __restrict__ amax, uint8_t * __restrict__ Qt,
                          float * __restrict__ col_scales) {
	__shared__ __align__(16) uint8_t tile[TQ_COLS][TQ_PITCH];          // [column][token] codes
	__shared__ float inv[TQ_COLS];
	const int r0 = blockIdx.y * TQ_TOKENS, c0 = blockIdx.x * TQ_COLS, tid = threadIdx.x;
	if (tid < TQ_COLS) {
		const int c = c0 + tid;
		const float a = c < n_cols ? amax[c] : 0.0f;
		inv[tid] = a > 0.0f ? __fdiv_rn(448.0f, a) : 1.0f;
		if (blockIdx.y == 0 && c < n_cols) col_scales[c] = a > 0.0f ? __fdiv_rn(a, 448.0f) : 1.0f;
	}
	__syncthreads();
	// phase 1: 32 token quads x 8 column chunks, one item per thread. 8 consecutive lanes read one 128-byte row segment of each of
	// their quad's 4 tokens; the 4 tokens' codes of a column go to the tile as ONE 32-bit store (byte stores, one per element, made
	// the shared-memory store pipe the limiter of this kernel: 4.5 TB/s).
	{
		static_assert(TQ_TOKENS * TQ_COLS / 32 == 256, "one (token quad, column chunk) item per thread");
		const int q = tid >> 3, ch = tid & 7;
		const int c = c0 + ch * 8;
		float x[4][8];
		#pragma unroll
		for (int j = 0; j < 4; j++) {
			const int r = r0 + 4 * q + j;
			if (r < n_rows && c < n_cols) load_elems<bf16_t, 8, Hint::STREAM>(X, (uint64_t) r * n_cols + c, x[j]);
			else { for (int i = 0; i < 8; i++) x[j][i] = 0.0f; }
		}
		#pragma unroll
		for (int i = 0; i < 8; i++) {
			const float f = inv[ch * 8 + i];
			const __nv_fp8x2_storage_t p01 = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(x[0][i], f), __fmul_rn(x[1][i], f)), __NV_SATFINITE, __NV_E4M3);
			const __nv_fp8x2_storage_t p23 = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(x[2][i], f), __fmul_rn(x[3][i], f)), __NV_SATFINITE, __NV_E4M3);
			*reinterpret_cast<uint32_t *>(&tile[ch * 8 + i][4 * q]) = (uint32_t) p01 | ((uint32_t) p23 << 16);
		}
	}
	__syncthreads();
	// phase 2: 64 columns x 8 segments of 16 tokens; 8 consecutive lanes write one 128-byte row of the transpose
	#pragma unroll
	for (int k = 0; k < (TQ_COLS * TQ_TOKENS / 16) / 256; k++) {
		const int item = tid + k * 256, cl = item >> 3, seg = item & 7;
		const int c = c0 + cl, r = r0 + seg * 16;
		if (c < n_cols && r < n_rows) {                 // n_rows is a multiple of 16
			const uint32_t * src = reinterpret_cast<const uint32_t *>(&tile[cl][seg * 16]);
			*reinterpret_cast<uint4 *>(Qt + (uint64_t) c * n_rows + r) = make_uint4(src[0], src[1], src[2], src[3]);
		}
	}
}

// out[c, r] = in[r, c] for byte matrices (weight codes): 32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256)
transpose_bytes_kernel(int rows, int cols, const uint8_t * __restrict__ in, int ld_in, uint8_t * __restrict__ out, int ld_out) {
	__shared__ uint8_t tile[32][33];
	const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
	const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
	for (int i = ty; i < 32; i += 8)
		if (r0 + i < rows && c0 + tx < cols) tile[i][tx] = in[(size_t) (r0 + i) * ld_in + c0 + tx];
	__syncthreads();
	for (int i = ty; i < 32; i += 8)
		if (c0 + i < cols && r0 + tx < rows) out[(size_t) (c0 + i) * ld_out + r0 + tx] = tile[tx][i];
}

// ---------------------------------------------------------------------------------------------------------------
// GEMM: D[m, n] = sum_k A[m, k] * B[n, k]  (e4m3 x e4m3 -> fp32 in TMEM), two 128-column halves per CTA.
//   MODE_SWIGLU    : half 0 = gate rows n0.., half 1 = up rows n0.. (tensor maps map_b0 / map_b1), 128 outputs:
//                    out[m, n0 + j] = bf16( silu(g) * u ),  g = acc0 * sa[m] * sb0[n], u = acc1 * sa[m] * sb1[n];
//                    g and u are also stored (bf16) to aux0 / aux1 when those are given (saved for the backward pass)
//   MODE_PLAIN     : halves are columns n0.. and n0 + 128.. of one weight matrix (map_b0 twice), 256 outputs:
//                    out[m, n] = bf16( acc * sa[m] * sb0[n] + residual[m, n] )   (sb0 == NULL: no column scale; residual = aux0, optional)
//   MODE_SWIGLU_BWD: as MODE_PLAIN for dh = acc * sa[m] (gradient w.r.t. the hidden activation), then with the saved
//                    g = aux0[m, n], u = aux1[m, n]:  out[m, n] = bf16( dh * u * dsilu(g) ),  out[m, N + n] = bf16( dh * silu(g) )
//                    (gate and up gradients side by side in one [M, 2N] buffer, ld_out = 2N)
enum GemmMode { MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_SWIGLU_BWD = 2 };
// ---------------------------------------------------------------------------------------------------------------
// PAIR = false: one CTA per 128 x 256 tile. PAIR = true: launched as clusters of two CTAs that share one 256 x 256 tile
// (tcgen05 cta_group::2): per flop a CTA pulls a third less operand data through L2 -> shared memory, which is what bounds
// the one-CTA form. Roles in the pair: both CTAs load (their A rows, their B half) and run an epilogue (their 128 rows); the
// leader (cluster rank 0) alone issues the MMAs. Barrier ownership: full[] and accum_empty[] are the leader's (the peer
// arrives on them remotely), empty[] and accum_full[] exist in both CTAs and are signalled by multicast commits.
template <int MODE, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_e4m3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1,
                 int M, int N, int K, int tiles_m, int tiles_n, const float * __restrict__ sa, const float * __restrict__ sb0,
                 const float * __restrict__ sb1, void * out, int ld_out, void * aux0, void * aux1, unsigned int * status) {
	constexpr bool SWIGLU = MODE == MODE_SWIGLU;
	constexpr int GEMM_STAGES = GemmShape<PAIR>::STAGES;
	constexpr uint32_t STAGE_BYTES = GemmShape<PAIR>::STAGE_BYTES;
	constexpr int TILE_M = GemmShape<PAIR>::TILE_M;
	const uint32_t rank = PAIR ? cluster_ctarank() : 0u;       // position in the pair; 0 = leader
	const int walker = PAIR ? blockIdx.x >> 1 : blockIdx.x, n_walkers = PAIR ? gridDim.x >> 1 : gridDim.x;
	extern __shared__ uint8_t smem_raw[];
	uint8_t * smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);   // swizzled tiles need 1024-byte alignment
	uint8_t * ring = smem;
	uint64_t * full = reinterpret_cast<uint64_t *>(smem + GEMM_STAGES * STAGE_BYTES);
	uint64_t * empty = full + GEMM_STAGES;
	uint64_t * accum_full = empty + GEMM_STAGES;            // [2]
	uint64_t * accum_empty = accum_full + 2;                // [2]
	uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(accum_empty + 2);
	float * s_scale = reinterpret_cast<float *>(tmem_slot + 2);        // [2 accumulator stages][256] column scales of the tile

	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	constexpr int N_PER_TILE = SWIGLU ? GEMM_BN_HALF : 2 * GEMM_BN_HALF;
	const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
	const int num_tiles = tiles_m * tiles_n;

	// Persistent CTAs walk tiles blockIdx.x, + gridDim.x, ... Tile raster: groups of 16 row tiles sweep the column tiles,
	// so that the CTAs running at the same time share A and B tiles in L2.
	auto tile_origin = [&](int tile, int & m0, int & n0) {
		const int group = 16, tiles_per_group = group * tiles_n;
		const int g = tile / tiles_per_group, r = tile % tiles_per_group;
		const int rows_in_group = min(group, tiles_m - g * group);
		m0 = (g * group + r % rows_in_group) * TILE_M + (int) rank * GEMM_BM;      // this CTA's 128 rows of the tile
		n0 = (r / rows_in_group) * N_PER_TILE;
	};

	if (threadIdx.x == 0) {
		for (int s = 0; s < GEMM_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
		// the pair's loads arrive on the leader's full[] from both CTAs; 4 epilogue warps per CTA release an accumulator
		if (PAIR) for (int s = 0; s < GEMM_STAGES; s++) mbar_init(&full[s], 2);
		for (int a = 0; a < 2; a++) { mbar_init(&accum_full[a], 1); mbar_init(&accum_empty[a], (PAIR ? 2 : 1) * GEMM_EPI_WARPS); }
		mbar_fence_init();
		prefetch_tensormap(&map_a); prefetch_tensormap(&map_b0); prefetch_tensormap(&map_b1);
	}
	if (warp == 1) { if (PAIR) tmem_alloc_pair(tmem_slot, TMEM_COLS); else tmem_alloc(tmem_slot, TMEM_COLS); }
	tc_fence_before_sync();
	if (PAIR) cluster_sync_all(); else __syncthreads();        // barriers initialised and tensor memory allocated in both CTAs
	tc_fence_after_sync();
	const uint32_t tmem_base = *tmem_slot;

	if (warp == 0) {
		// ---------------- TMA producer: one stream of k-blocks across all of this CTA's tiles
		if (lane == 0) {
			uint32_t it = 0;
			bool ok = true;
			for (int tile = walker; tile < num_tiles && ok; tile += n_walkers) {
				int m0, n0;
				tile_origin(tile, m0, n0);
				for (int kb = 0; kb < num_kb; kb++, it++) {
					const int s = it % GEMM_STAGES;
					ok = mbar_wait_bounded(&empty[s], ((it / GEMM_STAGES) & 1) ^ 1, status, 0x300u + s);
					if (!ok) break;
					uint8_t * a_dst = ring + (size_t) s * STAGE_BYTES;
					uint8_t * b_dst = a_dst + A_STAGE_BYTES;
					if constexpr (PAIR) {
						// this CTA's share of the stage (A rows, one B half: the gate or the up tile, or the lower/upper 128 weight rows),
						// counted on the LEADER's full barrier
						const uint32_t leader_full = mapa_u32(smem_u32(&full[s]), 0);
						mbar_arrive_expect_tx_cluster(leader_full, STAGE_BYTES);
						tma_load_2d_pair(a_dst, &map_a, kb * GEMM_BK, m0, leader_full);
						if (SWIGLU) tma_load_2d_pair(b_dst, rank ? &map_b1 : &map_b0, kb * GEMM_BK, n0, leader_full);
						else tma_load_2d_pair(b_dst, &map_b0, kb * GEMM_BK, n0 + (int) rank * GEMM_BN_HALF, leader_full);
						continue;
					}
					mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
					tma_load_2d(a_dst, &map_a, kb * GEMM_BK, m0, &full[s]);
					if (SWIGLU) {
						tma_load_2d(b_dst, &map_b0, kb * GEMM_BK, n0, &full[s]);
						tma_load_2d(b_dst + GEMM_BN_HALF * GEMM_BK, &map_b1, kb * GEMM_BK, n0, &full[s]);
					} else {
						tma_load_2d(b_dst, &map_b0, kb * GEMM_BK, n0, &full[s]);
						tma_load_2d(b_dst + GEMM_BN_HALF * GEMM_BK, &map_b0, kb * GEMM_BK, n0 + GEMM_BN_HALF, &full[s]);
					}
				}
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer: accumulator stage (tile index % 2) lets the epilogue of one tile overlap the next tile's MMAs
		if (lane == 0 && rank == 0) {
			constexpr uint32_t idesc = umma_idesc_e4m3(TILE_M, 2 * GEMM_BN_HALF);
			uint32_t it = 0, local = 0;
			bool ok = true;
			for (int tile = walker; tile < num_tiles && ok; tile += n_walkers, local++) {
				const uint32_t acc_stage = local & 1;
				ok = PAIR ? mbar_wait_bounded_cluster(&accum_empty[acc_stage], ((local >> 1) & 1) ^ 1, status, 0x330u + acc_stage)
				          : mbar_wait_bounded(&accum_empty[acc_stage], ((local >> 1) & 1) ^ 1, status, 0x330u + acc_stage);
				if (!ok) break;
				tc_fence_after_sync();
				const uint32_t d_tmem = tmem_base + acc_stage * (2 * GEMM_BN_HALF);
				for (int kb = 0; kb < num_kb; kb++, it++) {
					const int s = it % GEMM_STAGES;
					ok = PAIR ? mbar_wait_bounded_cluster(&full[s], (it / GEMM_STAGES) & 1, status, 0x310u + s)
					          : mbar_wait_bounded(&full[s], (it / GEMM_STAGES) & 1, status, 0x310u + s);
					if (!ok) break;
					tc_fence_after_sync();
					const uint8_t * a_tile = ring + (size_t) s * STAGE_BYTES;
					// The two 128-row B halves are adjacent in shared memory and form one 256-row K-major tile, so a single
					// M128 x N256 x K32 instruction (the largest 1-CTA shape) fills both accumulator halves.
					const uint64_t da = umma_desc_k_sw128(a_tile);
					const uint64_t db = umma_desc_k_sw128(a_tile + A_STAGE_BYTES);
					#pragma unroll
					for (int j = 0; j < GEMM_BK / 32; j++) {          // K = 32 per instruction: advance 32 bytes inside the swizzle atom
						if (PAIR) tc_mma_f8_pair(d_tmem, da + 2 * j, db + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
						else tc_mma_f8(d_tmem, da + 2 * j, db + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
					}
					if (PAIR) tc_commit_pair(&empty[s], 3); else tc_commit(&empty[s]);     // stage reusable (in both CTAs) once these MMAs have read it
				}
				if (PAIR) tc_commit_pair(&accum_full[acc_stage], 3); else tc_commit(&accum_full[acc_stage]);   // accumulator complete (or abandoned) -> epilogue(s)
			}
		}
	} else {
		// ---------------- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 32
		const int quarter = warp & 3;
		const int etid = threadIdx.x - 64;                   // index among the epilogue threads
		const int col_half = (warp - 2) >> 2;                // which half of the tile's column chunks this warp handles
		uint32_t local = 0;
		bool ok = true;
		int tile = walker;
		for (; tile < num_tiles && ok; tile += n_walkers, local++) {
			const uint32_t acc_stage = local & 1;
			int m0, n0;
			tile_origin(tile, m0, n0);
			float * scale = s_scale + acc_stage * (2 * GEMM_BN_HALF);
			for (int j = etid; j < 2 * GEMM_BN_HALF; j += 32 * GEMM_EPI_WARPS) {         // column scales of this tile (buffer last read two tiles ago)
				const int half = j / GEMM_BN_HALF, col = SWIGLU ? n0 + (j % GEMM_BN_HALF) : n0 + j;
				const float * sb = (SWIGLU && half == 1) ? sb1 : sb0;
				scale[j] = col < N ? (sb ? __ldg(sb + col) : 1.0f) : 0.0f;
			}
			const int row = m0 + quarter * 32 + lane;
			const float a_scale = row < M ? __ldg(sa + row) : 0.0f;
			// Inputs the epilogue reads from global memory (saved g, u in the backward mode; the residual in the plain mode) are
			// requested one 32-column chunk ahead -- the first chunk before the accumulator is even complete -- so that their
			// latency overlaps the tensor-memory reads and the arithmetic of the chunk before.
			constexpr int N_CHUNKS = N_PER_TILE / 32;
			constexpr bool READS_AUX = MODE != MODE_SWIGLU;
			const bool reads_aux = READS_AUX && (MODE == MODE_SWIGLU_BWD || aux0 != nullptr);
			// Global accesses of the epilogue are made in the TRANSPOSED assignment: a thread owns one accumulator row (32 columns =
			// four 16-byte pieces per chunk), but a warp instruction in which every lane touches its own row would reach 32 different
			// 128-byte lines. Groups of four lanes therefore exchange pieces (transpose4, two shuffle rounds) so that in access i lane
			// 4k + j moves piece j of row 4k + i: four lanes cover 64 contiguous bytes and an instruction touches 8 lines instead of 32.
			const int grp_row0 = m0 + quarter * 32 + (lane & ~3), piece = lane & 3;
			auto cols_whole = [&](int c) { return n0 + c * 32 + 32 <= N; };           // warp-uniform: chunk c lies inside the matrix
			auto fetch = [&](const void * src, int c, uint4 (&r)[4]) {                   // r[i] = piece `piece` of row grp_row0 + i
				#pragma unroll
				for (int i = 0; i < 4; i++) {
					const int ri = grp_row0 + i;
					r[i] = ri < M ? __ldcs(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(src) + (size_t) ri * N + n0 + c * 32) + piece)
					              : make_uint4(0u, 0u, 0u, 0u);
				}
			};
			auto transpose4 = [&](uint4 (&a)[4]) {
				#pragma unroll
				for (int sft = 1; sft <= 2; sft <<= 1) {
					const bool upper = (lane & sft) != 0;
					#pragma unroll
					for (int i = 0; i < 4; i++) {
						if (i & sft) continue;
						const uint4 send = upper ? a[i] : a[i | sft];
						uint4 recv;
						recv.x = __shfl_xor_sync(0xffffffffu, send.x, sft); recv.y = __shfl_xor_sync(0xffffffffu, send.y, sft);
						recv.z = __shfl_xor_sync(0xffffffffu, send.z, sft); recv.w = __shfl_xor_sync(0xffffffffu, send.w, sft);
						if (upper) a[i] = recv; else a[i | sft] = recv;
					}
				}
			};
			auto unpack32 = [&](uint4 (&r)[4], float (&val)[32]) {                        // fetched words -> this thread's 32 columns
				transpose4(r);
				#pragma unroll
				for (int i = 0; i < 4; i++) {
					Word<bf16_t>::unpack(r[i].x, &val[8 * i]); Word<bf16_t>::unpack(r[i].y, &val[8 * i + 2]);
					Word<bf16_t>::unpack(r[i].z, &val[8 * i + 4]); Word<bf16_t>::unpack(r[i].w, &val[8 * i + 6]);
				}
			};
			static_assert(GEMM_EPI_WARPS == 8 && N_CHUNKS % 4 == 0, "two warps per quarter, an even number of chunks each");
			const int c_first = col_half * (N_CHUNKS / 2), c_end = c_first + N_CHUNKS / 2;
			uint4 pre0[2][4], pre1[2][4];                       // [chunk parity]: aux0 / aux1 words of the current and the next chunk
			if (reads_aux && cols_whole(c_first)) {
				fetch(aux0, c_first, pre0[0]);
				if constexpr (MODE == MODE_SWIGLU_BWD) fetch(aux1, c_first, pre1[0]);
			}
			const bool mine = mbar_wait_bounded(&accum_full[acc_stage], (local >> 1) & 1, status, 0x320u + acc_stage);
			// One named barrier over the 256 epilogue threads does two jobs: it publishes the scales, and it ANDs the
			// outcome of the wait so that all epilogue warps take the same branch (tcgen05.ld and the barrier are collective).
			uint32_t all_ok;
			asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
			             : "=r"(all_ok) : "r"((uint32_t) mine) : "memory");
			ok = all_ok != 0;
			tc_fence_after_sync();
			if (!ok) break;
			const uint32_t taddr = tmem_base + acc_stage * (2 * GEMM_BN_HALF) + ((uint32_t) (quarter * 32) << 16);
			// val = this thread's 32 columns of its row; dst = matrix base with row pitch `pitch`, columns starting at col0
			auto store32 = [&](void * dst, size_t pitch, int col0, const float (&val)[32], bool whole, int n_valid) {
				__nv_bfloat16 * base = reinterpret_cast<__nv_bfloat16 *>(dst);
				if (whole) {
					uint4 w[4];
					#pragma unroll
					for (int i = 0; i < 4; i++)
						w[i] = make_uint4(Word<bf16_t>::pack(&val[8 * i]), Word<bf16_t>::pack(&val[8 * i + 2]), Word<bf16_t>::pack(&val[8 * i + 4]),
						                  Word<bf16_t>::pack(&val[8 * i + 6]));
					transpose4(w);
					#pragma unroll
					for (int i = 0; i < 4; i++) {
						const int ri = grp_row0 + i;
						if (ri < M) *(reinterpret_cast<uint4 *>(base + (size_t) ri * pitch + col0) + piece) = w[i];
					}
				} else if (row < M) {
					for (int i = 0; i < n_valid; i++) base[(size_t) row * pitch + col0 + i] = __float2bfloat16_rn(val[i]);
				}
			};
			auto load32_edge = [&](const void * src, int col0, float (&val)[32]) {        // chunk that crosses the matrix edge
				const __nv_bfloat16 * src_row = reinterpret_cast<const __nv_bfloat16 *>(src) + (size_t) row * N;
				for (int i = 0; i < 32; i++) val[i] = (row < M && col0 + i < N) ? __bfloat162float(src_row[col0 + i]) : 0.0f;
			};
			// one 32-column chunk; `cur` holds its prefetched aux words, `nxt` receives the next chunk's
			auto chunk = [&](int c, uint4 (&cur0)[4], uint4 (&cur1)[4], uint4 (&nxt0)[4], uint4 (&nxt1)[4]) {
				float v0[32], o[32];
				const int col0 = n0 + c * 32;
				const bool whole = cols_whole(c);
				const int n_valid = min(32, N - col0);               // columns of this chunk inside the matrix (<= 0: none)
				if (READS_AUX && reads_aux && c + 1 < c_end && cols_whole(c + 1)) {
					fetch(aux0, c + 1, nxt0);
					if constexpr (MODE == MODE_SWIGLU_BWD) fetch(aux1, c + 1, nxt1);
				}
				if constexpr (MODE == MODE_SWIGLU) {
					float v1[32];
					tmem_ld_32cols(taddr + c * 32, v0);
					tmem_ld_32cols(taddr + GEMM_BN_HALF + c * 32, v1);
					#pragma unroll
					for (int i = 0; i < 32; i++) {
						v0[i] = (v0[i] * a_scale) * scale[c * 32 + i];                       // gate pre-activation
						v1[i] = (v1[i] * a_scale) * scale[GEMM_BN_HALF + c * 32 + i];        // up pre-activation
						o[i] = (v0[i] * fast_rcp(1.0f + fast_exp(-v0[i]))) * v1[i];
					}
					if (aux0) {
						store32(aux0, (size_t) N, col0, v0, whole, n_valid);
						store32(aux1, (size_t) N, col0, v1, whole, n_valid);
					}
				} else {
					tmem_ld_32cols(taddr + c * 32, v0);
					#pragma unroll
					for (int i = 0; i < 32; i++) o[i] = (v0[i] * a_scale) * scale[c * 32 + i];
					if (MODE == MODE_PLAIN && reads_aux) {                 // residual: out = bf16( acc * scales + residual )
						float res[32];
						if (whole) unpack32(cur0, res); else load32_edge(aux0, col0, res);
						#pragma unroll
						for (int i = 0; i < 32; i++) o[i] += res[i];
					}
				}
				if (c == c_end - 1) {                             // this warp's last read of the accumulator: hand it back to the MMA warp
					tc_fence_before_sync();
					__syncwarp();
					if (lane == 0) {
						if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&accum_empty[acc_stage]), 0));
						else mbar_arrive(&accum_empty[acc_stage]);
					}
				}
				if constexpr (MODE == MODE_SWIGLU_BWD) {
					// o = dL/dh; saved pre-activations give the gate and up gradients (same expressions as swiglu_bwd_x)
					float gte[32], up[32], dgate[32], dup[32];
					if (whole) { unpack32(cur0, gte); unpack32(cur1, up); }
					else { load32_edge(aux0, col0, gte); load32_edge(aux1, col0, up); }
					#pragma unroll
					for (int i = 0; i < 32; i++) {
						const float e = fast_exp(-gte[i]), ope = 1.0f + e, r = fast_rcp(ope);
						dup[i] = o[i] * (gte[i] * r);
						dgate[i] = o[i] * ((up[i] * (ope + gte[i] * e)) * (r * r));
					}
					store32(out, (size_t) ld_out, col0, dgate, whole, n_valid);
					store32(out, (size_t) ld_out, N + col0, dup, whole, n_valid);
				} else {
					store32(out, (size_t) ld_out, col0, o, whole, n_valid);
				}
			};
			#pragma unroll 1
			for (int c = c_first; c < c_end; c += 2) {
				chunk(c, pre0[0], pre1[0], pre0[1], pre1[1]);
				chunk(c + 1, pre0[1], pre1[1], pre0[0], pre1[0]);
			}
		}
		// A wait gave up (the status word says which): the tile it was for and every later tile of this walker get NaN, so that the
		// failure shows in the data and not only in the status word. Cold path: plain 2-byte stores.
		if (!ok) {
			const __nv_bfloat16 nan = __float2bfloat16_rn(__int_as_float(0x7fc00000));
			__nv_bfloat16 * o = reinterpret_cast<__nv_bfloat16 *>(out);
			for (; tile < num_tiles; tile += n_walkers) {
				int m0, n0;
				tile_origin(tile, m0, n0);
				const int row = m0 + quarter * 32 + lane;
				if (row >= M) continue;
				for (int j = col_half * (N_PER_TILE / 2); j < (col_half + 1) * (N_PER_TILE / 2) && n0 + j < N; j++) {
					o[(size_t) row * ld_out + n0 + j] = nan;
					if constexpr (MODE == MODE_SWIGLU_BWD) o[(size_t) row * ld_out + N + n0 + j] = nan;
				}
			}
		}
	}
	tc_fence_before_sync();
	// no CTA of a pair frees its tensor memory or leaves while the other may still use its shared or tensor memory
	if (PAIR) cluster_sync_all(); else __syncthreads();
	if (warp == 1) { tc_fence_after_sync(); if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
	static EncodeTiledFn fn = nullptr;
	if (!fn) {
		void * p = nullptr;
		cudaDriverEntryPointQueryResult q;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) { cudaGetLastError(); return nullptr; }
		fn = reinterpret_cast<EncodeTiledFn>(p);
	}
	return fn;
}

// Tensor map of a row-major [rows, k] e4m3 matrix, boxes of 128 rows x 128 bytes, 128-byte swizzle, zero fill outside.
static int make_map(CUtensorMap * map, const void * base, uint64_t rows, uint64_t k) {
	EncodeTiledFn fn = encode_tiled_fn();
	if (!fn) return set_error(DFB200_ERR_CUDA, "ffn_fp8: cuTensorMapEncodeTiled is not available");
	cuuint64_t dims[2] = {k, rows};
	cuuint64_t strides[1] = {k};
	cuuint32_t box[2] = {(cuuint32_t) GEMM_BK, (cuuint32_t) GEMM_BM};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
	                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) return set_error(DFB200_ERR_CUDA, "ffn_fp8: cuTensorMapEncodeTiled failed (%d)", (int) r);
	return DFB200_OK;
}

// DFB200_GEMM_SINGLE_CTA=1 in the environment keeps every GEMM on the one-CTA-per-tile kernel (for A/B measurements).
// Read on every launch (a getenv is nanoseconds beside a launch), so a test can switch forms inside one process.
static bool force_single_cta() {
	const char * e = getenv("DFB200_GEMM_SINGLE_CTA");
	return e && e[0] == '1';
}

// Clusters of two CTAs of the pair kernel that fit on the current device at once (0 when the query fails); remembered per device.
template <int MODE>
static int max_resident_pairs() {
	// plain host statics, not synchronised: two threads that race here both run the query and store the same value (the occupancy of
	// a kernel on a device does not change), so the worst case is one redundant query
	static int memo[64];
	static bool known[64];
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 0; }
	if (known[dev]) return memo[dev];
	auto kernel = gemm_e4m3_kernel<MODE, true>;
	allow_dyn_smem(reinterpret_cast<const void *>(kernel), GemmShape<true>::SMEM);
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(2 * sm_count(), 1, 1);
	cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
	cfg.dynamicSmemBytes = GemmShape<true>::SMEM;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
	cfg.attrs = attr; cfg.numAttrs = 1;
	int n = 0;
	if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
	memo[dev] = n; known[dev] = true;
	return n;
}

template <int MODE>
static int launch_gemm(int M, int N, int K, const void * A, const float * sa, const void * B0, const float * sb0, const void * B1, const float * sb1,
                       void * out, int ld_out, void * aux0, void * aux1, cudaStream_t stream) {
	constexpr bool SWIGLU = MODE == MODE_SWIGLU;
	if (K % 16 || N % 8 || !aligned16(A) || !aligned16(B0) || (SWIGLU && !aligned16(B1)) || !aligned16(out) || ld_out % 8 || !aligned16(aux0) || !aligned16(aux1))
		return set_error(DFB200_ERR_ARG, "ffn_fp8: K must be a multiple of 16, N of 8, tensors 16-byte aligned, output pitch a multiple of 8");
	if (!A || !sa || !B0 || !out || (SWIGLU && (!B1 || !sb0 || !sb1)) || (MODE == MODE_SWIGLU_BWD && (!aux0 || !aux1)) || (SWIGLU && !aux0 != !aux1))   // plain: aux0 = optional residual
		return set_error(DFB200_ERR_ARG, "ffn_fp8: NULL tensor argument");
	CUtensorMap ma, mb0, mb1;
	int rc = make_map(&ma, A, (uint64_t) M, (uint64_t) K);
	if (!rc) rc = make_map(&mb0, B0, (uint64_t) N, (uint64_t) K);
	if (!rc) rc = make_map(&mb1, SWIGLU ? B1 : B0, (uint64_t) N, (uint64_t) K);
	if (rc) return rc;
	unsigned int * status = kernel_status_word(STATUS_FFN);
	if (!status) return set_error(DFB200_ERR_CUDA, "ffn_fp8: no status word");
	constexpr int n_per_tile = SWIGLU ? GEMM_BN_HALF : 2 * GEMM_BN_HALF;
	const int tiles_n = (N + n_per_tile - 1) / n_per_tile;
	const float * sb1_arg = SWIGLU ? sb1 : sb0;
	// More than one 128-row tile: CTA pairs on 256 x 256 tiles, as many pairs as the device can hold at once.
	const int pairs = M > GEMM_BM && !force_single_cta() ? max_resident_pairs<MODE>() : 0;
	if (pairs > 0) {
		const int tiles_m = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
		auto kernel = gemm_e4m3_kernel<MODE, true>;
		allow_dyn_smem(reinterpret_cast<const void *>(kernel), GemmShape<true>::SMEM);     // per context; max_resident_pairs remembers per device
		cudaLaunchConfig_t cfg = {};
		const int n_pairs = tiles_m * tiles_n < pairs ? tiles_m * tiles_n : pairs;
		cfg.gridDim = dim3(2 * n_pairs, 1, 1);
		cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
		cfg.dynamicSmemBytes = GemmShape<true>::SMEM;
		cfg.stream = stream;
		cudaLaunchAttribute attr[1];
		attr[0].id = cudaLaunchAttributeClusterDimension;
		attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
		cfg.attrs = attr; cfg.numAttrs = 1;
		cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mb0, mb1, M, N, K, tiles_m, tiles_n, sa, sb0, sb1_arg, out, ld_out, aux0, aux1, status);
		if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "ffn_fp8 gemm (CTA pairs): %s", cudaGetErrorString(e)); }
		return DFB200_OK;
	}
	const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
	auto kernel = gemm_e4m3_kernel<MODE, false>;
	allow_dyn_smem(reinterpret_cast<const void *>(kernel), GemmShape<false>::SMEM);
	const int grid = tiles_m * tiles_n < sm_count() ? tiles_m * tiles_n : sm_count();      // persistent: one CTA per SM
	kernel<<<grid, GEMM_THREADS, GemmShape<false>::SMEM, stream>>>(ma, mb0, mb1, M, N, K, tiles_m, tiles_n, sa, sb0, sb1_arg, out, ld_out, aux0, aux1, status);
	return check_launch("ffn_fp8 gemm");
}

static uint64_t align256(uint64_t x) { return (x + 255) & ~255ull; }

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_quantize_rows_e4m3(int n_rows, int n_cols, const void * X_bf16, const float * col_factors, void * Q_e4m3, float * row_scales,
                                         void * stream) {
	if (n_rows < 0 || n_cols <= 0 || n_cols % 8) return set_error(DFB200_ERR_ARG, "quantize_rows_e4m3: bad shape %d x %d (columns must be a multiple of 8)", n_rows, n_cols);
	if (n_rows == 0) return DFB200_OK;
	if (!X_bf16 || !Q_e4m3 || !row_scales || !aligned16(X_bf16) || !aligned16(Q_e4m3)) return set_error(DFB200_ERR_ARG, "quantize_rows_e4m3: NULL or misaligned tensor");
	const int n_chunks = n_cols / 8;
	if (n_chunks > 1024 * 4) return set_error(DFB200_ERR_ARG, "quantize_rows_e4m3: n_cols = %d exceeds the supported maximum of %d", n_cols, 1024 * 4 * 8);
	if (col_factors && (reinterpret_cast<uintptr_t>(col_factors) & 15u)) return set_error(DFB200_ERR_ARG, "quantize_rows_e4m3: col_factors must be 16-byte aligned");
	// packets per thread: 2 once a row fills 256 threads with them (enough bytes in flight per thread), 4 above 1024 threads' worth
	int vpt = n_chunks >= 512 ? 2 : 1;
	while (vpt < 4 && (n_chunks + vpt - 1) / vpt > 1024) vpt *= 2;
	if (n_chunks > 2048) vpt = 4;
	const int threads = ((n_chunks + vpt - 1) / vpt + 31) / 32 * 32;
	cudaStream_t s = (cudaStream_t) stream;
#define DFB200_QUANT_CASE(V) \
	if (col_factors) quantize_rows_e4m3_kernel<V, true><<<n_rows, threads, 0, s>>>(n_rows, n_cols, X_bf16, col_factors, Q_e4m3, row_scales); \
	else quantize_rows_e4m3_kernel<V, false><<<n_rows, threads, 0, s>>>(n_rows, n_cols, X_bf16, col_factors, Q_e4m3, row_scales)
	switch (vpt) {
		case 1: DFB200_QUANT_CASE(1); break;
		case 2: DFB200_QUANT_CASE(2); break;
		default: DFB200_QUANT_CASE(4); break;
	}
#undef DFB200_QUANT_CASE
	return check_launch("quantize_rows_e4m3");
}

static int launch_swiglu_quantize(bool bwd, int n_rows, int f, const void * G, const void * U, const void * dH, const float * col_factors, void * Q,
                                  float * row_scales, void * bf16_out, void * stream) {
	const char * op = bwd ? "swiglu_bwd_quantize_rows_e4m3" : "swiglu_quantize_rows_e4m3";
	if (n_rows < 0 || f <= 0 || f % 8) return set_error(DFB200_ERR_ARG, "%s: bad shape %d x %d (columns must be a multiple of 8)", op, n_rows, f);
	if (n_rows == 0) return DFB200_OK;
	if (!G || !U || (bwd && !dH) || !Q || !row_scales || !aligned16(G) || !aligned16(U) || !aligned16(dH) || !aligned16(Q) || (f % 16 && bwd))
		return set_error(DFB200_ERR_ARG, "%s: NULL or misaligned tensor", op);
	if (col_factors && (reinterpret_cast<uintptr_t>(col_factors) & 15u)) return set_error(DFB200_ERR_ARG, "%s: col_factors must be 16-byte aligned", op);
	if (!aligned16(bf16_out)) return set_error(DFB200_ERR_ARG, "%s: the bf16 output must be 16-byte aligned", op);
	const int n_chunks = f / 8;
	if (n_chunks > 1024 * 4) return set_error(DFB200_ERR_ARG, "%s: f = %d exceeds the supported maximum of %d", op, f, 1024 * 4 * 8);
	int vpt = n_chunks >= 512 ? 2 : 1;
	if (n_chunks > 2048) vpt = 4;
	const int threads = ((n_chunks + vpt - 1) / vpt + 31) / 32 * 32;
	cudaStream_t s = (cudaStream_t) stream;
#define DFB200_SQ_CASE(V) \
	if (bwd && col_factors) swiglu_quantize_rows_kernel<V, true, true><<<n_rows, threads, 0, s>>>(n_rows, f, G, U, dH, col_factors, Q, row_scales, bf16_out); \
	else if (bwd) swiglu_quantize_rows_kernel<V, true, false><<<n_rows, threads, 0, s>>>(n_rows, f, G, U, dH, col_factors, Q, row_scales, bf16_out); \
	else swiglu_quantize_rows_kernel<V, false, false><<<n_rows, threads, 0, s>>>(n_rows, f, G, U, dH, col_factors, Q, row_scales, bf16_out)
	switch (vpt) {
		case 1: DFB200_SQ_CASE(1); break;
		case 2: DFB200_SQ_CASE(2); break;
		default: DFB200_SQ_CASE(4); break;
	}
#undef DFB200_SQ_CASE
	return check_launch(op);
}

extern "C" int dfb200_swiglu_quantize_rows_e4m3(int n_rows, int f, const void * gate_bf16, const void * up_bf16, void * Q_e4m3, float * row_scales,
                                                void * stream) {
	return launch_swiglu_quantize(false, n_rows, f, gate_bf16, up_bf16, nullptr, nullptr, Q_e4m3, row_scales, nullptr, stream);
}

extern "C" int dfb200_swiglu_bwd_quantize_rows_e4m3(int n_rows, int f, const void * gate_bf16, const void * up_bf16, const void * dH_bf16,
                                                    const float * col_factors, void * Q_e4m3, float * row_scales, void * dgate_dup_bf16, void * stream) {
	return launch_swiglu_quantize(true, n_rows, f, gate_bf16, up_bf16, dH_bf16, col_factors, Q_e4m3, row_scales, dgate_dup_bf16, stream);
}

extern "C" int dfb200_col_amax_bf16(int n_rows, int n_cols, const void * X_bf16, float * col_amax, void * stream) {
	if (n_rows <= 0 || n_cols <= 0 || n_cols % 8) return set_error(DFB200_ERR_ARG, "col_amax_bf16: bad shape %d x %d (columns must be a multiple of 8)", n_rows, n_cols);
	if (!X_bf16 || !col_amax || !aligned16(X_bf16) || (reinterpret_cast<uintptr_t>(col_amax) & 3u)) return set_error(DFB200_ERR_ARG, "col_amax_bf16: NULL or misaligned tensor");
	const int n_chunks = n_cols / 8;
	if (n_chunks > 1024 * 4) return set_error(DFB200_ERR_ARG, "col_amax_bf16: n_cols = %d exceeds the supported maximum of %d", n_cols, 1024 * 4 * 8);
	cudaStream_t s = (cudaStream_t) stream;
	cudaError_t e = cudaMemsetAsync(col_amax, 0, (size_t) n_cols * sizeof(float), s);
	if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "col_amax_bf16: %s", cudaGetErrorString(e)); }
	int vpt = 1;
	while (vpt < 4 && (n_chunks + vpt - 1) / vpt > 1024) vpt *= 2;
	const int group_threads = ((n_chunks + vpt - 1) / vpt + 31) / 32 * 32;
	int groups = 1024 / group_threads;
	if (groups < 1) groups = 1;
	int grid = sm_count();
	if ((long long) grid * groups > n_rows) grid = (n_rows + groups - 1) / groups;
	const size_t smem = (size_t) n_cols * sizeof(unsigned int);
	switch (vpt) {
		case 1: allow_dyn_smem(reinterpret_cast<const void *>(col_amax_kernel<1>), smem);
		        col_amax_kernel<1><<<grid, groups * group_threads, smem, s>>>(n_rows, n_cols, group_threads, X_bf16, col_amax); break;
		case 2: allow_dyn_smem(reinterpret_cast<const void *>(col_amax_kernel<2>), smem);
		        col_amax_kernel<2><<<grid, groups * group_threads, smem, s>>>(n_rows, n_cols, group_threads, X_bf16, col_amax); break;
		default: allow_dyn_smem(reinterpret_cast<const void *>(col_amax_kernel<4>), smem);
		        col_amax_kernel<4><<<grid, groups * group_threads, smem, s>>>(n_rows, n_cols, group_threads, X_bf16, col_amax); break;
	}
	return check_launch("col_amax_bf16");
}

extern "C" int dfb200_transpose_quantize_e4m3(int n_rows, int n_cols, const void * X_bf16, const float * col_amax, void * Qt_e4m3, float * col_scales,
                                              void * stream) {
	if (n_rows <= 0 || n_cols <= 0 || n_cols % 8 || n_rows % 16)
		return set_error(DFB200_ERR_ARG, "transpose_quantize_e4m3: bad shape %d x %d (rows a multiple of 16, columns of 8)", n_rows, n_cols);
	if (!X_bf16 || !col_amax || !Qt_e4m3 || !col_scales || !aligned16(X_bf16) || !aligned16(Qt_e4m3))
		return set_error(DFB200_ERR_ARG, "transpose_quantize_e4m3: NULL or misaligned tensor");
	dim3 grid((n_cols + TQ_COLS - 1) / TQ_COLS, (n_rows + TQ_TOKENS - 1) / TQ_TOKENS);
	if (grid.y > 65535) return set_error(DFB200_ERR_ARG, "transpose_quantize_e4m3: too many rows");
	transpose_quantize_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(n_rows, n_cols, X_bf16, col_amax, static_cast<uint8_t *>(Qt_e4m3), col_scales);
	return check_launch("transpose_quantize_e4m3");
}

extern "C" int dfb200_transpose_bytes(int rows, int cols, const void * in, int ld_in, void * out, int ld_out, void * stream) {
	if (rows <= 0 || cols <= 0 || !in || !out || ld_in < cols || ld_out < rows) return set_error(DFB200_ERR_ARG, "transpose_bytes: bad arguments");
	dim3 grid((cols + 31) / 32, (rows + 31) / 32);
	transpose_bytes_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(rows, cols, static_cast<const uint8_t *>(in), ld_in, static_cast<uint8_t *>(out), ld_out);
	return check_launch("transpose_bytes");
}

extern "C" int dfb200_gemm_e4m3_swiglu(int M, int N, int K, const void * A_e4m3, const float * a_row_scales, const void * Wgate_e4m3, const float * gate_scales,
                                       const void * Wup_e4m3, const float * up_scales, void * H_bf16, void * gate_save_bf16, void * up_save_bf16, void * stream) {
	if (M <= 0 || N <= 0 || K <= 0) return set_error(DFB200_ERR_ARG, "gemm_e4m3_swiglu: bad shape");
	return launch_gemm<MODE_SWIGLU>(M, N, K, A_e4m3, a_row_scales, Wgate_e4m3, gate_scales, Wup_e4m3, up_scales, H_bf16, N, gate_save_bf16, up_save_bf16,
	                                (cudaStream_t) stream);
}

extern "C" int dfb200_gemm_e4m3(int M, int N, int K, const void * A_e4m3, const float * a_row_scales, const void * W_e4m3, const float * w_scales,
                                const void * residual_bf16, void * out_bf16, void * stream) {
	if (M <= 0 || N <= 0 || K <= 0) return set_error(DFB200_ERR_ARG, "gemm_e4m3: bad shape");
	return launch_gemm<MODE_PLAIN>(M, N, K, A_e4m3, a_row_scales, W_e4m3, w_scales, nullptr, nullptr, out_bf16, N, const_cast<void *>(residual_bf16), nullptr,
	                               (cudaStream_t) stream);
}

extern "C" int dfb200_gemm_e4m3_swiglu_bwd(int M, int N, int K, const void * dOut_e4m3, const float * dout_row_scales, const void * WdownT_e4m3,
                                           const void * gate_saved_bf16, const void * up_saved_bf16, void * dgate_dup_bf16, void * stream) {
	if (M <= 0 || N <= 0 || K <= 0) return set_error(DFB200_ERR_ARG, "gemm_e4m3_swiglu_bwd: bad shape");
	return launch_gemm<MODE_SWIGLU_BWD>(M, N, K, dOut_e4m3, dout_row_scales, WdownT_e4m3, nullptr, nullptr, nullptr, dgate_dup_bf16, 2 * N,
	                                    const_cast<void *>(gate_saved_bf16), const_cast<void *>(up_saved_bf16), (cudaStream_t) stream);
}

// Forward:  Aq, sa = quantise_rows(A);  g = (Aq Wgate^T) sa sg;  u = (Aq Wup^T) sa su   (two GEMMs, bf16 [T, f] each: exactly what the
// backward pass needs saved);  Hq, sh = quantise_rows( bf16(silu(g) u) )  (one fused row pass, H itself is never stored);
// out = bf16( (Hq Wdown^T) sh sd + residual ).
extern "C" uint64_t dfb200_swiglu_ffn_fp8_workspace_bytes(int T, int d, int f) {
	// forward: quantised input [T, d] + scales, g and u [T, f] bf16 (used when the caller does not ask for them), quantised hidden [T, f] + scales
	// backward: quantised dOut [T, d] + scales, dH [T, f] bf16, quantised gate|up gradients [T, 2f] + scales
	const uint64_t fwd = align256((uint64_t) T * d) + align256((uint64_t) T * 4) + 2 * align256((uint64_t) T * f * 2) + align256((uint64_t) T * f) + align256((uint64_t) T * 4);
	const uint64_t bwd = align256((uint64_t) T * d) + align256((uint64_t) T * 4) + align256((uint64_t) T * f * 2) + align256((uint64_t) T * f * 2) + align256((uint64_t) T * 4);
	return fwd > bwd ? fwd : bwd;
}

extern "C" int dfb200_swiglu_ffn_fp8(int T, int d, int f, const void * A_bf16, const void * Wgate, const float * gate_scales, const void * Wup,
                                     const float * up_scales, const void * Wdown, const float * down_scales, const void * residual_bf16, void * out_bf16,
                                     void * gate_save_bf16, void * up_save_bf16, void * workspace, uint64_t workspace_bytes, void * stream) {
	if (T <= 0 || d <= 0 || f <= 0 || d % 16 || f % 16) return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8: bad shape (T %d, d %d, f %d; d and f multiples of 16)", T, d, f);
	if (!gate_save_bf16 != !up_save_bf16) return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8: gate_save and up_save are given together or not at all");
	const uint64_t need = dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "swiglu_ffn_fp8: needs %llu bytes of 16-byte aligned workspace, got %llu", (unsigned long long) need, (unsigned long long) workspace_bytes);
	uint8_t * p = static_cast<uint8_t *>(workspace);
	auto take = [&](uint64_t bytes) { uint8_t * q = p; p += align256(bytes); return q; };
	void * Aq = take((uint64_t) T * d);
	float * sa = reinterpret_cast<float *>(take((uint64_t) T * 4));
	void * G = take((uint64_t) T * f * 2);
	void * U = take((uint64_t) T * f * 2);
	void * Hq = take((uint64_t) T * f);
	float * sh = reinterpret_cast<float *>(take((uint64_t) T * 4));
	if (gate_save_bf16) { G = gate_save_bf16; U = up_save_bf16; }
	int rc = dfb200_quantize_rows_e4m3(T, d, A_bf16, nullptr, Aq, sa, stream);
	if (!rc) rc = dfb200_gemm_e4m3(T, f, d, Aq, sa, Wgate, gate_scales, nullptr, G, stream);
	if (!rc) rc = dfb200_gemm_e4m3(T, f, d, Aq, sa, Wup, up_scales, nullptr, U, stream);
	if (!rc) rc = dfb200_swiglu_quantize_rows_e4m3(T, f, G, U, Hq, sh, stream);
	if (!rc) rc = dfb200_gemm_e4m3(T, d, f, Hq, sh, Wdown, down_scales, residual_bf16, out_bf16, stream);
	return rc;
}

// Backward weights: the gradient GEMMs contract over the OUTPUT channels of the forward weights, so they need the codes
// transposed: WdownT [f, d] = Wdown^T, and WgateupT [d, 2f] = [Wgate^T | Wup^T] side by side (one GEMM with K = 2f gives
// dA = dG Wg + dU Wu). The per-output-channel scales then sit on the contraction index; they are folded into the
// activation gradients before those are quantised (column factors of dfb200_quantize_rows_e4m3).
extern "C" int dfb200_ffn_fp8_prepare_bwd_weights(int d, int f, const void * Wgate, const void * Wup, const void * Wdown, void * WgateupT, void * WdownT,
                                                  void * stream) {
	if (d <= 0 || f <= 0 || d % 16 || f % 16) return set_error(DFB200_ERR_ARG, "ffn_fp8_prepare_bwd_weights: bad shape");
	int rc = dfb200_transpose_bytes(f, d, Wgate, d, WgateupT, 2 * f, stream);                                   // [f, d] -> [d, f] into columns [0, f)
	if (!rc) rc = dfb200_transpose_bytes(f, d, Wup, d, static_cast<uint8_t *>(WgateupT) + f, 2 * f, stream);     // columns [f, 2f)
	if (!rc) rc = dfb200_transpose_bytes(d, f, Wdown, f, WdownT, d, stream);                                     // [d, f] -> [f, d]
	return rc;
}

// dA = d(loss)/d(input) of the FFN, given dOut and the pre-activations saved by the forward pass:
//   dOq, s1     = quantise_rows(dOut * down_scales[col])                         (scale of the contraction index folded in)
//   dH          = bf16( (dOq WdownT^T) * s1 )                                    [T, f]
//   dGUq, s2    = quantise_rows( swiglu_bwd_x(g, u, dH) * [gate_scales | up_scales] )   one fused row pass, [T, 2f] codes
//   dA          = bf16( (dGUq WgateupT^T) * s2 )                                 [T, d]
// gateup_scales is the concatenation [gate_scales | up_scales] (2f floats, 16-byte aligned). Weight gradients are not computed here.
extern "C" int dfb200_swiglu_ffn_fp8_bwd(int T, int d, int f, const void * dOut_bf16, const void * gate_saved_bf16, const void * up_saved_bf16,
                                         const void * WdownT, const float * down_scales, const void * WgateupT, const float * gateup_scales,
                                         void * dA_bf16, void * dgate_dup_bf16, void * workspace, uint64_t workspace_bytes, void * stream) {
	if (T <= 0 || d <= 0 || f <= 0 || d % 16 || f % 16) return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8_bwd: bad shape (T %d, d %d, f %d; d and f multiples of 16)", T, d, f);
	const uint64_t need = dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "swiglu_ffn_fp8_bwd: needs %llu bytes of 16-byte aligned workspace, got %llu", (unsigned long long) need, (unsigned long long) workspace_bytes);
	uint8_t * p = static_cast<uint8_t *>(workspace);
	auto take = [&](uint64_t bytes) { uint8_t * q = p; p += align256(bytes); return q; };
	void * dOq = take((uint64_t) T * d);
	float * s1 = reinterpret_cast<float *>(take((uint64_t) T * 4));
	void * dH = take((uint64_t) T * f * 2);
	void * dGUq = take((uint64_t) T * f * 2);
	float * s2 = reinterpret_cast<float *>(take((uint64_t) T * 4));
	int rc = dfb200_quantize_rows_e4m3(T, d, dOut_bf16, down_scales, dOq, s1, stream);
	if (!rc) rc = dfb200_gemm_e4m3(T, f, d, dOq, s1, WdownT, nullptr, nullptr, dH, stream);
	if (!rc) rc = dfb200_swiglu_bwd_quantize_rows_e4m3(T, f, gate_saved_bf16, up_saved_bf16, dH, gateup_scales, dGUq, s2, dgate_dup_bf16, stream);
	if (!rc) rc = dfb200_gemm_e4m3(T, d, 2 * f, dGUq, s2, WgateupT, nullptr, nullptr, dA_bf16, stream);
	return rc;
}

// Weight gradients of the FFN (bf16), from the forward input A, the output gradient, the saved pre-activations and the gate|up
// gradients [T, 2f] that dfb200_swiglu_ffn_fp8_bwd stores on request:
//   dWdown[d, f] = dOut^T H,  H = bf16(silu(g) u);   dWgate[f, d] = dG^T A;   dWup[f, d] = dU^T A
// Each operand is transposed and quantised to e4m3 with one scale per row of the transpose (col_amax + transpose_quantize), so the
// three GEMMs (reduction over the T tokens) are the plain kernel with both scales on output indices.
extern "C" uint64_t dfb200_swiglu_ffn_fp8_wgrad_workspace_bytes(int T, int d, int f) {
	return align256((uint64_t) T * f * 2)                                              // H bf16
	     + 2 * align256((uint64_t) T * d) + align256((uint64_t) T * f) + align256((uint64_t) T * f * 2)   // dOut^T, A^T, H^T, [dG | dU]^T codes
	     + 2 * (2 * align256((uint64_t) d * 4) + align256((uint64_t) f * 4) + align256((uint64_t) f * 8));   // column maxima and scales of the four
}

extern "C" int dfb200_swiglu_ffn_fp8_wgrad(int T, int d, int f, const void * A_bf16, const void * dOut_bf16, const void * gate_saved_bf16,
                                           const void * up_saved_bf16, const void * dgate_dup_bf16, void * dWgate_bf16, void * dWup_bf16,
                                           void * dWdown_bf16, void * workspace, uint64_t workspace_bytes, void * stream) {
	if (T <= 0 || d <= 0 || f <= 0 || d % 16 || f % 16 || T % 16)
		return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8_wgrad: bad shape (T %d, d %d, f %d; all multiples of 16)", T, d, f);
	if (!A_bf16 || !dOut_bf16 || !gate_saved_bf16 || !up_saved_bf16 || !dgate_dup_bf16 || !dWgate_bf16 || !dWup_bf16 || !dWdown_bf16)
		return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8_wgrad: NULL tensor argument");
	const uint64_t need = dfb200_swiglu_ffn_fp8_wgrad_workspace_bytes(T, d, f);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "swiglu_ffn_fp8_wgrad: needs %llu bytes of 16-byte aligned workspace, got %llu", (unsigned long long) need, (unsigned long long) workspace_bytes);
	uint8_t * p = static_cast<uint8_t *>(workspace);
	auto take = [&](uint64_t bytes) { uint8_t * q = p; p += align256(bytes); return q; };
	void * H = take((uint64_t) T * f * 2);
	void * dOt = take((uint64_t) T * d);  void * At = take((uint64_t) T * d);  void * Ht = take((uint64_t) T * f);  uint8_t * dGUt = take((uint64_t) T * f * 2);
	float * m_do = reinterpret_cast<float *>(take((uint64_t) d * 4)), * s_do = reinterpret_cast<float *>(take((uint64_t) d * 4));
	float * m_a = reinterpret_cast<float *>(take((uint64_t) d * 4)),  * s_a = reinterpret_cast<float *>(take((uint64_t) d * 4));
	float * m_h = reinterpret_cast<float *>(take((uint64_t) f * 4)),  * s_h = reinterpret_cast<float *>(take((uint64_t) f * 4));
	float * m_gu = reinterpret_cast<float *>(take((uint64_t) f * 8)), * s_gu = reinterpret_cast<float *>(take((uint64_t) f * 8));
	int rc = dfb200_swiglu(DATAFLOW_BF16, T, f, gate_saved_bf16, up_saved_bf16, H, stream);
	auto transposed = [&](int cols, const void * X, float * m, void * Qt, float * sc) {
		if (!rc) rc = dfb200_col_amax_bf16(T, cols, X, m, stream);
		if (!rc) rc = dfb200_transpose_quantize_e4m3(T, cols, X, m, Qt, sc, stream);
	};
	transposed(d, dOut_bf16, m_do, dOt, s_do);
	transposed(d, A_bf16, m_a, At, s_a);
	transposed(f, H, m_h, Ht, s_h);
	transposed(2 * f, dgate_dup_bf16, m_gu, dGUt, s_gu);
	if (!rc) rc = dfb200_gemm_e4m3(d, f, T, dOt, s_do, Ht, s_h, nullptr, dWdown_bf16, stream);
	if (!rc) rc = dfb200_gemm_e4m3(f, d, T, dGUt, s_gu, At, s_a, nullptr, dWgate_bf16, stream);
	if (!rc) rc = dfb200_gemm_e4m3(f, d, T, dGUt + (uint64_t) f * T, s_gu + f, At, s_a, nullptr, dWup_bf16, stream);
	return rc;
}
