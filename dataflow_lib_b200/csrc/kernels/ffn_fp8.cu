// FP8-weight SwiGLU FFN forward on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
//   H   = silu(A Wg^T * sa sg) * (A Wu^T * sa su)        [T, f]  bf16
//   Out = (H Wd^T) * sh sd                                [T, d]  bf16
//
// Weights are e4m3 with one fp32 scale per OUTPUT channel and are stored [out_features, in_features] (reduction
// dimension contiguous). tcgen05.mma kind::f8f6f4 needs both operands in 8 bits, so activations are quantised to e4m3
// with one fp32 scale per ROW (token) by quantize_rows_e4m3_kernel; both scales leave the contraction and are applied
// to the fp32 accumulator in the epilogue. The reference has no such op (its only GEMM is a cuBLASLt call without
// scale pointers, src/ops/nvidia/external/matmul_helper/src/matmul_helper.c:379-416); the arithmetic contract is the
// one restated by the CPU oracle (oracle_ffn_fp8_*).
//
// GEMM kernel: persistent CTAs (one per SM) walk 128 x 256 accumulator tiles; two accumulator stages in tensor memory
// (2 x 256 of the 512 columns) let the epilogue of one tile overlap the MMAs of the next. Warp-specialised:
//   warp 0      one thread issues TMA tile loads (cp.async.bulk.tensor, 128-byte swizzle, CTA-local destination)
//               into a 4-stage shared-memory ring (A 128x128 B + B 256x128 B per stage), completion on mbarriers;
//   warp 1      allocates the tensor memory; one thread issues tcgen05.mma (M128 N256 K32, fp32
//               accumulation in TMEM) and tcgen05.commit, which releases ring stages and finally signals the epilogue;
//   warps 2-5   read the accumulator with tcgen05.ld (each warp its 32-lane quarter), apply the scales (and SwiGLU
//               for the gate/up pair, whose two 128-column halves are the gate and the up projection of the same 128
//               output channels), convert to bf16 and store.
// Every mbarrier wait is bounded and reports through the kernel status word.
#include "common.cuh"
#include "tma.cuh"

#include <cuda.h>

namespace dfb200 {

constexpr int GEMM_BM = 128, GEMM_BK = 128;            // BK in elements = bytes (e4m3)
constexpr int GEMM_BN_HALF = 128;                        // columns per accumulator half
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;                      // two 256-column accumulator stages
constexpr uint32_t A_STAGE_BYTES = GEMM_BM * GEMM_BK;                   // 16 KB
constexpr uint32_t B_STAGE_BYTES = 2 * GEMM_BN_HALF * GEMM_BK;          // 32 KB
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;

// ---------------------------------------------------------------------------------------------------------------
// PTX wrappers (tensor-map TMA, tcgen05)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void * smem_dst, const CUtensorMap * map, int x, int y, uint64_t * bar) {
	asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
	             :: "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
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
template <int VPT>
__global__ void __launch_bounds__(512)
quantize_rows_e4m3_kernel(int n_rows, int n_cols, const void * __restrict__ X, const float * __restrict__ col_mult, void * __restrict__ Q,
                          float * __restrict__ scales) {
	__shared__ float red[16];
	const int n_chunks = n_cols / 8, tid = threadIdx.x, nthr = blockDim.x;
	float mult[VPT][8];                               // optional per-column factor applied before quantisation (1 when absent)
	#pragma unroll
	for (int v = 0; v < VPT; v++) {
		const int c = tid + v * nthr;
		#pragma unroll
		for (int i = 0; i < 8; i++) mult[v][i] = (col_mult && c < n_chunks) ? __ldg(col_mult + c * 8 + i) : 1.0f;
	}
	for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
		float x[VPT][8];
		float amax = 0.0f;
		#pragma unroll
		for (int v = 0; v < VPT; v++) {
			const int c = tid + v * nthr;
			if (c < n_chunks) {
				load_elems<bf16_t, 8>(X, (uint64_t) row * n_cols + (uint64_t) c * 8, x[v]);
				#pragma unroll
				for (int i = 0; i < 8; i++) { x[v][i] = __fmul_rn(x[v][i], mult[v][i]); amax = fmaxf(amax, fabsf(x[v][i])); }
			}
		}
		amax = warp_max(amax);
		__syncthreads();                               // red[] of the previous row has been read
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
				float q[8];
				#pragma unroll
				for (int i = 0; i < 8; i++) q[i] = __fmul_rn(x[v][i], inv);
				store_elems<e4m3_t, 8>(Q, (uint64_t) row * n_cols + (uint64_t) c * 8, q);
			}
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
template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_e4m3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1,
                 int M, int N, int K, int tiles_m, int tiles_n, const float * __restrict__ sa, const float * __restrict__ sb0,
                 const float * __restrict__ sb1, void * out, int ld_out, void * aux0, void * aux1, unsigned int * status) {
	constexpr bool SWIGLU = MODE == MODE_SWIGLU;
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
		m0 = (g * group + r % rows_in_group) * GEMM_BM;
		n0 = (r / rows_in_group) * N_PER_TILE;
	};

	if (threadIdx.x == 0) {
		for (int s = 0; s < GEMM_STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
		for (int a = 0; a < 2; a++) { mbar_init(&accum_full[a], 1); mbar_init(&accum_empty[a], 4); }      // 4 epilogue warps release an accumulator
		mbar_fence_init();
		prefetch_tensormap(&map_a); prefetch_tensormap(&map_b0); prefetch_tensormap(&map_b1);
	}
	if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
	tc_fence_before_sync();
	__syncthreads();
	tc_fence_after_sync();
	const uint32_t tmem_base = *tmem_slot;

	if (warp == 0) {
		// ---------------- TMA producer: one stream of k-blocks across all of this CTA's tiles
		if (lane == 0) {
			uint32_t it = 0;
			bool ok = true;
			for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
				int m0, n0;
				tile_origin(tile, m0, n0);
				for (int kb = 0; kb < num_kb; kb++, it++) {
					const int s = it % GEMM_STAGES;
					ok = mbar_wait_bounded(&empty[s], ((it / GEMM_STAGES) & 1) ^ 1, status, 0x300u + s);
					if (!ok) break;
					uint8_t * a_dst = ring + (size_t) s * STAGE_BYTES;
					uint8_t * b_dst = a_dst + A_STAGE_BYTES;
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
		if (lane == 0) {
			constexpr uint32_t idesc = umma_idesc_e4m3(GEMM_BM, 2 * GEMM_BN_HALF);
			uint32_t it = 0, local = 0;
			bool ok = true;
			for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
				const uint32_t acc_stage = local & 1;
				ok = mbar_wait_bounded(&accum_empty[acc_stage], ((local >> 1) & 1) ^ 1, status, 0x330u + acc_stage);
				if (!ok) break;
				tc_fence_after_sync();
				const uint32_t d_tmem = tmem_base + acc_stage * (2 * GEMM_BN_HALF);
				for (int kb = 0; kb < num_kb; kb++, it++) {
					const int s = it % GEMM_STAGES;
					ok = mbar_wait_bounded(&full[s], (it / GEMM_STAGES) & 1, status, 0x310u + s);
					if (!ok) break;
					tc_fence_after_sync();
					const uint8_t * a_tile = ring + (size_t) s * STAGE_BYTES;
					// The two 128-row B halves are adjacent in shared memory and form one 256-row K-major tile, so a single
					// M128 x N256 x K32 instruction (the largest 1-CTA shape) fills both accumulator halves.
					const uint64_t da = umma_desc_k_sw128(a_tile);
					const uint64_t db = umma_desc_k_sw128(a_tile + A_STAGE_BYTES);
					#pragma unroll
					for (int j = 0; j < GEMM_BK / 32; j++)            // K = 32 per instruction: advance 32 bytes inside the swizzle atom
						tc_mma_f8(d_tmem, da + 2 * j, db + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
					tc_commit(&empty[s]);                               // stage reusable once these MMAs have read it
				}
				tc_commit(&accum_full[acc_stage]);                       // accumulator complete (or abandoned) -> epilogue
			}
		}
	} else {
		// ---------------- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 32
		const int quarter = warp & 3;
		const int etid = threadIdx.x - 64;                   // 0..127 among the epilogue threads
		uint32_t local = 0;
		bool ok = true;
		for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
			const uint32_t acc_stage = local & 1;
			int m0, n0;
			tile_origin(tile, m0, n0);
			float * scale = s_scale + acc_stage * (2 * GEMM_BN_HALF);
			for (int j = etid; j < 2 * GEMM_BN_HALF; j += 128) {         // column scales of this tile (buffer last read two tiles ago)
				const int half = j / GEMM_BN_HALF, col = SWIGLU ? n0 + (j % GEMM_BN_HALF) : n0 + j;
				const float * sb = (SWIGLU && half == 1) ? sb1 : sb0;
				scale[j] = col < N ? (sb ? __ldg(sb + col) : 1.0f) : 0.0f;
			}
			const int row = m0 + quarter * 32 + lane;
			const float a_scale = row < M ? __ldg(sa + row) : 0.0f;
			const bool mine = mbar_wait_bounded(&accum_full[acc_stage], (local >> 1) & 1, status, 0x320u + acc_stage);
			// One named barrier over the 128 epilogue threads does two jobs: it publishes the scales, and it ANDs the
			// outcome of the wait so that all four warps take the same branch (tcgen05.ld and the barrier are collective).
			uint32_t all_ok;
			asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
			             : "=r"(all_ok) : "r"((uint32_t) mine) : "memory");
			ok = all_ok != 0;
			tc_fence_after_sync();
			if (!ok) break;
			const uint32_t taddr = tmem_base + acc_stage * (2 * GEMM_BN_HALF) + ((uint32_t) (quarter * 32) << 16);
			__nv_bfloat16 * out_row = reinterpret_cast<__nv_bfloat16 *>(out) + (size_t) row * ld_out;
			auto store32 = [&](__nv_bfloat16 * dst_row, int col0, const float (&val)[32], int n_limit) {
				if (col0 + 32 <= n_limit) {
					#pragma unroll
					for (int i = 0; i < 32; i += 8) {
						uint32_t w[4];
						#pragma unroll
						for (int k = 0; k < 4; k++) w[k] = Word<bf16_t>::pack(&val[i + 2 * k]);
						*reinterpret_cast<uint4 *>(dst_row + col0 + i) = make_uint4(w[0], w[1], w[2], w[3]);
					}
				} else {
					for (int i = 0; i < 32 && col0 + i < n_limit; i++) dst_row[col0 + i] = __float2bfloat16_rn(val[i]);
				}
			};
			auto load32 = [&](const __nv_bfloat16 * src_row, int col0, float (&val)[32], int n_limit) {
				if (col0 + 32 <= n_limit) {
					#pragma unroll
					for (int i = 0; i < 32; i += 8) {
						const uint4 w = *reinterpret_cast<const uint4 *>(src_row + col0 + i);
						Word<bf16_t>::unpack(w.x, &val[i]); Word<bf16_t>::unpack(w.y, &val[i + 2]);
						Word<bf16_t>::unpack(w.z, &val[i + 4]); Word<bf16_t>::unpack(w.w, &val[i + 6]);
					}
				} else {
					for (int i = 0; i < 32; i++) val[i] = col0 + i < n_limit ? __bfloat162float(src_row[col0 + i]) : 0.0f;
				}
			};
			#pragma unroll 1
			for (int c = 0; c < N_PER_TILE / 32; c++) {
				float v0[32], o[32];
				const int col0 = n0 + c * 32;
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
					if (row < M && aux0) {
						store32(reinterpret_cast<__nv_bfloat16 *>(aux0) + (size_t) row * N, col0, v0, N);
						store32(reinterpret_cast<__nv_bfloat16 *>(aux1) + (size_t) row * N, col0, v1, N);
					}
				} else {
					tmem_ld_32cols(taddr + c * 32, v0);
					#pragma unroll
					for (int i = 0; i < 32; i++) o[i] = (v0[i] * a_scale) * scale[c * 32 + i];
					if (MODE == MODE_PLAIN && aux0 && row < M) {          // residual: out = bf16( acc * scales + residual )
						float res[32];
						load32(reinterpret_cast<const __nv_bfloat16 *>(aux0) + (size_t) row * N, col0, res, N);
						#pragma unroll
						for (int i = 0; i < 32; i++) o[i] += res[i];
					}
				}
				if (c == N_PER_TILE / 32 - 1) {                  // last read of this accumulator: hand it back to the MMA warp
					tc_fence_before_sync();
					__syncwarp();
					if (lane == 0) mbar_arrive(&accum_empty[acc_stage]);
				}
				if (row < M) {
					if constexpr (MODE == MODE_SWIGLU_BWD) {
						// o = dL/dh; saved pre-activations give the gate and up gradients (same expressions as swiglu_bwd_x)
						float gte[32], up[32], dgate[32], dup[32];
						load32(reinterpret_cast<const __nv_bfloat16 *>(aux0) + (size_t) row * N, col0, gte, N);
						load32(reinterpret_cast<const __nv_bfloat16 *>(aux1) + (size_t) row * N, col0, up, N);
						#pragma unroll
						for (int i = 0; i < 32; i++) {
							const float e = fast_exp(-gte[i]), ope = 1.0f + e, r = fast_rcp(ope);
							dup[i] = o[i] * (gte[i] * r);
							dgate[i] = o[i] * ((up[i] * (ope + gte[i] * e)) * (r * r));
						}
						store32(out_row, col0, dgate, N);
						store32(out_row + N, col0, dup, N);
					} else {
						store32(out_row, col0, o, N);
					}
				}
			}
		}
	}
	tc_fence_before_sync();
	__syncthreads();
	if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, TMEM_COLS); }
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
	const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM, tiles_n = (N + n_per_tile - 1) / n_per_tile;
	const size_t smem = 1024 + GEMM_STAGES * STAGE_BYTES + (2 * GEMM_STAGES + 4) * sizeof(uint64_t) + 2 * sizeof(uint32_t) + 4 * GEMM_BN_HALF * sizeof(float);
	auto kernel = gemm_e4m3_kernel<MODE>;
	allow_dyn_smem(reinterpret_cast<const void *>(kernel), smem);
	const int grid = tiles_m * tiles_n < sm_count() ? tiles_m * tiles_n : sm_count();      // persistent: one CTA per SM
	kernel<<<grid, GEMM_THREADS, smem, stream>>>(ma, mb0, mb1, M, N, K, tiles_m, tiles_n, sa, sb0, SWIGLU ? sb1 : sb0, out, ld_out, aux0, aux1, status);
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
	if (n_chunks > 512 * 8) return set_error(DFB200_ERR_ARG, "quantize_rows_e4m3: n_cols = %d exceeds the supported maximum of %d", n_cols, 512 * 8 * 8);
	int vpt = 1;
	while (vpt < 8 && (n_chunks + vpt - 1) / vpt > 256) vpt *= 2;
	int threads = ((n_chunks + vpt - 1) / vpt + 31) / 32 * 32;       // <= 256 unless the row needs 8 packets per thread at 512 threads
	const int grid = n_rows < sm_count() * 4 ? n_rows : sm_count() * 4;
	cudaStream_t s = (cudaStream_t) stream;
	switch (vpt) {
		case 1: quantize_rows_e4m3_kernel<1><<<grid, threads, 0, s>>>(n_rows, n_cols, X_bf16, col_factors, Q_e4m3, row_scales); break;
		case 2: quantize_rows_e4m3_kernel<2><<<grid, threads, 0, s>>>(n_rows, n_cols, X_bf16, col_factors, Q_e4m3, row_scales); break;
		case 4: quantize_rows_e4m3_kernel<4><<<grid, threads, 0, s>>>(n_rows, n_cols, X_bf16, col_factors, Q_e4m3, row_scales); break;
		default: quantize_rows_e4m3_kernel<8><<<grid, threads, 0, s>>>(n_rows, n_cols, X_bf16, col_factors, Q_e4m3, row_scales); break;
	}
	return check_launch("quantize_rows_e4m3");
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

extern "C" uint64_t dfb200_swiglu_ffn_fp8_workspace_bytes(int T, int d, int f) {
	// forward: quantised input [T, d] + scales, hidden [T, f] bf16, quantised hidden [T, f] + scales
	// backward: quantised dOut [T, d] + scales, gate|up gradients [T, 2f] bf16, their quantised form [T, 2f] + scales (larger: it is the bound)
	const uint64_t fwd = align256((uint64_t) T * d) + align256((uint64_t) T * 4) + align256((uint64_t) T * f * 2) + align256((uint64_t) T * f) + align256((uint64_t) T * 4);
	const uint64_t bwd = align256((uint64_t) T * d) + align256((uint64_t) T * 4) + align256((uint64_t) T * f * 4) + align256((uint64_t) T * f * 2) + align256((uint64_t) T * 4);
	return fwd > bwd ? fwd : bwd;
}

extern "C" int dfb200_swiglu_ffn_fp8(int T, int d, int f, const void * A_bf16, const void * Wgate, const float * gate_scales, const void * Wup,
                                     const float * up_scales, const void * Wdown, const float * down_scales, const void * residual_bf16, void * out_bf16,
                                     void * gate_save_bf16, void * up_save_bf16, void * workspace, uint64_t workspace_bytes, void * stream) {
	if (T <= 0 || d <= 0 || f <= 0 || d % 16 || f % 16) return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8: bad shape (T %d, d %d, f %d; d and f multiples of 16)", T, d, f);
	const uint64_t need = dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "swiglu_ffn_fp8: needs %llu bytes of 16-byte aligned workspace, got %llu", (unsigned long long) need, (unsigned long long) workspace_bytes);
	uint8_t * p = static_cast<uint8_t *>(workspace);
	auto take = [&](uint64_t bytes) { uint8_t * q = p; p += align256(bytes); return q; };
	void * Aq = take((uint64_t) T * d);
	float * sa = reinterpret_cast<float *>(take((uint64_t) T * 4));
	void * H = take((uint64_t) T * f * 2);
	void * Hq = take((uint64_t) T * f);
	float * sh = reinterpret_cast<float *>(take((uint64_t) T * 4));
	int rc = dfb200_quantize_rows_e4m3(T, d, A_bf16, nullptr, Aq, sa, stream);
	if (!rc) rc = dfb200_gemm_e4m3_swiglu(T, f, d, Aq, sa, Wgate, gate_scales, Wup, up_scales, H, gate_save_bf16, up_save_bf16, stream);
	if (!rc) rc = dfb200_quantize_rows_e4m3(T, f, H, nullptr, Hq, sh, stream);
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
//   dH          = (dOq WdownT^T) * s1                                            [T, f]   never stored
//   dG | dU     = swiglu backward of dH with the saved gate / up pre-activations  [T, 2f] bf16
//   dGUq, s2    = quantise_rows([dG | dU] * [gate_scales | up_scales])
//   dA          = bf16( (dGUq WgateupT^T) * s2 )                                 [T, d]
// gateup_scales is the concatenation [gate_scales | up_scales] (2f floats). Weight gradients are not computed here.
extern "C" int dfb200_swiglu_ffn_fp8_bwd(int T, int d, int f, const void * dOut_bf16, const void * gate_saved_bf16, const void * up_saved_bf16,
                                         const void * WdownT, const float * down_scales, const void * WgateupT, const float * gateup_scales,
                                         void * dA_bf16, void * workspace, uint64_t workspace_bytes, void * stream) {
	if (T <= 0 || d <= 0 || f <= 0 || d % 16 || f % 16) return set_error(DFB200_ERR_ARG, "swiglu_ffn_fp8_bwd: bad shape (T %d, d %d, f %d; d and f multiples of 16)", T, d, f);
	const uint64_t need = dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f);
	if (!workspace || workspace_bytes < need || !aligned16(workspace))
		return set_error(DFB200_ERR_WORKSPACE, "swiglu_ffn_fp8_bwd: needs %llu bytes of 16-byte aligned workspace, got %llu", (unsigned long long) need, (unsigned long long) workspace_bytes);
	uint8_t * p = static_cast<uint8_t *>(workspace);
	auto take = [&](uint64_t bytes) { uint8_t * q = p; p += align256(bytes); return q; };
	void * dOq = take((uint64_t) T * d);
	float * s1 = reinterpret_cast<float *>(take((uint64_t) T * 4));
	void * dGU = take((uint64_t) T * f * 4);
	void * dGUq = take((uint64_t) T * f * 2);
	float * s2 = reinterpret_cast<float *>(take((uint64_t) T * 4));
	int rc = dfb200_quantize_rows_e4m3(T, d, dOut_bf16, down_scales, dOq, s1, stream);
	if (!rc) rc = dfb200_gemm_e4m3_swiglu_bwd(T, f, d, dOq, s1, WdownT, gate_saved_bf16, up_saved_bf16, dGU, stream);
	if (!rc) rc = dfb200_quantize_rows_e4m3(T, 2 * f, dGU, gateup_scales, dGUq, s2, stream);
	if (!rc) rc = dfb200_gemm_e4m3(T, d, 2 * f, dGUq, s2, WgateupT, nullptr, nullptr, dA_bf16, stream);
	return rc;
}
