// Row gather / scatter ops either side of the layer chain: the embedding lookup and the copy of new K/V rows
// into per-sequence context buffers. Both move whole rows unchanged, so they are byte copies whatever the
// datatype; what matters is 16-byte packets, one packet per thread (occupancy gives the bytes in flight,
// as in the SwiGLU kernels) and no integer division per element: a thread's (row, packet) comes from one
// 32-bit division by the packets-per-row of the launch.
//
// Reference semantics:
//   embedding (src/ops/nvidia/preprocess/embedding.cu:3-24): output[t, :] = table[token_ids[t], :]. The reference
//     multiplies its element offsets by sizeof(element) while indexing typed pointers (:14-20), which lands
//     outside the row for every type wider than one byte; the intended row copy is implemented here.
//   copy_to_seq_context (src/ops/nvidia/attention/copy_to_seq_context.cu:3-20): for token t with context base
//     C = seq_context_ptrs[t], position p = seq_positions[t] and context size S = seq_context_sizes[t]:
//     C[p, :] = keys[t, :] and C[S + p, :] = values[t, :] (keys of the whole context first, values after).
#include "common.cuh"

namespace dfb200 {

constexpr int ROW_COPY_THREADS = 512;

// PACKET = bytes moved per thread: 16 when rows and bases allow it, else the largest power of two that divides them.
template <int PACKET> struct Packet;
template <> struct Packet<16> { using T = uint4; };
template <> struct Packet<8> { using T = uint2; };
template <> struct Packet<4> { using T = uint32_t; };
template <> struct Packet<2> { using T = uint16_t; };
template <> struct Packet<1> { using T = uint8_t; };

template <int PACKET>
__global__ void __launch_bounds__(ROW_COPY_THREADS)
embedding_kernel(uint64_t n_packets, uint32_t packets_per_row, const uint32_t * __restrict__ token_ids, const uint8_t * __restrict__ table,
                 uint8_t * __restrict__ out) {
	using P = typename Packet<PACKET>::T;
	const uint64_t i = (uint64_t) blockIdx.x * ROW_COPY_THREADS + threadIdx.x;
	if (i >= n_packets) return;
	const uint64_t row = i / packets_per_row;
	const uint32_t col = (uint32_t) (i - row * packets_per_row);
	const uint64_t src_row = __ldg(token_ids + row);
	const P v = __ldg(reinterpret_cast<const P *>(table + (src_row * packets_per_row + col) * PACKET));
	__stcs(reinterpret_cast<P *>(out + i * PACKET), v);
}

// The context bases are only known on the device, so their alignment is checked here: a base that is not a multiple of
// PACKET falls back to byte stores for that token instead of issuing a misaligned access.
template <int PACKET>
__global__ void __launch_bounds__(ROW_COPY_THREADS)
copy_to_seq_context_kernel(uint64_t n_packets, uint32_t packets_per_row, const uint8_t * __restrict__ keys, const uint8_t * __restrict__ values,
                           const int * __restrict__ seq_positions, const uint64_t * __restrict__ seq_context_ptrs,
                           const int * __restrict__ seq_context_sizes) {
	using P = typename Packet<PACKET>::T;
	const uint64_t i = (uint64_t) blockIdx.x * ROW_COPY_THREADS + threadIdx.x;
	if (i >= n_packets) return;
	const uint64_t tok = i / packets_per_row;
	const uint32_t col = (uint32_t) (i - tok * packets_per_row);
	const uint64_t row_bytes = (uint64_t) packets_per_row * PACKET;
	uint8_t * ctx = reinterpret_cast<uint8_t *>(__ldg(seq_context_ptrs + tok));
	const uint64_t pos = (uint64_t) __ldg(seq_positions + tok);
	const uint64_t size = (uint64_t) __ldg(seq_context_sizes + tok);
	const P k = __ldcs(reinterpret_cast<const P *>(keys + i * PACKET));
	const P v = __ldcs(reinterpret_cast<const P *>(values + i * PACKET));
	uint8_t * dst_k = ctx + pos * row_bytes + (uint64_t) col * PACKET;
	uint8_t * dst_v = ctx + (size + pos) * row_bytes + (uint64_t) col * PACKET;
	if (PACKET == 1 || (reinterpret_cast<uintptr_t>(ctx) & (PACKET - 1)) == 0) {
		*reinterpret_cast<P *>(dst_k) = k;
		*reinterpret_cast<P *>(dst_v) = v;
	} else {
		const uint8_t * kb = reinterpret_cast<const uint8_t *>(&k), * vb = reinterpret_cast<const uint8_t *>(&v);
		#pragma unroll
		for (int b = 0; b < PACKET; b++) { dst_k[b] = kb[b]; dst_v[b] = vb[b]; }
	}
}

static int packet_bytes(uint64_t row_bytes, const void * a, const void * b, const void * c) {
	const uintptr_t bits = (uintptr_t) row_bytes | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
	for (int p = 16; p > 1; p >>= 1)
		if ((bits & (uintptr_t) (p - 1)) == 0) return p;
	return 1;
}

}  // namespace dfb200

using namespace dfb200;

extern "C" int dfb200_embedding(int dt, int num_tokens, int embed_dim, const uint32_t * token_ids, const void * embedding_table, void * output,
                                void * stream) {
	const int es = dtype_size(dt);
	if (!es) return set_error(DFB200_ERR_DTYPE, "embedding: unsupported datatype %d", dt);
	if (num_tokens < 0 || embed_dim <= 0) return set_error(DFB200_ERR_ARG, "embedding: bad shape (%d tokens, dim %d)", num_tokens, embed_dim);
	if (num_tokens == 0) return DFB200_OK;
	if (!token_ids || !embedding_table || !output) return set_error(DFB200_ERR_ARG, "embedding: NULL pointer");
	if (reinterpret_cast<uintptr_t>(token_ids) & 3u) return set_error(DFB200_ERR_ARG, "embedding: token_ids must be 4-byte aligned");
	const uint64_t row_bytes = (uint64_t) embed_dim * es;
	const int p = packet_bytes(row_bytes, embedding_table, output, nullptr);
	if (p < es) return set_error(DFB200_ERR_ARG, "embedding: table and output must be aligned to the element size");
	const uint64_t ppr = row_bytes / p, n = ppr * (uint64_t) num_tokens;
	if (ppr > 0xffffffffull) return set_error(DFB200_ERR_ARG, "embedding: row too long");
	const unsigned grid = (unsigned) ((n + ROW_COPY_THREADS - 1) / ROW_COPY_THREADS);
	const uint8_t * t = static_cast<const uint8_t *>(embedding_table);
	uint8_t * o = static_cast<uint8_t *>(output);
	cudaStream_t s = (cudaStream_t) stream;
	switch (p) {
		case 16: embedding_kernel<16><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, token_ids, t, o); break;
		case 8:  embedding_kernel<8><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, token_ids, t, o); break;
		case 4:  embedding_kernel<4><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, token_ids, t, o); break;
		case 2:  embedding_kernel<2><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, token_ids, t, o); break;
		default: embedding_kernel<1><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, token_ids, t, o); break;
	}
	return check_launch("embedding");
}

extern "C" int dfb200_copy_to_seq_context(int dt, uint64_t N, int total_tokens, int kv_dim, const void * keys, const void * values,
                                          const int * seq_positions, const uint64_t * seq_context_ptrs, const int * seq_context_sizes, void * stream) {
	const int es = dtype_size(dt);
	if (!es) return set_error(DFB200_ERR_DTYPE, "copy_to_seq_context: unsupported datatype %d", dt);
	if (total_tokens < 0 || kv_dim <= 0 || N != (uint64_t) total_tokens * (uint64_t) kv_dim)
		return set_error(DFB200_ERR_ARG, "copy_to_seq_context: N (%llu) must equal total_tokens (%d) x kv_dim (%d)", (unsigned long long) N, total_tokens, kv_dim);
	if (total_tokens == 0) return DFB200_OK;
	if (!keys || !values || !seq_positions || !seq_context_ptrs || !seq_context_sizes) return set_error(DFB200_ERR_ARG, "copy_to_seq_context: NULL pointer");
	if ((reinterpret_cast<uintptr_t>(seq_positions) & 3u) || (reinterpret_cast<uintptr_t>(seq_context_sizes) & 3u) || (reinterpret_cast<uintptr_t>(seq_context_ptrs) & 7u))
		return set_error(DFB200_ERR_ARG, "copy_to_seq_context: misaligned index array");
	const uint64_t row_bytes = (uint64_t) kv_dim * es;
	const int p = packet_bytes(row_bytes, keys, values, nullptr);
	if (p < es) return set_error(DFB200_ERR_ARG, "copy_to_seq_context: keys and values must be aligned to the element size");
	const uint64_t ppr = row_bytes / p, n = ppr * (uint64_t) total_tokens;
	const unsigned grid = (unsigned) ((n + ROW_COPY_THREADS - 1) / ROW_COPY_THREADS);
	const uint8_t * k = static_cast<const uint8_t *>(keys), * v = static_cast<const uint8_t *>(values);
	cudaStream_t s = (cudaStream_t) stream;
	switch (p) {
		case 16: copy_to_seq_context_kernel<16><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, k, v, seq_positions, seq_context_ptrs, seq_context_sizes); break;
		case 8:  copy_to_seq_context_kernel<8><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, k, v, seq_positions, seq_context_ptrs, seq_context_sizes); break;
		case 4:  copy_to_seq_context_kernel<4><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, k, v, seq_positions, seq_context_ptrs, seq_context_sizes); break;
		case 2:  copy_to_seq_context_kernel<2><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, k, v, seq_positions, seq_context_ptrs, seq_context_sizes); break;
		default: copy_to_seq_context_kernel<1><<<grid, ROW_COPY_THREADS, 0, s>>>(n, (uint32_t) ppr, k, v, seq_positions, seq_context_ptrs, seq_context_sizes); break;
	}
	return check_launch("copy_to_seq_context");
}
