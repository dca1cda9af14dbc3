// Shared device/host helpers for the sm_100a op kernels: element-type traits with the
// datatype conversions folded into 128-bit global loads/stores, warp/block reductions,
// error reporting and launch-geometry queries.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>

#include "dataflow_abi.h"
#include "dataflow_b200_kernels.h"

namespace dfb200 {

// ---------------------------------------------------------------------------------------
// host side: errors, device properties
// ---------------------------------------------------------------------------------------

int set_error(int code, const char * fmt, ...);     // stores a thread-local message, returns code
int sm_count();                                      // SMs of the current device (cached per device)
int check_launch(const char * what);                 // cudaGetLastError -> DFB200_ERR_CUDA or OK
// Resident CTAs per SM of `kernel` at this launch shape on the current device (>= 1); the driver query is made
// once per (kernel, threads, shared memory, device) and remembered.
int ctas_per_sm(const void * kernel, int threads, size_t dyn_smem);
// Opts `kernel` in to `dyn_smem` bytes of dynamic shared memory (needed above 48 KB); remembered per kernel and CUDA context.
void allow_dyn_smem(const void * kernel, size_t dyn_smem);
// Unique id of the CUDA context current on the calling thread (binds the device's primary context when the thread has none).
uint64_t context_key();
// Device address of a __device__ variable in the current context (cudaGetSymbolAddress), remembered per (variable, context);
// NULL on error. Host code must never pass the variable's name itself to a kernel: there it is a host-side stand-in.
void * symbol_address(const void * symbol);

// Launch with programmatic stream serialisation: the kernel's CTAs may become resident while the previous kernel of the stream
// is still draining (that kernel calls pdl_prologue(), which lets its successor be scheduled early). A kernel launched this way
// must call pdl_prologue() before its first access to global memory: it returns once the predecessor has completed and its
// writes are visible, so stream order is kept exactly; what is saved is the launch latency and the ramp between short kernels.
template <typename... KArgs, typename... Args>
static inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&... args) {
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr; cfg.numAttrs = 1;
	(void) cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);      // a failure stays readable through cudaGetLastError (check_launch)
}
#ifdef __CUDACC__
// Asks L2 for the line that holds *p. Legal before cudaGridDependencySynchronize() whatever the previous kernel of the stream writes:
// nothing reaches a register, and a line that the previous kernel still writes stays coherent in the one L2. A kernel that waits for
// its predecessor's last CTAs uses the wait to have its own first loads hit L2 instead of starting a trip to DRAM afterwards.
__device__ __forceinline__ void prefetch_l2(const void * p) { asm volatile("prefetch.global.L2 [%0];" :: "l"(p)); }

__device__ __forceinline__ void pdl_prologue() {
	cudaTriggerProgrammaticLaunchCompletion();       // the next kernel of the stream may be scheduled; it still waits for this one to finish
	cudaGridDependencySynchronize();                 // the previous kernel of the stream has finished and its writes are visible
}
#endif

static inline bool aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline int dtype_size(int dt) {
	switch (dt) {
		case DATAFLOW_FP32: return 4;
		case DATAFLOW_FP16: case DATAFLOW_BF16: return 2;
		case DATAFLOW_FP8E4M3: case DATAFLOW_FP8E5M2: return 1;
		default: return 0;
	}
}

// ---------------------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------------------

struct f32_t  { float v; };
struct f16_t  { __half v; };
struct bf16_t { __nv_bfloat16 v; };
struct e4m3_t { uint8_t v; };
struct e5m2_t { uint8_t v; };

// Conversions work on 32-bit words: a word holds EPW elements of T (1 fp32, 2 half/bf16,
// 4 fp8). They are the CUDA intrinsics' conversions: round-to-nearest-even, fp8 saturating
// to the largest finite value.
template <typename T> struct Word;

template <> struct Word<f32_t> {
	static constexpr int EPW = 1;
	static __device__ __forceinline__ void unpack(uint32_t w, float * f) { f[0] = __uint_as_float(w); }
	static __device__ __forceinline__ uint32_t pack(const float * f) { return __float_as_uint(f[0]); }
};
template <> struct Word<bf16_t> {
	static constexpr int EPW = 2;
	static __device__ __forceinline__ void unpack(uint32_t w, float * f) {   // bf16 -> fp32 is a 16-bit shift
		f[0] = __uint_as_float(w << 16); f[1] = __uint_as_float(w & 0xffff0000u);
	}
	static __device__ __forceinline__ uint32_t pack(const float * f) {
		__nv_bfloat162 h = __floats2bfloat162_rn(f[0], f[1]);
		return *reinterpret_cast<uint32_t *>(&h);
	}
};
template <> struct Word<f16_t> {
	static constexpr int EPW = 2;
	static __device__ __forceinline__ void unpack(uint32_t w, float * f) {
		float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w));
		f[0] = p.x; f[1] = p.y;
	}
	static __device__ __forceinline__ uint32_t pack(const float * f) {
		__half2 h = __floats2half2_rn(f[0], f[1]);
		return *reinterpret_cast<uint32_t *>(&h);
	}
};
template <__nv_fp8_interpretation_t KIND> struct WordFp8 {
	static constexpr int EPW = 4;
	static __device__ __forceinline__ void unpack(uint32_t w, float * f) {
		#pragma unroll
		for (int j = 0; j < 2; j++) {
			__half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w >> (16 * j)) & 0xffffu), KIND);
			float2 p = __half22float2(*reinterpret_cast<__half2 *>(&hr));
			f[2 * j] = p.x; f[2 * j + 1] = p.y;
		}
	}
	static __device__ __forceinline__ uint32_t pack(const float * f) {
		uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[0], f[1]), __NV_SATFINITE, KIND);
		uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[2], f[3]), __NV_SATFINITE, KIND);
		return lo | (hi << 16);
	}
};
template <> struct Word<e4m3_t> : WordFp8<__NV_E4M3> {};
template <> struct Word<e5m2_t> : WordFp8<__NV_E5M2> {};

// Round an fp32 value to T and back (the value a store of T followed by a load would give).
template <typename T> __device__ __forceinline__ float round_to(float x);
template <> __device__ __forceinline__ float round_to<f32_t>(float x) { return x; }
template <> __device__ __forceinline__ float round_to<bf16_t>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <> __device__ __forceinline__ float round_to<f16_t>(float x) { return __half2float(__float2half_rn(x)); }
template <> __device__ __forceinline__ float round_to<e4m3_t>(float x) {
	__half_raw hr = __nv_cvt_fp8_to_halfraw(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3), __NV_E4M3);
	return __half2float(*reinterpret_cast<__half *>(&hr));
}
template <> __device__ __forceinline__ float round_to<e5m2_t>(float x) {
	__half_raw hr = __nv_cvt_fp8_to_halfraw(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E5M2), __NV_E5M2);
	return __half2float(*reinterpret_cast<__half *>(&hr));
}

// ---------------------------------------------------------------------------------------
// 128-bit global memory access. Streaming variants mark lines evict-first: every tensor on
// this path is touched once per launch, so nothing is worth keeping in L1/L2.
// ---------------------------------------------------------------------------------------

enum class Hint { STREAM, KEEP };

template <int WORDS, Hint H> __device__ __forceinline__ void ld_words(const void * p, uint32_t (&w)[WORDS]) {
	static_assert(WORDS == 2 || WORDS == 4 || WORDS == 8, "8, 16 or 32 bytes per access");
	if constexpr (WORDS == 2) {
		if constexpr (H == Hint::STREAM) asm volatile("ld.global.cs.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "l"(p));
		else { uint2 r = __ldg(reinterpret_cast<const uint2 *>(p)); w[0] = r.x; w[1] = r.y; }
	} else {
		#pragma unroll
		for (int i = 0; i < WORDS; i += 4) {
			const char * q = reinterpret_cast<const char *>(p) + 4 * i;
			if constexpr (H == Hint::STREAM)
				asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[i]), "=r"(w[i + 1]), "=r"(w[i + 2]), "=r"(w[i + 3]) : "l"(q));
			else { uint4 r = __ldg(reinterpret_cast<const uint4 *>(q)); w[i] = r.x; w[i + 1] = r.y; w[i + 2] = r.z; w[i + 3] = r.w; }
		}
	}
}
template <int WORDS> __device__ __forceinline__ void st_words(void * p, const uint32_t (&w)[WORDS]) {
	static_assert(WORDS == 2 || WORDS == 4 || WORDS == 8, "8, 16 or 32 bytes per access");
	if constexpr (WORDS == 2) {
		asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(w[0]), "r"(w[1]) : "memory");
	} else {
		#pragma unroll
		for (int i = 0; i < WORDS; i += 4) {
			char * q = reinterpret_cast<char *>(p) + 4 * i;
			asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(q), "r"(w[i]), "r"(w[i + 1]), "r"(w[i + 2]), "r"(w[i + 3]) : "memory");
		}
	}
}

// E consecutive elements of T starting at element index `idx` of `base`, as fp32.
template <typename T, int E, Hint H = Hint::STREAM>
__device__ __forceinline__ void load_elems(const void * base, uint64_t idx, float (&f)[E]) {
	constexpr int EPW = Word<T>::EPW;
	constexpr int WORDS = E / EPW;
	uint32_t w[WORDS];
	ld_words<WORDS, H>(reinterpret_cast<const char *>(base) + idx * (4 / EPW), w);
	#pragma unroll
	for (int i = 0; i < WORDS; i++) Word<T>::unpack(w[i], &f[i * EPW]);
}
template <typename T, int E>
__device__ __forceinline__ void store_elems(void * base, uint64_t idx, const float (&f)[E]) {
	constexpr int EPW = Word<T>::EPW;
	constexpr int WORDS = E / EPW;
	uint32_t w[WORDS];
	#pragma unroll
	for (int i = 0; i < WORDS; i++) w[i] = Word<T>::pack(&f[i * EPW]);
	st_words<WORDS>(reinterpret_cast<char *>(base) + idx * (4 / EPW), w);
}
// one element, rounded to T like store_elems rounds (the element occupies the low bits of a packed word)
template <typename T>
__device__ __forceinline__ void store_one(void * base, uint64_t idx, float f) {
	constexpr int EPW = Word<T>::EPW;
	float v[EPW];
	#pragma unroll
	for (int i = 0; i < EPW; i++) v[i] = i == 0 ? f : 0.0f;
	const uint32_t w = Word<T>::pack(v);
	if constexpr (EPW == 1) reinterpret_cast<uint32_t *>(base)[idx] = w;
	else if constexpr (EPW == 2) reinterpret_cast<uint16_t *>(base)[idx] = (uint16_t) w;
	else reinterpret_cast<uint8_t *>(base)[idx] = (uint8_t) w;
}

// one element as fp32 (the general-shape kernels: rows that are not multiples of 8 elements, tensors that are not 16-byte aligned)
template <typename T>
__device__ __forceinline__ float load_one(const void * base, uint64_t idx) {
	constexpr int EPW = Word<T>::EPW;
	float v[EPW];
	if constexpr (EPW == 1) { Word<T>::unpack(reinterpret_cast<const uint32_t *>(base)[idx], v); return v[0]; }
	else if constexpr (EPW == 2) { Word<T>::unpack((uint32_t) reinterpret_cast<const uint16_t *>(base)[idx], v); return v[0]; }
	else { Word<T>::unpack((uint32_t) reinterpret_cast<const uint8_t *>(base)[idx], v); return v[0]; }
}

// ---------------------------------------------------------------------------------------
// fast math: the approximate, flush-to-zero hardware forms that the reference build selects with
// --use_fast_math (expf -> ex2.approx.ftz(x * log2 e), a / b -> a * rcp.approx.ftz(b)). Written as PTX because the
// CUDA intrinsics without the global -ftz flag wrap the same instructions in denormal fix-ups (3 extra
// instructions per call), which matters in the instruction-bound softmax.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp(float x) {
	float t, y;
	asm("mul.ftz.f32 %0, %1, 0f3FB8AA3B;" : "=f"(t) : "f"(x));      // log2(e)
	asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(t));
	return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
	float y;
	asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
	return y;
}

// ---------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
	#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}
__device__ __forceinline__ float warp_max(float v) {
	#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
	return v;
}

// Dispatch a DataflowDatatype value to a template instantiation.
#define DFB200_DISPATCH_DTYPE(dt, T, ...)                                       \
	switch (dt) {                                                               \
		case DATAFLOW_FP32:    { using T = ::dfb200::f32_t;  __VA_ARGS__; break; } \
		case DATAFLOW_FP16:    { using T = ::dfb200::f16_t;  __VA_ARGS__; break; } \
		case DATAFLOW_BF16:    { using T = ::dfb200::bf16_t; __VA_ARGS__; break; } \
		case DATAFLOW_FP8E4M3: { using T = ::dfb200::e4m3_t; __VA_ARGS__; break; } \
		case DATAFLOW_FP8E5M2: { using T = ::dfb200::e5m2_t; __VA_ARGS__; break; } \
		default: break;                                                         \
	}

// The seven (forward, backward) datatype pairs the reference registers for its bwd ops.
static inline bool valid_fwd_bwd_pair(int fwd_dt, int bwd_dt) {
	switch (fwd_dt) {
		case DATAFLOW_FP32: return bwd_dt == DATAFLOW_FP32;
		case DATAFLOW_FP16: return bwd_dt == DATAFLOW_FP16;
		case DATAFLOW_BF16: return bwd_dt == DATAFLOW_BF16;
		case DATAFLOW_FP8E4M3: case DATAFLOW_FP8E5M2: return bwd_dt == DATAFLOW_FP16 || bwd_dt == DATAFLOW_BF16;
		default: return false;
	}
}

#define DFB200_DISPATCH_PAIR(fwd_dt, bwd_dt, F, B, ...)                                              \
	switch (fwd_dt) {                                                                                \
		case DATAFLOW_FP32: { using F = ::dfb200::f32_t;  using B = ::dfb200::f32_t;  __VA_ARGS__; break; } \
		case DATAFLOW_FP16: { using F = ::dfb200::f16_t;  using B = ::dfb200::f16_t;  __VA_ARGS__; break; } \
		case DATAFLOW_BF16: { using F = ::dfb200::bf16_t; using B = ::dfb200::bf16_t; __VA_ARGS__; break; } \
		case DATAFLOW_FP8E4M3:                                                                       \
			if (bwd_dt == DATAFLOW_FP16) { using F = ::dfb200::e4m3_t; using B = ::dfb200::f16_t;  __VA_ARGS__; } \
			else                         { using F = ::dfb200::e4m3_t; using B = ::dfb200::bf16_t; __VA_ARGS__; } \
			break;                                                                                   \
		case DATAFLOW_FP8E5M2:                                                                       \
			if (bwd_dt == DATAFLOW_FP16) { using F = ::dfb200::e5m2_t; using B = ::dfb200::f16_t;  __VA_ARGS__; } \
			else                         { using F = ::dfb200::e5m2_t; using B = ::dfb200::bf16_t; __VA_ARGS__; } \
			break;                                                                                   \
		default: break;                                                                              \
	}

}  // namespace dfb200
