// Bulk asynchronous copies (the TMA unit's untiled cp.async.bulk form) with mbarrier completion,
// as used for shared-memory staging of row tiles. Only CTA-local destinations are used: every
// copy lands in the issuing CTA's own shared memory and no copy is replicated to other CTAs.
//
// Every wait is bounded: a wait that gives up records where in g_kernel_status and returns
// false, so a lost copy shows up as a status word on the host instead of a hung GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dfb200 {

// One status word per kernel family; 0 = no problem seen since the last read. The words live in
// one device array owned by runtime.cu; launchers pass kernels the address of their word.
enum KernelStatusSlot { STATUS_ROPE = 0, STATUS_RMS = 1, STATUS_SOFTMAX = 2, STATUS_FFN = 3, STATUS_SLOTS = 8 };
unsigned int * kernel_status_word(int slot);     // host: device address of a status word on the current device (NULL on error)

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;     // a wait gives up after two seconds of wall time

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t arrivals) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
// Makes freshly initialised barriers visible to the async proxy; follow with __syncthreads().
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t * bar, uint32_t tx_bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(tx_bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
	uint32_t done;
	asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
	             : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
	return done != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
	unsigned long long t;
	asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
	return t;
}

// Waits for the phase with the given parity to complete. Returns false (and records `where`
// in *status) when the time limit is reached; the clock is only consulted every 1024 attempts.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t * bar, uint32_t parity, unsigned int * status, unsigned int where) {
	if (mbar_try_wait(bar, parity)) return true;
	const unsigned long long t0 = global_timer_ns();
	for (;;) {
		for (int i = 0; i < 1024; i++)
			if (mbar_try_wait(bar, parity)) return true;
		if (global_timer_ns() - t0 > WAIT_LIMIT_NS) break;
	}
	atomicMax(status, where);
	return false;
}

// global -> this CTA's shared memory; completion is counted in bytes on `bar`. Addresses and size
// must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void * smem_dst, const void * gmem_src, uint32_t bytes, uint64_t * bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
	             :: "r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Asks L2 for `bytes` of global memory (multiples of 16, address 16-byte aligned); nothing reaches shared memory or registers, so it is
// legal before the wait for the previous kernel of the stream (see prefetch_l2 in common.cuh).
__device__ __forceinline__ void bulk_prefetch_l2(const void * gmem_src, uint32_t bytes) {
	asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(gmem_src), "r"(bytes) : "memory");
}
// this CTA's shared memory -> global, tracked by the thread's bulk-group.
__device__ __forceinline__ void bulk_store(void * gmem_dst, const void * smem_src, uint32_t bytes) {
	asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's committed store groups still READ shared memory.
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
// Waits until at most N of this thread's committed store groups are incomplete.
template <int N> __device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" :: "n"(N) : "memory"); }
// Orders this thread's generic-proxy shared-memory writes before later async-proxy (bulk copy) reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace dfb200
