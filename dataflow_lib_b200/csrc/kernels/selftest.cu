// Self-test of the bounded device-side wait that every kernel with asynchronous copies relies on (tma.cuh: mbar_wait_bounded):
// one thread waits on an mbarrier that nothing will ever complete. The wait must give up at its time limit, record where in the
// kernel status word and let the kernel END normally -- the context stays usable and the host learns about it through
// dfb200_read_kernel_status. This is how a lost copy or a peer that never arrives is meant to surface: as a status, not as a hang.
#include "common.cuh"
#include "tma.cuh"

namespace dfb200 {

constexpr unsigned int SELFTEST_WAIT_CODE = 0x7e57u;

__global__ void bounded_wait_selftest_kernel(unsigned int * status, unsigned int * gave_up) {
	__shared__ uint64_t bar;
	if (threadIdx.x == 0) {
		mbar_init(&bar, 1);
		mbar_fence_init();
		const bool done = mbar_wait_bounded(&bar, 0, status, SELFTEST_WAIT_CODE);     // phase 0 never completes: no arrival is ever made
		*gave_up = done ? 0u : 1u;
	}
}

}  // namespace dfb200

using namespace dfb200;

// Launches the self-test kernel on `stream` (it runs for the wait limit, about two seconds) and synchronises. Returns 1 when the wait
// gave up as designed, 0 when it claims to have completed, negative on a CUDA error. The status word of `slot` then holds the code
// 0x7e57 until dfb200_read_kernel_status clears it.
extern "C" int dfb200_selftest_bounded_wait(int slot, void * stream) {
	if (slot < 0 || slot >= STATUS_SLOTS) return set_error(DFB200_ERR_ARG, "selftest_bounded_wait: slot %d out of range", slot);
	unsigned int * status = kernel_status_word(slot);
	if (!status) return set_error(DFB200_ERR_CUDA, "selftest_bounded_wait: no status word");
	unsigned int * flag = nullptr;
	cudaError_t e = cudaMalloc(&flag, sizeof(unsigned int));
	if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "selftest_bounded_wait: %s", cudaGetErrorString(e)); }
	bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t) stream>>>(status, flag);
	unsigned int host_flag = 0;
	e = cudaGetLastError();
	if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t) stream);
	if (e == cudaSuccess) e = cudaMemcpy(&host_flag, flag, sizeof(host_flag), cudaMemcpyDeviceToHost);
	cudaFree(flag);
	if (e != cudaSuccess) { cudaGetLastError(); return set_error(DFB200_ERR_CUDA, "selftest_bounded_wait: %s", cudaGetErrorString(e)); }
	return (int) host_flag;
}
