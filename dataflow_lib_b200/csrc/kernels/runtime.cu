// Host-side support shared by all launchers: thread-local error text, cached device
// properties, launch checking.
#include "common.cuh"

#include <stdarg.h>
#include <string.h>

namespace dfb200 {

static thread_local char g_err[512] = "";

int set_error(int code, const char * fmt, ...) {
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(g_err, sizeof(g_err), fmt, ap);
	va_end(ap);
	return code;
}

int sm_count() {
	static int cached[64];          // 0 = not queried yet
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
	if (dev < 0 || dev >= 64) return 0;
	if (cached[dev] == 0) {
		int n = 0;
		if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); return 0; }
		cached[dev] = n;
	}
	return cached[dev];
}

int check_launch(const char * what) {
	cudaError_t e = cudaGetLastError();
	if (e != cudaSuccess) return set_error(DFB200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
	return DFB200_OK;
}

}  // namespace dfb200

extern "C" const char * dfb200_last_error(void) { return dfb200::g_err; }
extern "C" const char * dfb200_target_arch(void) { return "sm_100a"; }
extern "C" int dfb200_sm_count(void) { return dfb200::sm_count(); }
