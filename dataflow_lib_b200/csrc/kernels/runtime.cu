// Host-side support shared by all launchers: thread-local error text, cached device
// properties, launch checking.
#include "common.cuh"
#include "tma.cuh"

#include <pthread.h>
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

// ---- the CUDA context current on the calling thread ----------------------------------------------------------------------
// Device symbols, loaded kernels and their attributes belong to a CONTEXT, not to a device. A program normally has one context
// per device (the primary one), but a caller may run these launchers inside a context of its own -- the reference's handle makes
// one with cuCtxCreate (src/dataflow_handle/nvidia/src/cuda_drv.c:35-49) and the runtime then works in whichever context is
// current -- so whatever is remembered about a symbol's address or a kernel's attributes is keyed by the context's unique id.
uint64_t context_key() {
	typedef int (*GetCurrentFn)(void **);
	typedef int (*GetIdFn)(void *, unsigned long long *);
	static GetCurrentFn get_current = nullptr;
	static GetIdFn get_id = nullptr;
	static bool resolved = false;
	if (!resolved) {
		void * p = nullptr, * q = nullptr;
		cudaDriverEntryPointQueryResult r;
		if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &r) != cudaSuccess || r != cudaDriverEntryPointSuccess) { cudaGetLastError(); p = nullptr; }
		if (cudaGetDriverEntryPoint("cuCtxGetId", &q, cudaEnableDefault, &r) != cudaSuccess || r != cudaDriverEntryPointSuccess) { cudaGetLastError(); q = nullptr; }
		get_current = reinterpret_cast<GetCurrentFn>(p);
		get_id = reinterpret_cast<GetIdFn>(q);
		resolved = true;
	}
	void * ctx = nullptr;
	if (get_current && get_current(&ctx) == 0 && !ctx) {        // no context yet on this thread: let the runtime bind the primary one
		if (cudaFree(nullptr) != cudaSuccess) cudaGetLastError();
		get_current(&ctx);
	}
	unsigned long long id = 0;
	if (ctx && get_id && get_id(ctx, &id) == 0) return 0x8000000000000000ull | id;
	if (ctx) return (uint64_t) reinterpret_cast<uintptr_t>(ctx);
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = 0; }
	return (uint64_t) dev + 1;
}

namespace {
struct LaunchMemo { const void * kernel; int device, threads; size_t smem; int value; uint64_t ctx; };
struct SymbolMemo { const void * symbol; uint64_t ctx; void * address; };
constexpr int MEMO_SLOTS = 256;
LaunchMemo g_occ[MEMO_SLOTS];      // written under g_memo_lock; entries are immutable once published
LaunchMemo g_smem[MEMO_SLOTS];
SymbolMemo g_sym[MEMO_SLOTS];
int g_occ_n = 0, g_smem_n = 0, g_sym_n = 0;
pthread_mutex_t g_memo_lock = PTHREAD_MUTEX_INITIALIZER;
}

int ctas_per_sm(const void * kernel, int threads, size_t dyn_smem) {
	int dev = 0;
	cudaGetDevice(&dev);
	pthread_mutex_lock(&g_memo_lock);
	for (int i = 0; i < g_occ_n; i++) {
		const LaunchMemo & m = g_occ[i];
		if (m.kernel == kernel && m.device == dev && m.threads == threads && m.smem == dyn_smem) { const int v = m.value; pthread_mutex_unlock(&g_memo_lock); return v; }
	}
	int per_sm = 0;
	if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dyn_smem) != cudaSuccess || per_sm < 1) { cudaGetLastError(); per_sm = 1; }
	if (g_occ_n < MEMO_SLOTS) g_occ[g_occ_n++] = LaunchMemo{kernel, dev, threads, dyn_smem, per_sm, 0};
	pthread_mutex_unlock(&g_memo_lock);
	return per_sm;
}

void allow_dyn_smem(const void * kernel, size_t dyn_smem) {
	if (dyn_smem <= 32 * 1024) return;             // static + dynamic may use 48 KB without opting in; kernels here have up to a few KB static
	const uint64_t ctx = context_key();
	pthread_mutex_lock(&g_memo_lock);
	LaunchMemo * slot = nullptr;
	for (int i = 0; i < g_smem_n; i++)
		if (g_smem[i].kernel == kernel && g_smem[i].ctx == ctx) { slot = &g_smem[i]; break; }
	if (!slot || slot->smem < dyn_smem) {
		if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) dyn_smem) != cudaSuccess) cudaGetLastError();
		if (slot) slot->smem = dyn_smem;
		else if (g_smem_n < MEMO_SLOTS) g_smem[g_smem_n++] = LaunchMemo{kernel, 0, 0, dyn_smem, 0, ctx};
	}
	pthread_mutex_unlock(&g_memo_lock);
}

void * symbol_address(const void * symbol) {
	const uint64_t ctx = context_key();
	pthread_mutex_lock(&g_memo_lock);
	for (int i = 0; i < g_sym_n; i++)
		if (g_sym[i].symbol == symbol && g_sym[i].ctx == ctx) { void * a = g_sym[i].address; pthread_mutex_unlock(&g_memo_lock); return a; }
	void * p = nullptr;
	// in host code the symbol's name is only a handle for the runtime, not a device address: ask for the address
	if (cudaGetSymbolAddress(&p, symbol) != cudaSuccess) { cudaGetLastError(); p = nullptr; }
	if (p && g_sym_n < MEMO_SLOTS) g_sym[g_sym_n++] = SymbolMemo{symbol, ctx, p};
	pthread_mutex_unlock(&g_memo_lock);
	return p;
}

int check_launch(const char * what) {
	cudaError_t e = cudaGetLastError();
	if (e != cudaSuccess) return set_error(DFB200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
	return DFB200_OK;
}

// [0, STATUS_SLOTS): the status words; [STATUS_SLOTS, 2 * STATUS_SLOTS): per family, the number of the launch whose wait gave up
// last (lets the other waits of that launch give up early without a stale value shortening the waits of later launches).
static __device__ unsigned int g_kernel_status[2 * STATUS_SLOTS];

unsigned int * kernel_status_word(int slot) {
	unsigned int * base = static_cast<unsigned int *>(symbol_address(g_kernel_status));
	return base ? base + slot : nullptr;
}

}  // namespace dfb200

// Synchronises `stream`, returns the OR-free maximum of the kernels' status words (0 = every bounded
// wait completed) and clears them. A non-zero value means a kernel gave up waiting for an
// asynchronous copy or a peer; the value identifies the wait.
extern "C" int dfb200_read_kernel_status(void * stream, unsigned int * status_words, int n_words) {
	unsigned int host[dfb200::STATUS_SLOTS];
	cudaError_t e = cudaStreamSynchronize((cudaStream_t) stream);
	if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host, dfb200::g_kernel_status, sizeof(host));       // the status words only
	if (e != cudaSuccess) return dfb200::set_error(DFB200_ERR_CUDA, "read_kernel_status: %s", cudaGetErrorString(e));
	unsigned int zero[dfb200::STATUS_SLOTS] = {0};
	unsigned int worst = 0;
	for (int i = 0; i < dfb200::STATUS_SLOTS; i++) { if (host[i] > worst) worst = host[i]; if (status_words && i < n_words) status_words[i] = host[i]; }
	if (worst) cudaMemcpyToSymbol(dfb200::g_kernel_status, zero, sizeof(zero));
	return (int) worst;
}

extern "C" const char * dfb200_last_error(void) { return dfb200::g_err; }
extern "C" const char * dfb200_target_arch(void) { return "sm_100a"; }
extern "C" int dfb200_sm_count(void) { return dfb200::sm_count(); }
