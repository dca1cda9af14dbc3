/*
 * CUDA backend of the dataflow handle: streams, events, memory, transfers and op dispatch.
 * Same function table and behaviour as als244/dataflow_lib's backend
 * (src/dataflow_handle/nvidia/src/cuda_dataflow_handle.c:53-918), with these deliberate changes:
 *
 *   - the handle lives in the device's PRIMARY context (the reference creates a private
 *     context with cuCtxCreate), so CUDA-runtime kernels, NCCL and framework allocators in
 *     the same process can share its streams and memory;
 *   - every call first makes the handle's device current, so one thread may drive several
 *     handles;
 *   - submit_peer_transfer really is a device-to-device copy dest <- src (the reference binds
 *     it to the outbound copy and its DtoD wrappers copy src -> src);
 *   - stream_id == -1 means the default stream in every call that takes a stream, and any
 *     other out-of-range id is an error instead of an out-of-bounds read.
 *
 * The CUDA runtime is used for everything except cubin loading and launching
 * (register_native_code), whose driver entry points are resolved from libcuda.so.1 at run
 * time so that this shared object loads on machines without a driver.
 */
#define _GNU_SOURCE
#include "dataflow_api.h"
#include "dataflow_b200_kernels.h"

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

/* ---- minimal driver-API surface, resolved lazily --------------------------------------- */

typedef int CUresult_t;
typedef struct {
	void * lib;
	CUresult_t (*cuCtxGetCurrent)(void ** ctx);
	CUresult_t (*cuDeviceGet)(int * dev, int ordinal);
	CUresult_t (*cuModuleLoad)(void ** module, const char * fname);
	CUresult_t (*cuModuleUnload)(void * module);
	CUresult_t (*cuModuleGetFunction)(void ** func, void * module, const char * name);
	CUresult_t (*cuFuncGetAttribute)(int * value, int attrib, void * func);
	CUresult_t (*cuLaunchKernel)(void * f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
	                             unsigned smem, void * stream, void ** params, void ** extra);
	CUresult_t (*cuGetErrorString)(CUresult_t err, const char ** str);
} Driver_Api;

static Driver_Api g_drv;

static int load_driver(void) {
	if (g_drv.lib) return 0;
	void * lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
	if (!lib) { fprintf(stderr, "Error: cannot open libcuda.so.1: %s\n", dlerror()); return -1; }
	Driver_Api d = {0};
#define RESOLVE(field, sym) do { *(void **) &d.field = dlsym(lib, sym); if (!d.field) { fprintf(stderr, "Error: libcuda lacks %s\n", sym); return -1; } } while (0)
	RESOLVE(cuCtxGetCurrent, "cuCtxGetCurrent");
	RESOLVE(cuDeviceGet, "cuDeviceGet");
	RESOLVE(cuModuleLoad, "cuModuleLoad");
	RESOLVE(cuModuleUnload, "cuModuleUnload");
	RESOLVE(cuModuleGetFunction, "cuModuleGetFunction");
	RESOLVE(cuFuncGetAttribute, "cuFuncGetAttribute");
	RESOLVE(cuLaunchKernel, "cuLaunchKernel");
	RESOLVE(cuGetErrorString, "cuGetErrorString");
#undef RESOLVE
	d.lib = lib;
	g_drv = d;
	return 0;
}

static const char * drv_err(CUresult_t r) {
	const char * s = NULL;
	if (g_drv.cuGetErrorString) g_drv.cuGetErrorString(r, &s);
	return s ? s : "unknown driver error";
}

/* ---- helpers ---------------------------------------------------------------------------- */

#define RT_CHECK(call, what, fail)                                                                      \
	do {                                                                                            \
		cudaError_t e_ = (call);                                                                    \
		if (e_ != cudaSuccess) {                                                                    \
			fprintf(stderr, "Error: %s: %s\n", what, cudaGetErrorString(e_));                       \
			cudaGetLastError();                                                                     \
			return fail;                                                                            \
		}                                                                                           \
	} while (0)

static int bind_device(Dataflow_Handle * h) {
	int cur = -1;
	if (cudaGetDevice(&cur) == cudaSuccess && cur == h->device_id) return 0;
	RT_CHECK(cudaSetDevice(h->device_id), "cannot make the handle's device current", -1);
	return 0;
}

/* Resolves a stream id: -1 -> default stream; [0, num_streams) -> that stream. */
static int resolve_stream(Dataflow_Handle * h, int stream_id, const char * what, cudaStream_t * out) {
	if (stream_id == -1) { *out = NULL; return 0; }
	if (stream_id < 0 || stream_id >= h->num_streams) {
		fprintf(stderr, "Error: cannot %s on stream id %d, when device only has %d streams. Null stream specified by -1...\n",
		        what, stream_id, h->num_streams);
		return -1;
	}
	*out = ((cudaStream_t *) h->streams)[stream_id];
	return 0;
}

static uint64_t op_table_hash(void * fingerprint, uint64_t table_size) {
	return fingerprint_to_least_sig64((uint8_t *) fingerprint, OP_IDENTIFIER_FINGERPRINT_NUM_BYTES) % table_size;
}

/* ---- 0. ops: registration ---------------------------------------------------------------- */

static int cuda_register_native_code(Dataflow_Handle * h, char * native_code_filename, char * native_code_config_lib_filename,
                                     int num_funcs, Op_Skeleton * func_op_skeletons, char ** func_symbols,
                                     char ** func_set_launch_symbols, char ** func_init_symbols) {
	if (h->num_native_function_libs >= MAX_NATIVE_FUNCTION_LIBS) {
		fprintf(stderr, "Error: cannot register more than %d native function libs...\n", MAX_NATIVE_FUNCTION_LIBS);
		return -1;
	}
	if (!native_code_filename || !native_code_config_lib_filename || num_funcs < 0) {
		fprintf(stderr, "Error: native code registration needs a cubin path and a launch-config library path\n");
		return -1;
	}
	if (bind_device(h) || load_driver()) return -1;
	void * module = NULL;
	CUresult_t r = g_drv.cuModuleLoad(&module, native_code_filename);
	if (r) {
		fprintf(stderr, "Error: unable to load function lib from path: %s (%s)\n", native_code_filename, drv_err(r));
		return -1;
	}
	void * cfg_lib = dlopen(native_code_config_lib_filename, RTLD_LAZY);
	if (!cfg_lib) {
		fprintf(stderr, "Error: could not load function config shared lib with dlopen() from path: %s\n", native_code_config_lib_filename);
		g_drv.cuModuleUnload(module);
		return -1;
	}
	int added = 0;
	for (int i = 0; i < num_funcs; i++) {
		const char * sym = func_symbols[i];
		if (!sym) continue;
		if (!func_set_launch_symbols || !func_set_launch_symbols[i]) {
			fprintf(stderr, "Error: set launch symbol not set for native function %s, but is required for native functions..\n", sym);
			continue;
		}
		Cuda_Function fn;
		memset(&fn, 0, sizeof(fn));
		fn.is_native = true;
		r = g_drv.cuModuleGetFunction(&fn.function_handle, module, sym);
		if (r) { fprintf(stderr, "Error: failed to load function #%d with name %s from function lib (%s)\n", i, sym, drv_err(r)); continue; }
		g_drv.cuFuncGetAttribute(&fn.function_config.func_max_threads_per_block, 0 /* MAX_THREADS_PER_BLOCK */, fn.function_handle);
		if (func_init_symbols && func_init_symbols[i]) {
			Cuda_Set_Func_Attribute set_attr = (Cuda_Set_Func_Attribute) dlsym(cfg_lib, func_init_symbols[i]);
			if (!set_attr) { fprintf(stderr, "Error: failed to load symbol %s to initialize function %s\n", func_init_symbols[i], sym); continue; }
			if (set_attr(h, &fn)) { fprintf(stderr, "Error: failed to set function attributes for %s via %s\n", sym, func_init_symbols[i]); continue; }
		}
		*(void **) &fn.set_launch_config = dlsym(cfg_lib, func_set_launch_symbols[i]);
		if (!fn.set_launch_config) { fprintf(stderr, "Error: failed to get launch config function %s for %s\n", func_set_launch_symbols[i], sym); continue; }
		memcpy(&fn.op_skeleton, &func_op_skeletons[i], sizeof(Op_Skeleton));
		if (insert_table(&h->op_table, fn.op_skeleton.identifier.fingerprint, &fn)) {
			fprintf(stderr, "Error: failed to insert op for function #%d with name %s to op table...\n", i, sym);
			continue;
		}
		added++;
	}
	if (added == 0) {
		fprintf(stderr, "Error: no functions were added to op table...\n");
		g_drv.cuModuleUnload(module);
		return -1;
	}
	h->native_function_libs[h->num_native_function_libs++] = module;
	h->num_ops += added;
	return added;
}

static int cuda_register_external_code(Dataflow_Handle * h, char * external_code_filename, int num_funcs,
                                       Op_Skeleton * func_op_skeletons, char ** func_symbols, char ** func_init_symbols) {
	if (!external_code_filename || num_funcs < 0) { fprintf(stderr, "Error: external code registration needs a library path\n"); return -1; }
	void * lib = dlopen(external_code_filename, RTLD_LAZY);
	if (!lib) {
		fprintf(stderr, "Error: could not open external library with path: %s (%s)\n", external_code_filename, dlerror());
		return -1;
	}
	if (bind_device(h)) return -1;
	int added = 0;
	for (int i = 0; i < num_funcs; i++) {
		const char * sym = func_symbols[i];
		if (!sym) continue;
		Cuda_Function fn;
		memset(&fn, 0, sizeof(fn));
		*(void **) &fn.cuda_external_func = dlsym(lib, sym);
		if (!fn.cuda_external_func) { fprintf(stderr, "Error: could not obtain function symbol %s from external lib %s...\n", sym, external_code_filename); continue; }
		memcpy(&fn.op_skeleton, &func_op_skeletons[i], sizeof(Op_Skeleton));   /* visible to the init function */
		if (func_init_symbols && func_init_symbols[i]) {
			External_Lib_Func_Init init = (External_Lib_Func_Init) dlsym(lib, func_init_symbols[i]);
			if (!init) { fprintf(stderr, "Error: could not get ref to initialization function %s, for external function %s\n", func_init_symbols[i], sym); continue; }
			if (init(h, &fn)) { fprintf(stderr, "Error: initialization function %s, for external function %s returned an error...\n", func_init_symbols[i], sym); continue; }
		}
		if (insert_table(&h->op_table, fn.op_skeleton.identifier.fingerprint, &fn)) {
			fprintf(stderr, "Error: failed to insert op for function #%d with name %s to op table...\n", i, sym);
			continue;
		}
		added++;
	}
	h->num_ops += added;
	return added;
}

/* ---- 1. compute --------------------------------------------------------------------------- */

static int cuda_submit_op(Dataflow_Handle * h, Op * op, int stream_id) {
	const char * nick = op->op_skeleton.header.op_nickname;
	cudaStream_t stream;
	if (stream_id != -1 && (stream_id < 0 || stream_id >= h->num_streams)) {
		fprintf(stderr, "Error: cannot submit op with nickname %s to stream id %d, when device only has %d streams. Null stream specified by -1...\n",
		        nick, stream_id, h->num_streams);
		return -1;
	}
	resolve_stream(h, stream_id, "submit op", &stream);
	Cuda_Function * fn = NULL;
	if (find_table(&h->op_table, op->op_skeleton.identifier.fingerprint, false, (void **) &fn) < 0 || !fn) {
		fprintf(stderr, "Error: failed to find op with nickname %s and matching dtypes...\n", nick);
		return -1;
	}
	if (bind_device(h)) return -1;
	if (fn->is_native) {
		Cuda_Launch_Config cfg;
		if (!fn->set_launch_config || fn->set_launch_config(&cfg, h, fn, op)) {
			fprintf(stderr, "Error: failed to correctly set launch config for op with nickname %s...\n", nick);
			return -1;
		}
		CUresult_t r = g_drv.cuLaunchKernel(fn->function_handle, cfg.gridDimX, cfg.gridDimY, cfg.gridDimZ,
		                                    cfg.blockDimX, cfg.blockDimY, cfg.blockDimZ, cfg.sharedMemBytes, stream, op->op_args, NULL);
		if (r) { fprintf(stderr, "Error: failed to launch kernel for op with nickname %s (%s)\n", nick, drv_err(r)); return -1; }
		return 0;
	}
	if (!fn->cuda_external_func) {
		fprintf(stderr, "Error: if op is not native it must have a reference to external function (error with op having nickname %s)\n", nick);
		return -1;
	}
	if (fn->cuda_external_func(h, stream_id, op, fn->op_extra)) {
		fprintf(stderr, "Error: failed to do external cuda function for op with nickname %s...\n", nick);
		return -1;
	}
	return 0;
}

static int cuda_submit_host_op(Dataflow_Handle * h, void * host_func, void * host_func_arg, int stream_id) {
	cudaStream_t stream;
	if (!host_func || resolve_stream(h, stream_id, "submit host op", &stream) || bind_device(h)) return -1;
	RT_CHECK(cudaLaunchHostFunc(stream, (cudaHostFn_t) host_func, host_func_arg), "failed to launch host function", -1);
	return 0;
}

/* ---- 2. dependencies ------------------------------------------------------------------------ */

static void * cuda_get_stream_state(Dataflow_Handle * h, int stream_id) {
	if (stream_id < 0 || stream_id >= h->num_streams) {
		fprintf(stderr, "Error: cannot get state of stream id %d (handle has %d streams)\n", stream_id, h->num_streams);
		return NULL;
	}
	if (bind_device(h)) return NULL;
	cudaEvent_t * events = (cudaEvent_t *) h->stream_states;
	RT_CHECK(cudaEventRecord(events[stream_id], ((cudaStream_t *) h->streams)[stream_id]),
	         "failed to record event when trying to get stream state", NULL);
	return &events[stream_id];
}

static int cuda_submit_dependency(Dataflow_Handle * h, int stream_id, void * other_stream_state) {
	cudaStream_t stream;
	if (!other_stream_state || resolve_stream(h, stream_id, "submit dependency", &stream) || bind_device(h)) return -1;
	RT_CHECK(cudaStreamWaitEvent(stream, *(cudaEvent_t *) other_stream_state, 0), "failed to have stream wait on event", -1);
	return 0;
}

/* The kernels' bounded device-side waits report through status words on the device (dfb200_read_kernel_status). A synchronising
 * call is where a caller of this interface learns that earlier work is complete, so it is also where a wait that gave up must
 * surface: the words are read (and cleared) after the synchronisation and a non-zero word fails the call. The rows or tiles whose
 * wait gave up hold NaN. */
static int kernels_gave_up(const char * what) {
	unsigned int words[8] = {0};
	const int worst = dfb200_read_kernel_status(NULL, words, 8);
	if (worst == 0) return 0;
	if (worst < 0) { fprintf(stderr, "Error: %s: cannot read the kernels' status: %s\n", what, dfb200_last_error()); return -1; }
	fprintf(stderr, "Error: %s: a kernel gave up a bounded wait (status words rope 0x%x, rms_norm 0x%x, softmax 0x%x, ffn 0x%x); its outputs hold NaN\n",
	        what, words[0], words[1], words[2], words[3]);
	return -1;
}

static int cuda_sync_stream(Dataflow_Handle * h, int stream_id) {
	cudaStream_t stream;
	if (resolve_stream(h, stream_id, "sync", &stream) || bind_device(h)) return -1;
	RT_CHECK(cudaStreamSynchronize(stream), "unable to do cuda stream synchronize", -1);
	return kernels_gave_up("sync_stream");
}

static int cuda_sync_handle(Dataflow_Handle * h) {
	if (bind_device(h)) return -1;
	RT_CHECK(cudaDeviceSynchronize(), "unable to sync the handle's device", -1);
	return kernels_gave_up("sync_handle");
}

/* ---- 3. memory ---------------------------------------------------------------------------- */

static void * cuda_alloc_mem(Dataflow_Handle * h, uint64_t size_bytes) {
	void * p = NULL;
	if (bind_device(h)) return NULL;
	cudaError_t e = cudaMalloc(&p, size_bytes);
	if (e != cudaSuccess || !p) {
		fprintf(stderr, "Error: failed to alloc memory on device id %d of size %lu bytes (%s)\n", h->device_id, (unsigned long) size_bytes, cudaGetErrorString(e));
		cudaGetLastError();
		return NULL;
	}
	return p;
}

static void cuda_free_mem(Dataflow_Handle * h, void * dev_ptr) {
	if (bind_device(h)) return;
	cudaError_t e = cudaFree(dev_ptr);
	if (e != cudaSuccess) {
		fprintf(stderr, "Error: was unable to free memory on device id %d with ptr %p (%s)\n", h->device_id, dev_ptr, cudaGetErrorString(e));
		cudaGetLastError();
	}
}

static int cuda_set_mem(Dataflow_Handle * h, int stream_id, void * dev_ptr, uint8_t val, uint64_t size_bytes) {
	cudaStream_t stream;
	if (resolve_stream(h, stream_id, "set memory", &stream) || bind_device(h)) return -1;
	if (stream_id == -1) RT_CHECK(cudaMemset(dev_ptr, val, size_bytes), "was unable to set device memory", -1);
	else RT_CHECK(cudaMemsetAsync(dev_ptr, val, size_bytes, stream), "was unable to set device memory", -1);
	return 0;
}

static int cuda_enable_access_to_host_mem(Dataflow_Handle * h, void * host_ptr, uint64_t size_bytes, unsigned int flags) {
	if (bind_device(h)) return -1;
	RT_CHECK(cudaHostRegister(host_ptr, size_bytes, flags), "failed to page-lock host memory for the device", -1);
	return 0;
}

static int cuda_disable_access_to_host_mem(Dataflow_Handle * h, void * host_ptr) {
	if (bind_device(h)) return -1;
	RT_CHECK(cudaHostUnregister(host_ptr), "failed to release page-locked host memory", -1);
	return 0;
}

static int cuda_enable_access_to_peer_mem(Dataflow_Handle * h, Dataflow_Handle * peer) {
	if (!peer || peer->compute_type != h->compute_type) { fprintf(stderr, "Error: cannot enable peer access, must be same compute type...\n"); return -1; }
	if (bind_device(h)) return -1;
	cudaError_t e = cudaDeviceEnablePeerAccess(peer->device_id, 0);
	if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
	if (e != cudaSuccess) {
		fprintf(stderr, "Error: was unable to allow this device (id %d) to access memory on peer device (id %d): %s\n", h->device_id, peer->device_id, cudaGetErrorString(e));
		cudaGetLastError();
		return -1;
	}
	return 0;
}

static int cuda_disable_access_to_peer_mem(Dataflow_Handle * h, Dataflow_Handle * peer) {
	if (!peer || peer->compute_type != h->compute_type) { fprintf(stderr, "Error: cannot disable peer access, must be same compute type...\n"); return -1; }
	if (bind_device(h)) return -1;
	cudaError_t e = cudaDeviceDisablePeerAccess(peer->device_id);
	if (e != cudaSuccess) {
		fprintf(stderr, "Error: was unable to disable this device (id %d) from accessing memory on peer device (id %d): %s\n", h->device_id, peer->device_id, cudaGetErrorString(e));
		cudaGetLastError();
		return -1;
	}
	return 0;
}

/* ---- 4. transfers --------------------------------------------------------------------------- */

static int do_transfer(Dataflow_Handle * h, int stream_id, void * dst, const void * src, uint64_t size_bytes, enum cudaMemcpyKind kind, const char * what) {
	cudaStream_t stream;
	if (resolve_stream(h, stream_id, what, &stream) || bind_device(h)) return -1;
	if (stream_id == -1) RT_CHECK(cudaMemcpy(dst, src, size_bytes, kind), what, -1);
	else RT_CHECK(cudaMemcpyAsync(dst, src, size_bytes, kind, stream), what, -1);
	return 0;
}

static int cuda_submit_inbound_transfer(Dataflow_Handle * h, int stream_id, void * dev_dest, void * host_src, uint64_t size_bytes) {
	return do_transfer(h, stream_id, dev_dest, host_src, size_bytes, cudaMemcpyHostToDevice, "transfer host to device");
}
static int cuda_submit_outbound_transfer(Dataflow_Handle * h, int stream_id, void * host_dest, void * dev_src, uint64_t size_bytes) {
	return do_transfer(h, stream_id, host_dest, dev_src, size_bytes, cudaMemcpyDeviceToHost, "transfer device to host");
}
static int cuda_submit_peer_transfer(Dataflow_Handle * h, int stream_id, void * dev_dest, void * dev_src, uint64_t size_bytes) {
	return do_transfer(h, stream_id, dev_dest, dev_src, size_bytes, cudaMemcpyDeviceToDevice, "transfer device to device");
}

/* ---- init / destroy ------------------------------------------------------------------------- */

int init_cuda_dataflow_handle(Dataflow_Handle * h, ComputeType compute_type, int device_id, int ctx_id, unsigned int ctx_flags,
                              int num_streams, int * opt_stream_prios, char ** opt_stream_names) {
	if (!h) return -1;
	if (num_streams < 0 || num_streams > MAX_STREAMS) {
		fprintf(stderr, "Error: number of streams %d outside [0, %d]\n", num_streams, MAX_STREAMS);
		return -1;
	}
	memset(h, 0, sizeof(*h));
	h->compute_type = compute_type;
	h->device_id = device_id;
	h->ctx_id = ctx_id;

	int n_dev = 0;
	RT_CHECK(cudaGetDeviceCount(&n_dev), "failed to initialize cuda", -1);
	if (device_id < 0 || device_id >= n_dev) { fprintf(stderr, "Error: failed to get device handle for dev id: %d...\n", device_id); return -1; }
	if (ctx_flags) {                       /* only takes effect while the primary context is inactive */
		cudaError_t e = cudaSetDeviceFlags(ctx_flags);
		if (e != cudaSuccess) cudaGetLastError();
	}
	RT_CHECK(cudaSetDevice(device_id), "unable to bind device", -1);
	RT_CHECK(cudaFree(0), "unable to initialize the device's primary context", -1);

	Cuda_Device_Info * info = (Cuda_Device_Info *) calloc(1, sizeof(Cuda_Device_Info));
	h->device_handle = calloc(1, sizeof(int));
	h->ctx = calloc(1, sizeof(void *));
	if (!info || !h->device_handle || !h->ctx) { fprintf(stderr, "Error: malloc failed while creating handle\n"); return -1; }
	h->device_info = info;
	*(int *) h->device_handle = device_id;
	if (load_driver() == 0) {
		g_drv.cuDeviceGet((int *) h->device_handle, device_id);
		g_drv.cuCtxGetCurrent((void **) h->ctx);
	}

	size_t free_b = 0, total_b = 0;
	RT_CHECK(cudaMemGetInfo(&free_b, &total_b), "unable to query device memory", -1);
	info->total_mem = total_b;
	int major = 0, minor = 0;
	cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_id);
	cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device_id);
	info->arch_num = 10 * major + minor;
	cudaDeviceGetAttribute(&info->sm_count, cudaDevAttrMultiProcessorCount, device_id);
	cudaDeviceGetAttribute(&info->max_threads_per_block, cudaDevAttrMaxThreadsPerBlock, device_id);
	if (info->max_threads_per_block > CUDA_DEV_UPPER_BOUND_MAX_THREADS_ALL_FUNC) info->max_threads_per_block = CUDA_DEV_UPPER_BOUND_MAX_THREADS_ALL_FUNC;
	cudaDeviceGetAttribute(&info->max_smem_per_block, cudaDevAttrMaxSharedMemoryPerBlock, device_id);
	cudaDeviceGetAttribute(&info->optin_max_smem_per_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_id);
	if (cudaDeviceGetAttribute(&info->host_numa_id, cudaDevAttrHostNumaId, device_id) != cudaSuccess) { cudaGetLastError(); info->host_numa_id = -1; }

	h->num_streams = num_streams;
	for (int i = 0; i < MAX_STREAMS; i++) {
		h->stream_prios[i] = i < num_streams ? (opt_stream_prios ? opt_stream_prios[i] : CUDA_DEFAULT_STREAM_PRIO) : -1;
		h->stream_names[i] = (i < num_streams && opt_stream_names && opt_stream_names[i]) ? strdup(opt_stream_names[i]) : NULL;
	}
	cudaStream_t * streams = (cudaStream_t *) calloc(num_streams ? num_streams : 1, sizeof(cudaStream_t));
	cudaEvent_t * events = (cudaEvent_t *) calloc(num_streams ? num_streams : 1, sizeof(cudaEvent_t));
	if (!streams || !events) { fprintf(stderr, "Error: malloc failed to allocate stream containers...\n"); return -1; }
	h->streams = streams;
	h->stream_states = events;
	for (int i = 0; i < num_streams; i++) {
		RT_CHECK(cudaStreamCreateWithPriority(&streams[i], cudaStreamNonBlocking, h->stream_prios[i]), "unable to initialize stream", -1);
		RT_CHECK(cudaEventCreateWithFlags(&events[i], cudaEventDisableTiming), "unable to initialize stream event", -1);
	}

	h->num_native_function_libs = 0;
	h->num_ops = 0;
	if (init_table(&h->op_table, op_table_hash, OP_IDENTIFIER_FINGERPRINT_NUM_BYTES, sizeof(Cuda_Function),
	               OP_TABLE_MIN_SIZE, OP_TABLE_MAX_SIZE, 1.0f, 1.0f)) {
		fprintf(stderr, "Error: failed to init op table...\n");
		return -1;
	}

	h->register_native_code = cuda_register_native_code;
	h->register_external_code = cuda_register_external_code;
	h->submit_op = cuda_submit_op;
	h->submit_host_op = cuda_submit_host_op;
	h->get_stream_state = cuda_get_stream_state;
	h->submit_dependency = cuda_submit_dependency;
	h->sync_stream = cuda_sync_stream;
	h->sync_handle = cuda_sync_handle;
	h->alloc_mem = cuda_alloc_mem;
	h->free_mem = cuda_free_mem;
	h->set_mem = cuda_set_mem;
	h->enable_access_to_host_mem = cuda_enable_access_to_host_mem;
	h->disable_access_to_host_mem = cuda_disable_access_to_host_mem;
	h->enable_access_to_peer_mem = cuda_enable_access_to_peer_mem;
	h->disable_access_to_peer_mem = cuda_disable_access_to_peer_mem;
	h->submit_inbound_transfer = cuda_submit_inbound_transfer;
	h->submit_outbound_transfer = cuda_submit_outbound_transfer;
	h->submit_peer_transfer = cuda_submit_peer_transfer;
	return 0;
}

void destroy_cuda_dataflow_handle(Dataflow_Handle * h) {
	if (!h || !h->streams) return;
	if (bind_device(h) == 0) {
		cudaDeviceSynchronize();
		for (int i = 0; i < h->num_streams; i++) {
			cudaStreamDestroy(((cudaStream_t *) h->streams)[i]);
			cudaEventDestroy(((cudaEvent_t *) h->stream_states)[i]);
		}
		for (int i = 0; i < h->num_native_function_libs; i++) if (g_drv.cuModuleUnload) g_drv.cuModuleUnload(h->native_function_libs[i]);
		/* scratch blocks that this library's ops keep in their table entries (entries of other plug-ins are not touched) */
		const Table * t = &h->op_table;
		const uint64_t slot = t->config.key_size_bytes + t->config.value_size_bytes;
		for (uint64_t i = 0; t->items && i < t->size; i++)
			if (!((t->is_empty_bit_vector[i >> 6] >> (i & 63)) & 1ULL))
				dataflow_b200_workspace_release((uint8_t *) t->items + i * slot + t->config.key_size_bytes);
	}
	for (int i = 0; i < MAX_STREAMS; i++) free(h->stream_names[i]);
	free(h->streams); free(h->stream_states); free(h->device_info); free(h->device_handle); free(h->ctx);
	destroy_table(&h->op_table);
	memset(h, 0, sizeof(*h));
}
