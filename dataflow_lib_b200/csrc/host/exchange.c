/*
 * The token-sharded step's one collective (include/dataflow_b200_exchange.h): a sum all-reduce of the packed fp32 buffer
 * [loss sum, valid rows | RMSNorm weight gradients] over NCCL, enqueued on a stream of the rank's handle. The reference's handle has
 * no network section (src/dataflow_handle/include/dataflow_handle.h:120); this follows the conventions of its other calls.
 *
 * NCCL is not linked: its six entry points are resolved when the first exchange is set up, from the copy of libnccl.so.2 that is
 * already in the process when there is one (two NCCL copies in one process would each keep their own state), else from the loader path.
 */
#define _GNU_SOURCE
#include "dataflow_api.h"
#include "dataflow_b200_exchange.h"

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <string.h>

typedef struct { char internal[DATAFLOW_EXCHANGE_ID_BYTES]; } Nccl_Unique_Id;       /* ncclUniqueId */
typedef int (*Nccl_Get_Unique_Id)(Nccl_Unique_Id * id);
typedef int (*Nccl_Comm_Init_Rank)(void ** comm, int nranks, Nccl_Unique_Id id, int rank);
typedef int (*Nccl_All_Reduce)(const void * send, void * recv, size_t count, int datatype, int op, void * comm, void * stream);
typedef int (*Nccl_Comm_Destroy)(void * comm);
typedef const char * (*Nccl_Get_Error_String)(int result);
typedef int (*Nccl_Get_Version)(int * version);
enum { NCCL_FLOAT32 = 7, NCCL_SUM = 0 };                                            /* ncclFloat32, ncclSum */
enum { FN_UNIQUE_ID, FN_INIT_RANK, FN_ALL_REDUCE, FN_DESTROY, FN_ERROR_STRING, FN_VERSION };

static int load_nccl(void ** lib_out, void * fn[6]) {
	static const char * const names[6] = {"ncclGetUniqueId", "ncclCommInitRank", "ncclAllReduce", "ncclCommDestroy", "ncclGetErrorString", "ncclGetVersion"};
	void * lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);          /* the copy already in the process, if any */
	if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
	if (!lib) { fprintf(stderr, "Error: exchange: cannot load libnccl.so.2 (%s)\n", dlerror()); return -1; }
	for (int i = 0; i < 6; i++) {
		fn[i] = dlsym(lib, names[i]);
		if (!fn[i]) { fprintf(stderr, "Error: exchange: libnccl.so.2 lacks %s\n", names[i]); dlclose(lib); return -1; }
	}
	*lib_out = lib;
	return 0;
}

static const char * nccl_error(void * fn[6], int result) { return ((Nccl_Get_Error_String) fn[FN_ERROR_STRING])(result); }

int dataflow_exchange_unique_id(uint8_t id[DATAFLOW_EXCHANGE_ID_BYTES]) {
	void * lib, * fn[6];
	if (!id || load_nccl(&lib, fn)) return -1;
	Nccl_Unique_Id uid;
	const int r = ((Nccl_Get_Unique_Id) fn[FN_UNIQUE_ID])(&uid);
	if (r) { fprintf(stderr, "Error: exchange: ncclGetUniqueId failed: %s\n", nccl_error(fn, r)); return -1; }
	memcpy(id, uid.internal, DATAFLOW_EXCHANGE_ID_BYTES);
	return 0;
}

int dataflow_exchange_init(Dataflow_Exchange * exchange, Dataflow_Handle * handle, int world_size, int rank,
                           const uint8_t id[DATAFLOW_EXCHANGE_ID_BYTES]) {
	if (!exchange || !handle || world_size < 1 || rank < 0 || rank >= world_size) {
		fprintf(stderr, "Error: exchange: bad arguments (world size %d, rank %d)\n", world_size, rank);
		return -1;
	}
	memset(exchange, 0, sizeof(*exchange));
	exchange->handle = handle;
	exchange->world_size = world_size;
	exchange->rank = rank;
	if (world_size == 1) return 0;
	if (!id) { fprintf(stderr, "Error: exchange: a world of %d ranks needs the unique id made by rank 0\n", world_size); return -1; }
	if (load_nccl(&exchange->nccl_lib, exchange->fn)) return -1;
	cudaError_t e = cudaSetDevice(handle->device_id);
	if (e != cudaSuccess) { fprintf(stderr, "Error: exchange: cannot make device %d current: %s\n", handle->device_id, cudaGetErrorString(e)); cudaGetLastError(); return -1; }
	Nccl_Unique_Id uid;
	memcpy(uid.internal, id, DATAFLOW_EXCHANGE_ID_BYTES);
	const int r = ((Nccl_Comm_Init_Rank) exchange->fn[FN_INIT_RANK])(&exchange->comm, world_size, uid, rank);
	if (r || !exchange->comm) {
		fprintf(stderr, "Error: exchange: ncclCommInitRank failed on rank %d of %d: %s\n", rank, world_size, nccl_error(exchange->fn, r));
		exchange->comm = NULL;
		return -1;
	}
	return 0;
}

int dataflow_exchange_all_reduce_f32(Dataflow_Exchange * exchange, int stream_id, float * packed, uint64_t count) {
	if (!exchange || !exchange->handle) { fprintf(stderr, "Error: exchange: not initialised\n"); return -1; }
	if (exchange->world_size == 1 || count == 0) return 0;
	Dataflow_Handle * h = exchange->handle;
	if (!packed || !exchange->comm) { fprintf(stderr, "Error: exchange: NULL buffer or communicator\n"); return -1; }
	if (stream_id != -1 && (stream_id < 0 || stream_id >= h->num_streams)) {
		fprintf(stderr, "Error: exchange: stream id %d, when the handle has %d streams\n", stream_id, h->num_streams);
		return -1;
	}
	void * stream = stream_id == -1 ? NULL : ((void **) h->streams)[stream_id];
	const int r = ((Nccl_All_Reduce) exchange->fn[FN_ALL_REDUCE])(packed, packed, (size_t) count, NCCL_FLOAT32, NCCL_SUM, exchange->comm, stream);
	if (r) { fprintf(stderr, "Error: exchange: ncclAllReduce of %lu floats failed: %s\n", (unsigned long) count, nccl_error(exchange->fn, r)); return -1; }
	return 0;
}

void dataflow_exchange_destroy(Dataflow_Exchange * exchange) {
	if (!exchange) return;
	if (exchange->comm && exchange->fn[FN_DESTROY]) ((Nccl_Comm_Destroy) exchange->fn[FN_DESTROY])(exchange->comm);
	memset(exchange, 0, sizeof(*exchange));
}
