/*
 * dataflow_abi.h -- binary layout shared between callers, the handle and op plug-ins.
 *
 * Every type in this file is laid out byte-for-byte like the type of the same name in
 * als244/dataflow_lib, so that code written against that library (its submit_* callers,
 * its external-op plug-ins, its launch-config objects) links and runs against this one:
 *
 *   DataflowDatatype                      src/datatype/include/dataflow_datatype.h:7-36
 *   Op_Skeleton_Header / Op_Identifier /
 *   Op_Skeleton / Op                      src/ops/include/ops.h:6-35        (388/32/420/680 B)
 *   Table_Config / Table                  src/table/include/table.h:28-69
 *   ComputeType / Dataflow_Handle         src/dataflow_handle/include/dataflow_handle.h:17-122
 *   External_Lib_Func(_Init)              src/dataflow_handle/include/dataflow_handle.h:131,136
 *   Cuda_Device_Info / Cuda_Function_Config /
 *   Cuda_Launch_Config / Cuda_Function    src/dataflow_handle/nvidia/include/cuda_dataflow_handle.h:15-62
 *
 * The enumerator ORDER of DataflowDatatype is part of an op's identity: the values are
 * hashed (SHA-256 over the 388-byte skeleton header) to form the registry key.
 */
#ifndef DATAFLOW_ABI_H
#define DATAFLOW_ABI_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ datatypes */

typedef enum {
	DATAFLOW_NONE, DATAFLOW_VOID,
	DATAFLOW_FP64, DATAFLOW_FP32, DATAFLOW_FP16, DATAFLOW_BF16, DATAFLOW_FP8E4M3, DATAFLOW_FP8E5M2,
	DATAFLOW_UINT64, DATAFLOW_UINT32, DATAFLOW_UINT16, DATAFLOW_UINT8,
	DATAFLOW_LONG, DATAFLOW_INT, DATAFLOW_BOOL,
	DATAFLOW_FP64_SCALAR, DATAFLOW_FP32_SCALAR, DATAFLOW_FP16_SCALAR, DATAFLOW_BF16_SCALAR,
	DATAFLOW_FP8E4M3_SCALAR, DATAFLOW_FP8E5M2_SCALAR,
	DATAFLOW_UINT64_SCALAR, DATAFLOW_UINT32_SCALAR, DATAFLOW_UINT16_SCALAR, DATAFLOW_UINT8_SCALAR,
	DATAFLOW_LONG_SCALAR, DATAFLOW_INT_SCALAR, DATAFLOW_BOOL_SCALAR
} DataflowDatatype;

/* ------------------------------------------------------------------ op identity */

#define MAX_OP_ARGS 32
#define MAX_OP_NICKNAME_SIZE 255
#define OP_IDENTIFIER_FINGERPRINT_TYPE 0      /* SHA-256 */
#define OP_IDENTIFIER_FINGERPRINT_NUM_BYTES 32

typedef struct op_skeleton_header {
	char op_nickname[MAX_OP_NICKNAME_SIZE + 1];   /* "<op>_<DTYPE>[_<DTYPE>]", NUL padded */
	int num_args;
	DataflowDatatype arg_dtypes[MAX_OP_ARGS];     /* unused slots hold DATAFLOW_NONE */
} Op_Skeleton_Header;

typedef struct op_identifier {
	uint8_t fingerprint[OP_IDENTIFIER_FINGERPRINT_NUM_BYTES];
} Op_Identifier;

typedef struct Op_Skeleton {
	Op_Skeleton_Header header;
	Op_Identifier identifier;                     /* SHA-256 of `header` */
} Op_Skeleton;

/* One submission. op_args[i] points at the VALUE of argument i (an int, a float, a
 * uint64_t or a device-pointer variable) and is only valid for the duration of submit_op. */
typedef struct op {
	Op_Skeleton op_skeleton;
	void * op_args[MAX_OP_ARGS];
} Op;

/* ------------------------------------------------------------------ hash table */

typedef int (*Item_Cmp)(void * item, void * other_item);
typedef uint64_t (*Hash_Func)(void * item, uint64_t table_size);

typedef struct table_config {
	uint64_t min_size;
	uint64_t max_size;
	float load_factor;      /* grow when cnt > size * load_factor (and size < max_size) */
	float shrink_factor;    /* shrink when cnt < size * shrink_factor (and size > min_size) */
	Hash_Func hash_func;
	uint64_t key_size_bytes;
	uint64_t value_size_bytes;
} Table_Config;

typedef struct table {
	uint64_t cnt;
	uint64_t size;
	Table_Config config;
	uint64_t * is_empty_bit_vector;   /* bit i set <=> slot i is free */
	void * items;                     /* size * (key_size_bytes + value_size_bytes) */
} Table;

/* ------------------------------------------------------------------ handle */

#define OP_TABLE_MIN_SIZE 1UL << 10
#define OP_TABLE_MAX_SIZE 1UL << 20
#define MAX_NATIVE_FUNCTION_LIBS 1024
#define MAX_STREAMS 256
#define FUNC_SYMBOL_MAX_LEN 512

typedef enum compute_type {
	COMPUTE_NONE, COMPUTE_CPU, COMPUTE_CUDA, COMPUTE_HSA, COMPUTE_LEVEL_ZERO
} ComputeType;

typedef struct dataflow_handle Dataflow_Handle;

struct dataflow_handle {
	ComputeType compute_type;
	int device_id;
	void * device_handle;       /* CUdevice *            */
	void * device_info;         /* Cuda_Device_Info *    */
	int ctx_id;
	void * ctx;                 /* CUcontext * (the device's primary context here) */
	int num_streams;
	void * streams;             /* CUstream[num_streams]; a CUstream is also a cudaStream_t */
	int stream_prios[MAX_STREAMS];
	char * stream_names[MAX_STREAMS];
	void * stream_states;       /* CUevent[num_streams]  */

	int num_native_function_libs;
	void * native_function_libs[MAX_NATIVE_FUNCTION_LIBS];

	int num_ops;
	Table op_table;             /* fingerprint[32] -> Cuda_Function */

	/* ops */
	int (*register_native_code)(Dataflow_Handle * dataflow_handle, char * native_code_filename, char * native_code_config_lib_filename,
								int num_funcs, Op_Skeleton * func_op_skeletons, char ** func_symbols, char ** func_set_launch_symbols, char ** func_init_symbols);
	int (*register_external_code)(Dataflow_Handle * dataflow_handle, char * external_code_filename, int num_funcs,
								Op_Skeleton * func_op_skeletons, char ** func_symbols, char ** func_init_symbols);
	/* compute */
	int (*submit_op)(Dataflow_Handle * dataflow_handle, Op * op, int stream_id);
	int (*submit_host_op)(Dataflow_Handle * dataflow_handle, void * host_func, void * host_func_arg, int stream_id);
	/* dependencies */
	void * (*get_stream_state)(Dataflow_Handle * dataflow_handle, int stream_id);
	int (*submit_dependency)(Dataflow_Handle * dataflow_handle, int stream_id, void * other_stream_state);
	int (*sync_stream)(Dataflow_Handle * dataflow_handle, int stream_id);
	int (*sync_handle)(Dataflow_Handle * dataflow_handle);
	/* memory */
	void * (*alloc_mem)(Dataflow_Handle * dataflow_handle, uint64_t size_bytes);
	void (*free_mem)(Dataflow_Handle * dataflow_handle, void * dev_ptr);
	int (*set_mem)(Dataflow_Handle * dataflow_handle, int stream_id, void * dev_ptr, uint8_t val, uint64_t size_bytes);
	int (*enable_access_to_host_mem)(Dataflow_Handle * dataflow_handle, void * host_ptr, uint64_t size_bytes, unsigned int flags);
	int (*disable_access_to_host_mem)(Dataflow_Handle * dataflow_handle, void * host_ptr);
	int (*enable_access_to_peer_mem)(Dataflow_Handle * dataflow_handle, Dataflow_Handle * peer_dataflow_handle);
	int (*disable_access_to_peer_mem)(Dataflow_Handle * dataflow_handle, Dataflow_Handle * peer_dataflow_handle);
	/* transfers */
	int (*submit_inbound_transfer)(Dataflow_Handle * dataflow_handle, int stream_id, void * dev_dest, void * host_src, uint64_t size_bytes);
	int (*submit_outbound_transfer)(Dataflow_Handle * dataflow_handle, int stream_id, void * host_dest, void * dev_src, uint64_t size_bytes);
	int (*submit_peer_transfer)(Dataflow_Handle * dataflow_handle, int stream_id, void * dev_dest, void * dev_src, uint64_t size_bytes);
};

/* Plug-in entry points of an external (shared-object) op. `op_table_value` is the
 * Cuda_Function about to be inserted; an init function may set its `op_extra`. */
typedef int (*External_Lib_Func_Init)(Dataflow_Handle * dataflow_handle, void * op_table_value);
typedef int (*External_Lib_Func)(Dataflow_Handle * dataflow_handle, int stream_id, Op * op, void * op_extra);

/* ------------------------------------------------------------------ CUDA backend records */

#define CUDA_DEFAULT_STREAM_PRIO 0
#define CUDA_DEV_UPPER_BOUND_MAX_THREADS_ALL_FUNC 1024

typedef struct cuda_device_info {
	size_t total_mem;
	int arch_num;                    /* 10 * major + minor, 100 on B200 */
	int sm_count;
	int max_threads_per_block;
	int max_smem_per_block;
	int optin_max_smem_per_block;
	int host_numa_id;
} Cuda_Device_Info;

typedef struct cuda_function_config {
	int func_max_smem;
	int func_max_threads_per_block;
} Cuda_Function_Config;

typedef struct cuda_launch_config {
	unsigned int gridDimX, gridDimY, gridDimZ;
	unsigned int blockDimX, blockDimY, blockDimZ;
	unsigned int sharedMemBytes;
} Cuda_Launch_Config;

typedef struct cuda_function Cuda_Function;

struct cuda_function {
	Cuda_Function_Config function_config;
	bool is_native;                  /* true: cubin kernel + launch-config callback */
	void * function_handle;          /* CUfunction */
	int (*set_launch_config)(Cuda_Launch_Config * cuda_launch_config, Dataflow_Handle * dataflow_handle, Cuda_Function * cuda_function, Op * op);
	int (*cuda_external_func)(Dataflow_Handle * dataflow_handle, int stream_id, Op * op, void * op_extra);
	void * op_extra;
	Op_Skeleton op_skeleton;
};

typedef int (*Cuda_Set_Func_Attribute)(Dataflow_Handle * dataflow_handle, Cuda_Function * cuda_function);

#ifdef __cplusplus
}
#endif
#endif
