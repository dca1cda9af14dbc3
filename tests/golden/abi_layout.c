/* Prints sizeof/offsetof of the ABI structs as JSON. Compiled twice: against the reference's headers
 * (-DUSE_REFERENCE_HEADERS, by make_fingerprints.py, where the reference tree is mounted) and against
 * include/dataflow_abi.h (by the CPU tests); the two outputs must be identical. */
#include <stddef.h>
#include <stdio.h>
#ifdef USE_REFERENCE_HEADERS
#include "cuda_dataflow_handle.h"
#else
#include "dataflow_abi.h"
#endif

#define SZ(T) printf("  \"sizeof(" #T ")\": %zu,\n", sizeof(T))
#define OFF(T, f) printf("  \"offsetof(" #T "," #f ")\": %zu,\n", offsetof(T, f))

int main(void) {
	printf("{\n");
	SZ(Op_Skeleton_Header); SZ(Op_Identifier); SZ(Op_Skeleton); SZ(Op);
	OFF(Op_Skeleton_Header, num_args); OFF(Op_Skeleton_Header, arg_dtypes); OFF(Op_Skeleton, identifier); OFF(Op, op_args);
	SZ(Table_Config); SZ(Table); OFF(Table, config); OFF(Table, is_empty_bit_vector); OFF(Table, items);
	OFF(Table_Config, hash_func); OFF(Table_Config, key_size_bytes); OFF(Table_Config, value_size_bytes);
	SZ(Dataflow_Handle);
	OFF(Dataflow_Handle, device_id); OFF(Dataflow_Handle, device_handle); OFF(Dataflow_Handle, device_info); OFF(Dataflow_Handle, ctx_id);
	OFF(Dataflow_Handle, ctx); OFF(Dataflow_Handle, num_streams); OFF(Dataflow_Handle, streams); OFF(Dataflow_Handle, stream_prios);
	OFF(Dataflow_Handle, stream_names); OFF(Dataflow_Handle, stream_states); OFF(Dataflow_Handle, num_native_function_libs);
	OFF(Dataflow_Handle, native_function_libs); OFF(Dataflow_Handle, num_ops); OFF(Dataflow_Handle, op_table);
	OFF(Dataflow_Handle, register_native_code); OFF(Dataflow_Handle, register_external_code); OFF(Dataflow_Handle, submit_op);
	OFF(Dataflow_Handle, submit_host_op); OFF(Dataflow_Handle, get_stream_state); OFF(Dataflow_Handle, submit_dependency);
	OFF(Dataflow_Handle, sync_stream); OFF(Dataflow_Handle, sync_handle); OFF(Dataflow_Handle, alloc_mem); OFF(Dataflow_Handle, free_mem);
	OFF(Dataflow_Handle, set_mem); OFF(Dataflow_Handle, enable_access_to_host_mem); OFF(Dataflow_Handle, disable_access_to_host_mem);
	OFF(Dataflow_Handle, enable_access_to_peer_mem); OFF(Dataflow_Handle, disable_access_to_peer_mem);
	OFF(Dataflow_Handle, submit_inbound_transfer); OFF(Dataflow_Handle, submit_outbound_transfer); OFF(Dataflow_Handle, submit_peer_transfer);
	SZ(Cuda_Device_Info); OFF(Cuda_Device_Info, arch_num); OFF(Cuda_Device_Info, sm_count); OFF(Cuda_Device_Info, optin_max_smem_per_block);
	OFF(Cuda_Device_Info, host_numa_id);
	SZ(Cuda_Function_Config); SZ(Cuda_Launch_Config); OFF(Cuda_Launch_Config, sharedMemBytes);
	SZ(Cuda_Function); OFF(Cuda_Function, is_native); OFF(Cuda_Function, function_handle); OFF(Cuda_Function, set_launch_config);
	OFF(Cuda_Function, cuda_external_func); OFF(Cuda_Function, op_extra); OFF(Cuda_Function, op_skeleton);
	printf("  \"DATAFLOW_BOOL_SCALAR\": %d, \"COMPUTE_LEVEL_ZERO\": %d, \"MAX_OP_ARGS\": %d, \"MAX_STREAMS\": %d\n",
	       (int) DATAFLOW_BOOL_SCALAR, (int) COMPUTE_LEVEL_ZERO, MAX_OP_ARGS, MAX_STREAMS);
	printf("}\n");
	return 0;
}
