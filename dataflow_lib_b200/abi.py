"""ctypes mirror of include/dataflow_abi.h (layouts of als244/dataflow_lib: src/ops/include/ops.h:6-35,
src/dataflow_handle/include/dataflow_handle.h:28-122, src/table/include/table.h:28-69,
src/dataflow_handle/nvidia/include/cuda_dataflow_handle.h:15-59)."""
import ctypes as C
import enum


class DataflowDatatype(enum.IntEnum):
    NONE = 0
    VOID = 1
    FP64 = 2
    FP32 = 3
    FP16 = 4
    BF16 = 5
    FP8E4M3 = 6
    FP8E5M2 = 7
    UINT64 = 8
    UINT32 = 9
    UINT16 = 10
    UINT8 = 11
    LONG = 12
    INT = 13
    BOOL = 14
    FP64_SCALAR = 15
    FP32_SCALAR = 16
    FP16_SCALAR = 17
    BF16_SCALAR = 18
    FP8E4M3_SCALAR = 19
    FP8E5M2_SCALAR = 20
    UINT64_SCALAR = 21
    UINT32_SCALAR = 22
    UINT16_SCALAR = 23
    UINT8_SCALAR = 24
    LONG_SCALAR = 25
    INT_SCALAR = 26
    BOOL_SCALAR = 27


MAX_OP_ARGS = 32
MAX_STREAMS = 256
MAX_NATIVE_FUNCTION_LIBS = 1024
COMPUTE_CUDA = 2


class OpSkeletonHeader(C.Structure):
    _fields_ = [("op_nickname", C.c_char * 256), ("num_args", C.c_int), ("arg_dtypes", C.c_int * MAX_OP_ARGS)]


class OpIdentifier(C.Structure):
    _fields_ = [("fingerprint", C.c_uint8 * 32)]


class OpSkeleton(C.Structure):
    _fields_ = [("header", OpSkeletonHeader), ("identifier", OpIdentifier)]


class Op(C.Structure):
    _fields_ = [("op_skeleton", OpSkeleton), ("op_args", C.c_void_p * MAX_OP_ARGS)]


class TableConfig(C.Structure):
    _fields_ = [("min_size", C.c_uint64), ("max_size", C.c_uint64), ("load_factor", C.c_float), ("shrink_factor", C.c_float),
                ("hash_func", C.c_void_p), ("key_size_bytes", C.c_uint64), ("value_size_bytes", C.c_uint64)]


class Table(C.Structure):
    _fields_ = [("cnt", C.c_uint64), ("size", C.c_uint64), ("config", TableConfig),
                ("is_empty_bit_vector", C.c_void_p), ("items", C.c_void_p)]


class CudaDeviceInfo(C.Structure):
    _fields_ = [("total_mem", C.c_size_t), ("arch_num", C.c_int), ("sm_count", C.c_int), ("max_threads_per_block", C.c_int),
                ("max_smem_per_block", C.c_int), ("optin_max_smem_per_block", C.c_int), ("host_numa_id", C.c_int)]


class CudaFunction(C.Structure):
    _fields_ = [("func_max_smem", C.c_int), ("func_max_threads_per_block", C.c_int), ("is_native", C.c_bool),
                ("function_handle", C.c_void_p), ("set_launch_config", C.c_void_p), ("cuda_external_func", C.c_void_p),
                ("op_extra", C.c_void_p), ("op_skeleton", OpSkeleton)]


class DataflowHandleStruct(C.Structure):
    pass


_H = C.POINTER(DataflowHandleStruct)
_fn = C.CFUNCTYPE

DataflowHandleStruct._fields_ = [
    ("compute_type", C.c_int), ("device_id", C.c_int), ("device_handle", C.c_void_p), ("device_info", C.c_void_p),
    ("ctx_id", C.c_int), ("ctx", C.c_void_p), ("num_streams", C.c_int), ("streams", C.c_void_p),
    ("stream_prios", C.c_int * MAX_STREAMS), ("stream_names", C.c_char_p * MAX_STREAMS), ("stream_states", C.c_void_p),
    ("num_native_function_libs", C.c_int), ("native_function_libs", C.c_void_p * MAX_NATIVE_FUNCTION_LIBS),
    ("num_ops", C.c_int), ("op_table", Table),
    ("register_native_code", _fn(C.c_int, _H, C.c_char_p, C.c_char_p, C.c_int, C.POINTER(OpSkeleton), C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), C.POINTER(C.c_char_p))),
    ("register_external_code", _fn(C.c_int, _H, C.c_char_p, C.c_int, C.POINTER(OpSkeleton), C.POINTER(C.c_char_p), C.POINTER(C.c_char_p))),
    ("submit_op", _fn(C.c_int, _H, C.POINTER(Op), C.c_int)),
    ("submit_host_op", _fn(C.c_int, _H, C.c_void_p, C.c_void_p, C.c_int)),
    ("get_stream_state", _fn(C.c_void_p, _H, C.c_int)),
    ("submit_dependency", _fn(C.c_int, _H, C.c_int, C.c_void_p)),
    ("sync_stream", _fn(C.c_int, _H, C.c_int)),
    ("sync_handle", _fn(C.c_int, _H)),
    ("alloc_mem", _fn(C.c_void_p, _H, C.c_uint64)),
    ("free_mem", _fn(None, _H, C.c_void_p)),
    ("set_mem", _fn(C.c_int, _H, C.c_int, C.c_void_p, C.c_uint8, C.c_uint64)),
    ("enable_access_to_host_mem", _fn(C.c_int, _H, C.c_void_p, C.c_uint64, C.c_uint)),
    ("disable_access_to_host_mem", _fn(C.c_int, _H, C.c_void_p)),
    ("enable_access_to_peer_mem", _fn(C.c_int, _H, _H)),
    ("disable_access_to_peer_mem", _fn(C.c_int, _H, _H)),
    ("submit_inbound_transfer", _fn(C.c_int, _H, C.c_int, C.c_void_p, C.c_void_p, C.c_uint64)),
    ("submit_outbound_transfer", _fn(C.c_int, _H, C.c_int, C.c_void_p, C.c_void_p, C.c_uint64)),
    ("submit_peer_transfer", _fn(C.c_int, _H, C.c_int, C.c_void_p, C.c_void_p, C.c_uint64)),
]

assert C.sizeof(OpSkeletonHeader) == 388 and C.sizeof(OpSkeleton) == 420 and C.sizeof(Op) == 680


# ---- include/dataflow_transformer.h -------------------------------------------------------------------------------------
class EmbeddingConfig(C.Structure):
    _fields_ = [("vocab_size", C.c_int), ("embedding_size", C.c_int)]


class TransformerHead(C.Structure):
    _fields_ = [("fwd_dt", C.c_int), ("bwd_dt", C.c_int), ("compute_dt", C.c_int), ("eps", C.c_float),
                ("embedding_config", EmbeddingConfig), ("buffer", C.c_void_p), ("w_head_norm", C.c_void_p), ("w_head", C.c_void_p)]


class TransformerHeadActivations(C.Structure):
    _fields_ = [("num_tokens", C.c_int), ("buffer", C.c_void_p), ("head_norm_out", C.c_void_p), ("head_norm_weighted_sums", C.c_void_p),
                ("head_norm_rms_vals", C.c_void_p), ("head_out", C.c_void_p), ("kernel_workspace", C.c_void_p),
                ("kernel_workspaceBytes", C.c_uint64)]


class TransformerBlockTransition(C.Structure):
    _fields_ = [("batch_config", C.c_void_p), ("X", C.c_void_p)]


class TransformerModelOutput(C.Structure):
    _fields_ = [("batch_config", C.c_void_p), ("token_ids", C.c_void_p), ("labels", C.c_void_p), ("logits", C.c_void_p),
                ("loss", C.c_void_p), ("loss_avg", C.c_float)]


class SeqBatchConfig(C.Structure):
    _fields_ = [("num_seqs", C.c_int), ("total_q", C.c_int), ("total_k", C.c_int), ("seq_positions", C.c_void_p),
                ("q_seq_offsets", C.c_void_p), ("q_seq_lens", C.c_void_p), ("max_seqlen_q", C.c_int),
                ("k_seq_offsets", C.c_void_p), ("k_seq_lens", C.c_void_p), ("max_seqlen_k", C.c_int)]


class SeqBatchSavedActivations(C.Structure):
    _fields_ = [("config", C.POINTER(SeqBatchConfig)), ("buffer", C.c_void_p), ("activationBufferBytes", C.c_uint64),
                ("attn_norm_weighted_sums", C.c_void_p), ("attn_norm_rms_vals", C.c_void_p), ("x_q", C.c_void_p),
                ("x_k_local", C.c_void_p), ("x_v_local", C.c_void_p), ("softmax_lse", C.c_void_p), ("x_attn_out", C.c_void_p),
                ("x_o", C.c_void_p), ("ffn_norm_weighted_sums", C.c_void_p), ("ffn_norm_rms_vals", C.c_void_p),
                ("x_1", C.POINTER(C.c_void_p)), ("x_2", C.POINTER(C.c_void_p)), ("x_3", C.POINTER(C.c_void_p))]


class SeqBatchContext(C.Structure):
    _fields_ = [("config", C.POINTER(SeqBatchConfig)), ("buffer", C.c_void_p), ("contextBufferBytes", C.c_uint64),
                ("x_k", C.c_void_p), ("x_v", C.c_void_p)]


class SeqBatchActivationWorkspace(C.Structure):
    _fields_ = [("config", C.POINTER(SeqBatchConfig)), ("buffer", C.c_void_p), ("activationWorkspaceBytes", C.c_uint64),
                ("x_temp", C.c_void_p), ("x_temp_mlp", C.c_void_p), ("recomputed_attn_norm", C.c_void_p),
                ("recomputed_ffn_norm", C.c_void_p), ("kernel_workspace", C.c_void_p), ("kernel_workspaceBytes", C.c_uint64)]


class MoEConfig(C.Structure):
    _fields_ = [("top_k_experts", C.c_int), ("num_global_experts", C.c_int), ("num_local_experts", C.c_int), ("local_expert_inds", C.c_void_p)]


class TransformerBlockWeightOffsets(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("w_attn_norm", "w_q", "w_k", "w_v", "w_o", "w_ffn_norm", "w_router")] + \
               [("w_1", C.c_void_p), ("w_2", C.c_void_p), ("w_3", C.c_void_p)]


class TransformerBlockConfig(C.Structure):
    _fields_ = [("block_dt", C.c_int), ("compute_dt", C.c_int), ("normalization_type", C.c_int), ("attention_type", C.c_int),
                ("mlp_type", C.c_int), ("activation_type", C.c_int), ("eps", C.c_float), ("theta", C.c_int), ("num_q_heads", C.c_int),
                ("num_kv_heads", C.c_int), ("head_dim", C.c_int), ("model_dim", C.c_int), ("kv_dim", C.c_int), ("ffn_dim", C.c_int),
                ("moe_config", MoEConfig), ("pointer_alignment", C.c_int), ("weight_offsets", TransformerBlockWeightOffsets),
                ("block_raw_size", C.c_uint64), ("block_aligned_size", C.c_uint64)]


class TransformerBlock(C.Structure):
    _fields_ = [("config", TransformerBlockConfig), ("buffer", C.c_void_p), ("w_attn_norm", C.c_void_p), ("w_q", C.c_void_p),
                ("w_k", C.c_void_p), ("w_v", C.c_void_p), ("w_o", C.c_void_p), ("w_ffn_norm", C.c_void_p), ("w_router", C.c_void_p),
                ("w_1", C.POINTER(C.c_void_p)), ("w_2", C.POINTER(C.c_void_p)), ("w_3", C.POINTER(C.c_void_p))]


class TransformerBlockActivations(C.Structure):
    _fields_ = [("block", C.POINTER(TransformerBlock)), ("batch_config", C.POINTER(SeqBatchConfig)),
                ("saved_activations", C.POINTER(SeqBatchSavedActivations)), ("context", C.POINTER(SeqBatchContext)),
                ("activation_workspace", C.POINTER(SeqBatchActivationWorkspace))]


# ---- include/dataflow_b200_exchange.h -----------------------------------------------------------------------------------------
EXCHANGE_ID_BYTES = 128


class DataflowExchange(C.Structure):
    _fields_ = [("handle", C.POINTER(DataflowHandleStruct)), ("world_size", C.c_int), ("rank", C.c_int), ("comm", C.c_void_p),
                ("nccl_lib", C.c_void_p), ("fn", C.c_void_p * 6)]
