"""Loads lib/libdataflow_b200.so (built in-tree by dataflow_lib_b200/csrc/Makefile) and declares the
C-ABI of include/dataflow_b200_kernels.h and include/dataflow_api.h. There is no fallback: a missing
library is an ImportError naming the build command."""
import ctypes as C
import os

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libdataflow_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
                      "(or python -c 'import __graft_entry__ as g; g.build()'); there is no CPU or PyTorch fallback")

lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)

_vp, _i, _f, _u64 = C.c_void_p, C.c_int, C.c_float, C.c_uint64

# name -> (restype, argtypes): every symbol include/dataflow_b200_kernels.h declares
KERNEL_ABI = {
    "dfb200_last_error": (C.c_char_p, []),
    "dfb200_target_arch": (C.c_char_p, []),
    "dfb200_sm_count": (_i, []),
    "dfb200_read_kernel_status": (_i, [_vp, _vp, _i]),
    "dfb200_selftest_bounded_wait": (_i, [_i, _vp]),
    "dfb200_rms_norm": (_i, [_i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_rms_norm_bwd_x": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_rms_norm_bwd_w_workspace_bytes": (_u64, [_i, _i]),
    "dfb200_rms_norm_bwd_w": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "dfb200_rms_norm_bwd_w_sums": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "dfb200_rms_norm_bwd_x_w": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "dfb200_rms_norm_bwd_x_w_sums": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "dfb200_rms_norm_bwd_w_static": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_rope": (_i, [_i, _u64, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "dfb200_rope_bwd_x": (_i, [_i, _u64, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu_bwd_x": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_softmax": (_i, [_i, _i, _i, _i, _vp, _vp, _vp]),
    "dfb200_cross_entropy_loss": (_i, [_i, _i, _i, _vp, _vp, _vp]),
    "dfb200_quantize_rows_e4m3": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_transpose_bytes": (_i, [_i, _i, _vp, _i, _vp, _i, _vp]),
    "dfb200_gemm_e4m3": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_gemm_e4m3_swiglu": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu_quantize_rows_e4m3": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu_bwd_quantize_rows_e4m3": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_col_amax_bf16": (_i, [_i, _i, _vp, _vp, _vp]),
    "dfb200_transpose_quantize_e4m3": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu_ffn_fp8_wgrad_workspace_bytes": (_u64, [_i, _i, _i]),
    "dfb200_swiglu_ffn_fp8_wgrad": (_i, [_i, _i, _i] + [_vp] * 9 + [_u64, _vp]),
    "dfb200_gemm_e4m3_swiglu_bwd": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu_ffn_fp8_workspace_bytes": (_u64, [_i, _i, _i]),
    "dfb200_swiglu_ffn_fp8": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "dfb200_ffn_fp8_prepare_bwd_weights": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_swiglu_ffn_fp8_bwd": (_i, [_i, _i, _i] + [_vp] * 10 + [_u64, _vp]),
    "dfb200_softmax_fp32_out": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "dfb200_embedding": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "dfb200_copy_to_seq_context": (_i, [_i, _u64, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_select_experts": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dfb200_softmax_cross_entropy_workspace_bytes": (_u64, [_i, _i]),
    "dfb200_softmax_cross_entropy": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
}

_H = C.POINTER(abi.DataflowHandleStruct)
_SK = C.POINTER(abi.OpSkeleton)

# host entry points of include/dataflow_api.h
HOST_ABI = {
    "dataflow_sizeof_element": (C.c_size_t, [_i]),
    "dataflow_datatype_as_string": (C.c_char_p, [_i]),
    "dataflow_convert_datatype": (_i, [_vp, _vp, _i, _i, C.c_long, _i]),
    "solo_bf16_to_fp32": (_f, [C.c_uint16]),
    "solo_fp32_to_bf16": (C.c_uint16, [_f]),
    "solo_fp16_to_fp32": (_f, [C.c_uint16]),
    "solo_fp32_to_fp16": (C.c_uint16, [_f]),
    "solo_fp16_to_bf16": (C.c_uint16, [C.c_uint16]),
    "solo_bf16_to_fp16": (C.c_uint16, [C.c_uint16]),
    "dataflow_sha256": (None, [_vp, _u64, _vp]),
    "do_fingerprinting": (None, [_vp, _u64, _vp, _i]),
    "fingerprint_to_least_sig64": (_u64, [_vp, _i]),
    "get_fingerprint_num_bytes": (C.c_uint8, [_i]),
    "get_fingerprint_type_name": (C.c_char_p, [_i]),
    "print_hex": (None, [_vp, _i]),
    "print_sha256": (None, [_vp]),
    "init_table": (_i, [_vp, _vp, _u64, _u64, _u64, _u64, _f, _f]),
    "destroy_table": (None, [_vp]),
    "insert_table": (_i, [_vp, _vp, _vp]),
    "find_table": (C.c_long, [_vp, _vp, C.c_bool, _vp]),
    "remove_table": (_i, [_vp, _vp, _vp]),
    "init_cuda_dataflow_handle": (_i, [_H, _i, _i, _i, C.c_uint, _i, C.POINTER(_i), C.POINTER(C.c_char_p)]),
    "destroy_cuda_dataflow_handle": (None, [_H]),
    "register_native_ops": (_i, [_H, C.c_char_p, C.c_char_p]),
    "set_native_op_skeleton": (_i, [_SK, C.c_char_p, _i, _i]),
    "set_native_embedding_skeleton": (None, [_SK, _i]),
    "set_native_rms_norm_skeleton": (None, [_SK, _i]),
    "set_native_rms_norm_bwd_x_skeleton": (None, [_SK, _i, _i]),
    "set_native_rms_norm_bwd_w_skeleton": (None, [_SK, _i, _i]),
    "set_native_rms_norm_bwd_w_sums_skeleton": (None, [_SK, _i, _i]),
    "set_native_rms_norm_bwd_x_w_skeleton": (None, [_SK, _i, _i]),
    "set_native_rms_norm_bwd_x_w_sums_skeleton": (None, [_SK, _i, _i]),
    "set_native_rope_skeleton": (None, [_SK, _i]),
    "set_native_rope_bwd_x_skeleton": (None, [_SK, _i]),
    "set_native_copy_to_seq_context_skeleton": (None, [_SK, _i]),
    "set_native_swiglu_skeleton": (None, [_SK, _i]),
    "set_native_swiglu_bwd_x_skeleton": (None, [_SK, _i, _i]),
    "set_native_softmax_skeleton": (None, [_SK, _i, _i]),
    "set_native_cross_entropy_loss_skeleton": (None, [_SK, _i]),
    "set_native_softmax_cross_entropy_skeleton": (None, [_SK, _i, _i]),
    "set_native_select_experts_skeleton": (None, [_SK, _i]),
    "set_native_softmax_argmax_skeleton": (None, [_SK, _i]),
    "set_native_swiglu_ffn_fp8_skeleton": (None, [_SK]),
    "set_native_swiglu_ffn_fp8_bwd_skeleton": (None, [_SK]),
    "submit_swiglu_ffn_fp8": (_i, [_H, _i, _i, _i, _i] + [_vp] * 11),
    "submit_swiglu_ffn_fp8_bwd": (_i, [_H, _i, _i, _i, _i] + [_vp] * 8),
    "submit_softmax_argmax": (_i, [_H, _i, _i, _i, _i, _vp, _vp, _vp]),
    "submit_embedding": (_i, [_H, _i, _i, _i, _i, _vp, _vp, _vp]),
    "submit_copy_to_seq_context": (_i, [_H, _i, _i, _u64, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "submit_select_experts": (_i, [_H, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "submit_rms_norm": (_i, [_H, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp]),
    "submit_rms_norm_bwd_x": (_i, [_H, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp]),
    "submit_rms_norm_bwd_w": (_i, [_H, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp]),
    "submit_rms_norm_bwd_w_sums": (_i, [_H, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp]),
    "submit_rms_norm_bwd_x_w": (_i, [_H, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "submit_rms_norm_bwd_x_w_sums": (_i, [_H, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "submit_rope": (_i, [_H, _i, _i, _u64, _i, _i, _i, _i, _vp, _vp, _vp]),
    "submit_rope_bwd_x": (_i, [_H, _i, _i, _u64, _i, _i, _i, _i, _vp, _vp, _vp]),
    "submit_swiglu": (_i, [_H, _i, _i, _i, _i, _vp, _vp, _vp]),
    "submit_swiglu_bwd_x": (_i, [_H, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "submit_softmax": (_i, [_H, _i, _i, _i, _i, _i, _vp, _vp]),
    "submit_cross_entropy_loss": (_i, [_H, _i, _i, _i, _i, _vp, _vp]),
    "submit_softmax_cross_entropy": (_i, [_H, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "set_external_matmul_skeleton": (None, [_SK]),
    "set_external_flash3_attention_fwd_skeleton": (None, [_SK]),
    "set_external_flash3_attention_bwd_skeleton": (None, [_SK]),
    "submit_matmul": (_i, [_H, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _u64, _vp]),
    "submit_attention": (_i, [_H, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "submit_attention_bwd": (_i, [_H, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i] + [_vp] * 9 + [_u64, _vp]),
    "submit_transformer_head": (_i, [_H, _i, _i, C.POINTER(abi.TransformerBlockTransition), C.POINTER(abi.TransformerHead),
                                    C.POINTER(abi.TransformerHeadActivations), C.POINTER(abi.TransformerModelOutput),
                                    C.POINTER(abi.TransformerHead), C.POINTER(abi.TransformerHeadActivations),
                                    C.POINTER(abi.TransformerBlockTransition), C.POINTER(abi.TransformerBlockTransition)]),
    "submit_transformer_block": (_i, [_H, _i, _i, C.POINTER(abi.TransformerBlockTransition), C.POINTER(abi.TransformerBlock),
                                     C.POINTER(abi.TransformerBlockActivations), C.POINTER(abi.TransformerBlockTransition)]),
    "submit_transformer_block_bwd_x": (_i, [_H, _i, _i, C.POINTER(abi.TransformerBlock), C.POINTER(abi.TransformerBlockTransition),
                                           C.POINTER(abi.TransformerBlockActivations), C.POINTER(abi.TransformerBlockTransition),
                                           C.POINTER(abi.TransformerBlockActivations), C.POINTER(abi.TransformerBlock),
                                           C.POINTER(abi.TransformerBlockTransition)]),
    "submit_transformer_block_bwd_w": (_i, [_H, _i, C.POINTER(abi.TransformerBlockTransition), C.POINTER(abi.TransformerBlockActivations),
                                           C.POINTER(abi.TransformerBlockActivations), C.POINTER(abi.TransformerBlock)]),
    # include/dataflow_b200_exchange.h
    "dataflow_exchange_unique_id": (_i, [_vp]),
    "dataflow_exchange_init": (_i, [C.POINTER(abi.DataflowExchange), _H, _i, _i, _vp]),
    "dataflow_exchange_all_reduce_f32": (_i, [C.POINTER(abi.DataflowExchange), _i, _vp, _u64]),
    "dataflow_exchange_destroy": (None, [C.POINTER(abi.DataflowExchange)]),
    # external-op plug-in symbols (ops_external.c)
    "dataflow_b200_workspace_init": (_i, [_H, _vp]),
    "dataflow_b200_reserve_workspace": (_i, [_H, _SK, _i, _u64]),
    "dataflow_b200_workspace_release": (None, [_vp]),
    "dataflow_b200_rms_norm": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rms_norm_bwd_x": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rms_norm_bwd_w": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rms_norm_bwd_w_sums": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rms_norm_bwd_x_w": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rms_norm_bwd_x_w_sums": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rope": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_rope_bwd_x": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_swiglu": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_swiglu_bwd_x": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_softmax": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_cross_entropy_loss": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_softmax_cross_entropy": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_embedding": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_copy_to_seq_context": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_select_experts": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_softmax_argmax": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_swiglu_ffn_fp8": (_i, [_H, _i, _vp, _vp]),
    "dataflow_b200_swiglu_ffn_fp8_bwd": (_i, [_H, _i, _vp, _vp]),
}

for _table in (KERNEL_ABI, HOST_ABI):
    for _name, (_res, _args) in _table.items():
        _fnp = getattr(lib, _name)          # AttributeError here = the library does not export a declared symbol
        _fnp.restype = _res
        _fnp.argtypes = _args


def last_error() -> str:
    return lib.dfb200_last_error().decode()
