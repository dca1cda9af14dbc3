"""Dataflow_Handle through the C host API (include/dataflow_api.h): the same calls a C program written
for als244/dataflow_lib makes -- init_cuda_dataflow_handle, register_native_ops, submit_*, the handle's
function-pointer table for streams, memory and transfers (src/dataflow_handle/include/dataflow_handle.h:72-118)."""
import ctypes as C

from . import _lib, abi
from .abi import DataflowDatatype as DT

_L = _lib.lib


def _p(x):
    """device/host pointer from an int, None, or anything with data_ptr()."""
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return int(x)


class DataflowHandle:
    def __init__(self, device_id=0, num_streams=2, ctx_id=0, ctx_flags=0, stream_prios=None, stream_names=None, register_ops=True):
        self.h = abi.DataflowHandleStruct()
        prios = (C.c_int * num_streams)(*stream_prios) if stream_prios else None
        names = (C.c_char_p * num_streams)(*[n.encode() for n in stream_names]) if stream_names else None
        rc = _L.init_cuda_dataflow_handle(C.byref(self.h), abi.COMPUTE_CUDA, device_id, ctx_id, ctx_flags, num_streams, prios, names)
        if rc != 0:
            raise RuntimeError("init_cuda_dataflow_handle failed (see stderr)")
        self.num_registered = 0
        if register_ops:
            self.num_registered = self.register_native_ops()

    # -- registry -------------------------------------------------------------------------------
    def register_native_ops(self, code_path=None, config_path=None):
        n = _L.register_native_ops(C.byref(self.h), code_path.encode() if code_path else None, config_path.encode() if config_path else None)
        if n < 0:
            raise RuntimeError("register_native_ops failed (see stderr)")
        return n

    def register_native_code(self, cubin_path, config_lib_path, skeletons, symbols, launch_symbols, init_symbols):
        """handle->register_native_code: a cubin plus a shared object of launch-config callbacks."""
        n = len(skeletons)
        sk = (abi.OpSkeleton * n)(*skeletons)
        to_arr = lambda xs: (C.c_char_p * n)(*[x.encode() if x else None for x in xs])
        return self.h.register_native_code(C.byref(self.h), cubin_path.encode(), config_lib_path.encode(), n, sk,
                                           to_arr(symbols), to_arr(launch_symbols), to_arr(init_symbols))

    def register_external_code(self, lib_path, skeletons, symbols, init_symbols):
        """handle->register_external_code: plug-in functions (External_Lib_Func) from a shared object, e.g. the reference's cuBLASLt matmul."""
        n = len(skeletons)
        sk = (abi.OpSkeleton * n)(*skeletons)
        to_arr = lambda xs: (C.c_char_p * n)(*[x.encode() if x else None for x in xs])
        return self.h.register_external_code(C.byref(self.h), lib_path.encode(), n, sk, to_arr(symbols), to_arr(init_symbols))

    def reserve_workspace(self, op_name, stream_id, nbytes, fwd_dt=DT.NONE, bwd_dt=DT.NONE):
        """dataflow_b200_reserve_workspace: size the scratch block of (op identity, stream) ahead of the step loop."""
        sk = abi.OpSkeleton()
        if _L.set_native_op_skeleton(C.byref(sk), op_name.encode(), int(fwd_dt), int(bwd_dt)) != 0:
            raise ValueError(f"unknown op {op_name}")
        return _L.dataflow_b200_reserve_workspace(C.byref(self.h), C.byref(sk), stream_id, nbytes)

    @property
    def device_info(self):
        return C.cast(self.h.device_info, C.POINTER(abi.CudaDeviceInfo)).contents

    def stream_ptr(self, stream_id):
        return C.cast(self.h.streams, C.POINTER(C.c_void_p))[stream_id]

    # -- streams / memory / transfers -------------------------------------------------------------
    def sync_stream(self, stream_id): return self.h.sync_stream(C.byref(self.h), stream_id)
    def sync_handle(self): return self.h.sync_handle(C.byref(self.h))
    def get_stream_state(self, stream_id): return self.h.get_stream_state(C.byref(self.h), stream_id)
    def submit_dependency(self, stream_id, state): return self.h.submit_dependency(C.byref(self.h), stream_id, state)
    def alloc_mem(self, nbytes): return self.h.alloc_mem(C.byref(self.h), nbytes)
    def free_mem(self, ptr): self.h.free_mem(C.byref(self.h), ptr)
    def set_mem(self, stream_id, ptr, val, nbytes): return self.h.set_mem(C.byref(self.h), stream_id, _p(ptr), val, nbytes)
    def enable_access_to_host_mem(self, ptr, nbytes, flags=0): return self.h.enable_access_to_host_mem(C.byref(self.h), _p(ptr), nbytes, flags)
    def disable_access_to_host_mem(self, ptr): return self.h.disable_access_to_host_mem(C.byref(self.h), _p(ptr))
    def submit_inbound_transfer(self, stream_id, dev_dst, host_src, nbytes): return self.h.submit_inbound_transfer(C.byref(self.h), stream_id, _p(dev_dst), _p(host_src), nbytes)
    def submit_outbound_transfer(self, stream_id, host_dst, dev_src, nbytes): return self.h.submit_outbound_transfer(C.byref(self.h), stream_id, _p(host_dst), _p(dev_src), nbytes)
    def submit_peer_transfer(self, stream_id, dev_dst, dev_src, nbytes): return self.h.submit_peer_transfer(C.byref(self.h), stream_id, _p(dev_dst), _p(dev_src), nbytes)

    # -- ops (the reference's submit_* signatures; datatypes are DataflowDatatype values) -----------
    def submit_rms_norm(self, stream_id, fwd_dt, n_rows, n_cols, eps, rms_weight, X, out, weighted_sums, rms_vals):
        return _L.submit_rms_norm(C.byref(self.h), stream_id, int(fwd_dt), n_rows, n_cols, eps, _p(rms_weight), _p(X), _p(out), _p(weighted_sums), _p(rms_vals))

    def submit_rms_norm_bwd_x(self, stream_id, fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX):
        return _L.submit_rms_norm_bwd_x(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), n_rows, n_cols, eps, _p(fwd_weighted_sums),
                                        _p(fwd_rms_vals), _p(rms_weight), _p(X_inp), _p(upstream_dX), _p(dX))

    def submit_rms_norm_bwd_w(self, stream_id, fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, dW):
        return _L.submit_rms_norm_bwd_w(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), n_rows, n_cols, eps, _p(fwd_rms_vals), _p(X_inp), _p(upstream_dX), _p(dW))

    def submit_rms_norm_bwd_w_sums(self, stream_id, fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, column_sums):
        return _L.submit_rms_norm_bwd_w_sums(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), n_rows, n_cols, eps, _p(fwd_rms_vals), _p(X_inp),
                                             _p(upstream_dX), _p(column_sums))

    def submit_rms_norm_bwd_x_w(self, stream_id, fwd_dt, bwd_dt, n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, dW,
                                sums=False):
        """rms_norm_bwd_x and rms_norm_bwd_w in one pass; sums=True: dW is the fp32 column-sums array of submit_rms_norm_bwd_w_sums."""
        fn = _L.submit_rms_norm_bwd_x_w_sums if sums else _L.submit_rms_norm_bwd_x_w
        return fn(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), n_rows, n_cols, eps, _p(fwd_weighted_sums), _p(fwd_rms_vals), _p(rms_weight),
                  _p(X_inp), _p(upstream_dX), _p(dX), _p(dW))

    def submit_rope(self, stream_id, fwd_dt, N, model_dim, head_dim, num_kv_heads, theta, seq_positions, X_q, X_k):
        return _L.submit_rope(C.byref(self.h), stream_id, int(fwd_dt), N, model_dim, head_dim, num_kv_heads, theta, _p(seq_positions), _p(X_q), _p(X_k))

    def submit_rope_bwd_x(self, stream_id, bwd_dt, N, model_dim, head_dim, num_kv_heads, theta, seq_positions, dX_q, dX_k):
        return _L.submit_rope_bwd_x(C.byref(self.h), stream_id, int(bwd_dt), N, model_dim, head_dim, num_kv_heads, theta, _p(seq_positions), _p(dX_q), _p(dX_k))

    def submit_swiglu(self, stream_id, fwd_dt, num_rows, num_cols, x_w1, x_w3, out):
        return _L.submit_swiglu(C.byref(self.h), stream_id, int(fwd_dt), num_rows, num_cols, _p(x_w1), _p(x_w3), _p(out))

    def submit_swiglu_bwd_x(self, stream_id, fwd_dt, bwd_dt, num_rows, num_cols, x_w1, x_w3, upstream_dX, dX_w1, dX_w3):
        return _L.submit_swiglu_bwd_x(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), num_rows, num_cols, _p(x_w1), _p(x_w3), _p(upstream_dX), _p(dX_w1), _p(dX_w3))

    def submit_softmax(self, stream_id, fwd_dt, bwd_dt, n_rows, n_cols, X, out):
        return _L.submit_softmax(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), n_rows, n_cols, _p(X), _p(out))

    def submit_cross_entropy_loss(self, stream_id, bwd_dt, n_rows, n_cols, pred_logits, labels):
        return _L.submit_cross_entropy_loss(C.byref(self.h), stream_id, int(bwd_dt), n_rows, n_cols, _p(pred_logits), _p(labels))

    def submit_softmax_cross_entropy(self, stream_id, fwd_dt, bwd_dt, n_rows, n_cols, logits, labels, dlogits, row_loss=None, loss_sum=None):
        return _L.submit_softmax_cross_entropy(C.byref(self.h), stream_id, int(fwd_dt), int(bwd_dt), n_rows, n_cols, _p(logits), _p(labels),
                                               _p(dlogits), _p(row_loss), _p(loss_sum))

    def submit_embedding(self, stream_id, fwd_dt, num_tokens, embed_dim, token_ids, embedding_table, output):
        return _L.submit_embedding(C.byref(self.h), stream_id, int(fwd_dt), num_tokens, embed_dim, _p(token_ids), _p(embedding_table), _p(output))

    def submit_copy_to_seq_context(self, stream_id, fwd_dt, N, total_tokens, kv_dim, X_k, X_v, seq_positions, seq_context_ptrs, seq_context_sizes):
        return _L.submit_copy_to_seq_context(C.byref(self.h), stream_id, int(fwd_dt), N, total_tokens, kv_dim, _p(X_k), _p(X_v), _p(seq_positions),
                                             _p(seq_context_ptrs), _p(seq_context_sizes))

    def submit_select_experts(self, stream_id, fwd_dt, total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts,
                              expert_counts, expert_counts_cumsum, num_routed_by_expert):
        return _L.submit_select_experts(C.byref(self.h), stream_id, int(fwd_dt), total_tokens, n_experts, top_k_experts, _p(X_routed),
                                        _p(token_expert_weights), _p(chosen_experts), _p(expert_counts), _p(expert_counts_cumsum),
                                        _p(num_routed_by_expert))

    def submit_softmax_argmax(self, stream_id, fwd_dt, n_rows, n_cols, X, out, arg_maxs=None):
        return _L.submit_softmax_argmax(C.byref(self.h), stream_id, int(fwd_dt), n_rows, n_cols, _p(X), _p(out), _p(arg_maxs))

    def submit_swiglu_ffn_fp8(self, stream_id, T, d, f, A, Wgate, gate_scales, Wup, up_scales, Wdown, down_scales, out, residual=None, gate_save=None,
                              up_save=None):
        return _L.submit_swiglu_ffn_fp8(C.byref(self.h), stream_id, T, d, f, _p(A), _p(Wgate), _p(gate_scales), _p(Wup), _p(up_scales), _p(Wdown),
                                        _p(down_scales), _p(residual), _p(out), _p(gate_save), _p(up_save))

    def submit_swiglu_ffn_fp8_bwd(self, stream_id, T, d, f, dOut, gate_saved, up_saved, WdownT, down_scales, WgateupT, gateup_scales, dA):
        return _L.submit_swiglu_ffn_fp8_bwd(C.byref(self.h), stream_id, T, d, f, _p(dOut), _p(gate_saved), _p(up_saved), _p(WdownT), _p(down_scales),
                                            _p(WgateupT), _p(gateup_scales), _p(dA))

    def close(self):
        if self.h.streams:
            _L.destroy_cuda_dataflow_handle(C.byref(self.h))

    def __del__(self):
        if getattr(self, "keep_until_exit", False):       # streams that other libraries may still reference: left to the process's end
            return
        try:
            self.close()
        except Exception:
            pass
