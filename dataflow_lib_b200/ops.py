"""The C-ABI kernel launchers (include/dataflow_b200_kernels.h) on torch CUDA tensors.

Function names and argument order mirror the reference's submit_* wrappers
(src/dataflow_ops/include/dataflow_ops.h:146-215) minus the handle: tensors in place of device
pointers, the current torch stream (or `stream=`) in place of a stream id. Nothing here computes:
every call goes to the shared object and raises RuntimeError with the library's message on failure.
"""
import torch

from . import _lib
from .abi import DataflowDatatype as DT

_lib_ = _lib.lib

TORCH_TO_DT = {
    torch.float32: DT.FP32, torch.float16: DT.FP16, torch.bfloat16: DT.BF16,
    torch.float8_e4m3fn: DT.FP8E4M3, torch.float8_e5m2: DT.FP8E5M2,
}


def dt_of(t: torch.Tensor) -> int:
    return int(TORCH_TO_DT[t.dtype])


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("dataflow_lib_b200.ops works on CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_lib.last_error()}")


def read_kernel_status(stream=None):
    """The device-side status words (one per kernel family that waits on asynchronous copies): all zero unless a bounded
    wait gave up. Synchronises `stream`."""
    import ctypes
    words = (ctypes.c_uint32 * 8)()
    rc = _lib_.dfb200_read_kernel_status(_stream(stream), words, 8)
    if rc < 0:
        _check(rc, "read_kernel_status")
    return list(words)


_workspaces = {}


def _workspace(device, nbytes):
    """Per-device scratch that only grows (the C-ABI leaves allocation to the caller)."""
    key = (device.type, device.index)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def rms_norm(n_rows, n_cols, eps, rms_weight, X, out, weighted_sums=None, rms_vals=None, stream=None):
    _check(_lib_.dfb200_rms_norm(dt_of(X), n_rows, n_cols, eps, _ptr(rms_weight), _ptr(X), _ptr(out),
                                 _ptr(weighted_sums), _ptr(rms_vals), _stream(stream)), "rms_norm")


def rms_norm_bwd_x(n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, stream=None):
    _check(_lib_.dfb200_rms_norm_bwd_x(dt_of(X_inp), dt_of(dX), n_rows, n_cols, eps, _ptr(fwd_weighted_sums), _ptr(fwd_rms_vals),
                                       _ptr(rms_weight), _ptr(X_inp), _ptr(upstream_dX), _ptr(dX), _stream(stream)), "rms_norm_bwd_x")


def rms_norm_bwd_w(n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, dW, stream=None, workspace=None):
    need = _lib_.dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols)
    ws = workspace if workspace is not None else _workspace(X_inp.device, need)
    _check(_lib_.dfb200_rms_norm_bwd_w(dt_of(X_inp), dt_of(dW), n_rows, n_cols, eps, _ptr(fwd_rms_vals), _ptr(X_inp),
                                       _ptr(upstream_dX), _ptr(dW), _ptr(ws), ws.numel() * ws.element_size(), _stream(stream)),
           "rms_norm_bwd_w")


def rms_norm_bwd_w_sums(n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, column_sums, stream=None, workspace=None):
    need = _lib_.dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols)
    ws = workspace if workspace is not None else _workspace(X_inp.device, need)
    _check(_lib_.dfb200_rms_norm_bwd_w_sums(dt_of(X_inp), dt_of(upstream_dX), n_rows, n_cols, eps, _ptr(fwd_rms_vals), _ptr(X_inp),
                                            _ptr(upstream_dX), _ptr(column_sums), _ptr(ws), ws.numel() * ws.element_size(), _stream(stream)),
           "rms_norm_bwd_w_sums")


def rms_norm_bwd_x_w(n_rows, n_cols, eps, fwd_weighted_sums, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, dW, stream=None, workspace=None, sums=False):
    """rms_norm_bwd_x and rms_norm_bwd_w in one pass over X and dY. sums=True: dW is an fp32 array that receives the column sums
    (the form of rms_norm_bwd_w_sums) instead of a gradient in dX's type that is accumulated into."""
    need = _lib_.dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols)
    ws = workspace if workspace is not None else _workspace(X_inp.device, need)
    fn = _lib_.dfb200_rms_norm_bwd_x_w_sums if sums else _lib_.dfb200_rms_norm_bwd_x_w
    _check(fn(dt_of(X_inp), dt_of(dX), n_rows, n_cols, eps, _ptr(fwd_weighted_sums), _ptr(fwd_rms_vals), _ptr(rms_weight), _ptr(X_inp),
              _ptr(upstream_dX), _ptr(dX), _ptr(dW), _ptr(ws), ws.numel() * ws.element_size(), _stream(stream)),
           "rms_norm_bwd_x_w_sums" if sums else "rms_norm_bwd_x_w")


def rope(N, model_dim, head_dim, num_kv_heads, theta, seq_positions, X_q, X_k, stream=None):
    _check(_lib_.dfb200_rope(dt_of(X_q), N, model_dim, head_dim, num_kv_heads, theta, _ptr(seq_positions), _ptr(X_q), _ptr(X_k),
                             _stream(stream)), "rope")


def rope_bwd_x(N, model_dim, head_dim, num_kv_heads, theta, seq_positions, dX_q, dX_k, stream=None):
    _check(_lib_.dfb200_rope_bwd_x(dt_of(dX_q), N, model_dim, head_dim, num_kv_heads, theta, _ptr(seq_positions), _ptr(dX_q),
                                   _ptr(dX_k), _stream(stream)), "rope_bwd_x")


def swiglu(num_rows, num_cols, x_w1, x_w3, out, stream=None):
    _check(_lib_.dfb200_swiglu(dt_of(x_w1), num_rows, num_cols, _ptr(x_w1), _ptr(x_w3), _ptr(out), _stream(stream)), "swiglu")


def swiglu_bwd_x(num_rows, num_cols, x_w1, x_w3, upstream_dX, dX_w1, dX_w3, stream=None):
    _check(_lib_.dfb200_swiglu_bwd_x(dt_of(x_w1), dt_of(upstream_dX), num_rows, num_cols, _ptr(x_w1), _ptr(x_w3), _ptr(upstream_dX),
                                     _ptr(dX_w1), _ptr(dX_w3), _stream(stream)), "swiglu_bwd_x")


def softmax(n_rows, n_cols, X, out, stream=None):
    _check(_lib_.dfb200_softmax(dt_of(X), dt_of(out), n_rows, n_cols, _ptr(X), _ptr(out), _stream(stream)), "softmax")


def softmax_fp32_out(n_rows, n_cols, X, out, arg_maxs=None, stream=None):
    _check(_lib_.dfb200_softmax_fp32_out(dt_of(X), n_rows, n_cols, _ptr(X), _ptr(out), _ptr(arg_maxs), _stream(stream)), "softmax_fp32_out")


def cross_entropy_loss(n_rows, n_cols, pred_logits, labels, stream=None):
    _check(_lib_.dfb200_cross_entropy_loss(dt_of(pred_logits), n_rows, n_cols, _ptr(pred_logits), _ptr(labels), _stream(stream)),
           "cross_entropy_loss")


def softmax_cross_entropy(n_rows, n_cols, logits, labels, dlogits, row_loss=None, loss_sum=None, stream=None, workspace=None):
    need = _lib_.dfb200_softmax_cross_entropy_workspace_bytes(n_rows, n_cols)
    ws = workspace if workspace is not None else _workspace(logits.device, need)
    _check(_lib_.dfb200_softmax_cross_entropy(dt_of(logits), dt_of(dlogits), n_rows, n_cols, _ptr(logits), _ptr(labels), _ptr(dlogits),
                                              _ptr(row_loss), _ptr(loss_sum), _ptr(ws), ws.numel() * ws.element_size(),
                                              _stream(stream)), "softmax_cross_entropy")


def embedding(num_tokens, embed_dim, token_ids, embedding_table, output, stream=None):
    _check(_lib_.dfb200_embedding(dt_of(embedding_table), num_tokens, embed_dim, _ptr(token_ids), _ptr(embedding_table), _ptr(output), _stream(stream)),
           "embedding")


def copy_to_seq_context(N, total_tokens, kv_dim, X_k, X_v, seq_positions, seq_context_ptrs, seq_context_sizes, stream=None):
    _check(_lib_.dfb200_copy_to_seq_context(dt_of(X_k), N, total_tokens, kv_dim, _ptr(X_k), _ptr(X_v), _ptr(seq_positions), _ptr(seq_context_ptrs),
                                            _ptr(seq_context_sizes), _stream(stream)), "copy_to_seq_context")


def select_experts(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts, expert_counts, expert_counts_cumsum,
                   num_routed_by_expert, stream=None):
    _check(_lib_.dfb200_select_experts(dt_of(X_routed), total_tokens, n_experts, top_k_experts, _ptr(X_routed), _ptr(token_expert_weights),
                                       _ptr(chosen_experts), _ptr(expert_counts), _ptr(expert_counts_cumsum), _ptr(num_routed_by_expert),
                                       _stream(stream)), "select_experts")


def quantize_rows_e4m3(n_rows, n_cols, X, Q, row_scales, col_factors=None, stream=None):
    _check(_lib_.dfb200_quantize_rows_e4m3(n_rows, n_cols, _ptr(X), _ptr(col_factors), _ptr(Q), _ptr(row_scales), _stream(stream)), "quantize_rows_e4m3")


def swiglu_quantize_rows_e4m3(n_rows, f, gate, up, Q, row_scales, stream=None):
    _check(_lib_.dfb200_swiglu_quantize_rows_e4m3(n_rows, f, _ptr(gate), _ptr(up), _ptr(Q), _ptr(row_scales), _stream(stream)), "swiglu_quantize_rows_e4m3")


def swiglu_bwd_quantize_rows_e4m3(n_rows, f, gate, up, dH, Q, row_scales, col_factors=None, dgate_dup=None, stream=None):
    _check(_lib_.dfb200_swiglu_bwd_quantize_rows_e4m3(n_rows, f, _ptr(gate), _ptr(up), _ptr(dH), _ptr(col_factors), _ptr(Q), _ptr(row_scales),
                                                      _ptr(dgate_dup), _stream(stream)), "swiglu_bwd_quantize_rows_e4m3")


def col_amax_bf16(n_rows, n_cols, X, col_amax, stream=None):
    _check(_lib_.dfb200_col_amax_bf16(n_rows, n_cols, _ptr(X), _ptr(col_amax), _stream(stream)), "col_amax_bf16")


def transpose_quantize_e4m3(n_rows, n_cols, X, col_amax, Qt, col_scales, stream=None):
    _check(_lib_.dfb200_transpose_quantize_e4m3(n_rows, n_cols, _ptr(X), _ptr(col_amax), _ptr(Qt), _ptr(col_scales), _stream(stream)),
           "transpose_quantize_e4m3")


def gemm_e4m3(M, N, K, A, a_row_scales, W, w_scales, out, residual=None, stream=None):
    _check(_lib_.dfb200_gemm_e4m3(M, N, K, _ptr(A), _ptr(a_row_scales), _ptr(W), _ptr(w_scales), _ptr(residual), _ptr(out), _stream(stream)), "gemm_e4m3")


def gemm_e4m3_swiglu(M, N, K, A, a_row_scales, Wgate, gate_scales, Wup, up_scales, H, gate_save=None, up_save=None, stream=None):
    _check(_lib_.dfb200_gemm_e4m3_swiglu(M, N, K, _ptr(A), _ptr(a_row_scales), _ptr(Wgate), _ptr(gate_scales), _ptr(Wup), _ptr(up_scales),
                                         _ptr(H), _ptr(gate_save), _ptr(up_save), _stream(stream)), "gemm_e4m3_swiglu")


def gemm_e4m3_swiglu_bwd(M, N, K, dOq, row_scales, WdownT, gate_saved, up_saved, dGU, stream=None):
    _check(_lib_.dfb200_gemm_e4m3_swiglu_bwd(M, N, K, _ptr(dOq), _ptr(row_scales), _ptr(WdownT), _ptr(gate_saved), _ptr(up_saved), _ptr(dGU),
                                             _stream(stream)), "gemm_e4m3_swiglu_bwd")


def swiglu_ffn_fp8(T, d, f, A, Wgate, gate_scales, Wup, up_scales, Wdown, down_scales, out, gate_save=None, up_save=None, residual=None, stream=None,
                   workspace=None):
    need = _lib_.dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f)
    ws = workspace if workspace is not None else _workspace(A.device, need)
    _check(_lib_.dfb200_swiglu_ffn_fp8(T, d, f, _ptr(A), _ptr(Wgate), _ptr(gate_scales), _ptr(Wup), _ptr(up_scales), _ptr(Wdown),
                                       _ptr(down_scales), _ptr(residual), _ptr(out), _ptr(gate_save), _ptr(up_save), _ptr(ws), ws.numel() * ws.element_size(),
                                       _stream(stream)), "swiglu_ffn_fp8")


def ffn_fp8_prepare_bwd_weights(d, f, Wgate, Wup, Wdown, WgateupT, WdownT, stream=None):
    _check(_lib_.dfb200_ffn_fp8_prepare_bwd_weights(d, f, _ptr(Wgate), _ptr(Wup), _ptr(Wdown), _ptr(WgateupT), _ptr(WdownT), _stream(stream)),
           "ffn_fp8_prepare_bwd_weights")


def swiglu_ffn_fp8_bwd(T, d, f, dOut, gate_saved, up_saved, WdownT, down_scales, WgateupT, gateup_scales, dA, dgate_dup=None, stream=None,
                       workspace=None):
    need = _lib_.dfb200_swiglu_ffn_fp8_workspace_bytes(T, d, f)
    ws = workspace if workspace is not None else _workspace(dOut.device, need)
    _check(_lib_.dfb200_swiglu_ffn_fp8_bwd(T, d, f, _ptr(dOut), _ptr(gate_saved), _ptr(up_saved), _ptr(WdownT), _ptr(down_scales), _ptr(WgateupT),
                                           _ptr(gateup_scales), _ptr(dA), _ptr(dgate_dup), _ptr(ws), ws.numel() * ws.element_size(), _stream(stream)),
           "swiglu_ffn_fp8_bwd")


def swiglu_ffn_fp8_wgrad(T, d, f, A, dOut, gate_saved, up_saved, dgate_dup, dWgate, dWup, dWdown, stream=None, workspace=None):
    need = _lib_.dfb200_swiglu_ffn_fp8_wgrad_workspace_bytes(T, d, f)
    ws = workspace if workspace is not None else _workspace(A.device, need)
    _check(_lib_.dfb200_swiglu_ffn_fp8_wgrad(T, d, f, _ptr(A), _ptr(dOut), _ptr(gate_saved), _ptr(up_saved), _ptr(dgate_dup), _ptr(dWgate), _ptr(dWup),
                                             _ptr(dWdown), _ptr(ws), ws.numel() * ws.element_size(), _stream(stream)), "swiglu_ffn_fp8_wgrad")
