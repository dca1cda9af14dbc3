"""numpy-level binding of oracle/liboracle.so -- the CPU restatement of the reference kernels' arithmetic
(oracle/oracle.c). TEST INFRASTRUCTURE: imported only by tests/, __graft_entry__.smoke() and bench.py's
CPU-baseline / reference arm.

Arrays of 16-bit floats are numpy uint16 (raw bits), fp8 arrays numpy uint8, fp32 numpy float32.
Datatype arguments are DataflowDatatype values (3 fp32, 4 fp16, 5 bf16, 6 e4m3, 7 e5m2)."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")

FP32, FP16, BF16, E4M3, E5M2 = 3, 4, 5, 6, 7
NP_OF = {FP32: np.float32, FP16: np.uint16, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8}


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])


if not os.path.exists(LIB_PATH):
    build()
_lib = C.CDLL(LIB_PATH)

_vp, _i, _f, _u64, _l = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_long
_sig = {
    "oracle_convert": (None, [_i, _vp, _i, _vp, _l]),
    "oracle_rms_norm": (None, [_i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_rms_norm_bwd_x": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "oracle_rms_norm_bwd_w": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i]),
    "oracle_rope": (None, [_i, _u64, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i]),
    "oracle_swiglu": (None, [_i, _i, _i, _vp, _vp, _vp, _i]),
    "oracle_swiglu_bwd_x": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_softmax": (None, [_i, _i, _i, _i, _vp, _vp, _i]),
    "oracle_cross_entropy_loss": (None, [_i, _i, _i, _vp, _vp]),
    "oracle_softmax_cross_entropy": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_quantize_rows_e4m3": (None, [_i, _i, _vp, _vp, _vp, _vp, _i]),
    "oracle_gemm_e4m3": (None, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_gemm_e4m3_swiglu": (None, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_gemm_e4m3_swiglu_bwd": (None, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_softmax_fp32_out": (None, [_i, _i, _i, _vp, _vp, _vp, _i]),
    "oracle_embedding": (None, [_i, _i, _i, _vp, _vp, _vp]),
    "oracle_copy_to_seq_context": (None, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "oracle_select_experts": (None, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "oracle_sigmoid_score": (_f, [_f]),
    "oracle_fill_normal": (None, [_i, _vp, _l, _l, _u64, _f, _f, _i]),
    "oracle_fill_labels": (None, [_vp, _l, _u64, C.c_uint32]),
}
for _n, (_r, _a) in _sig.items():
    getattr(_lib, _n).restype = _r
    getattr(_lib, _n).argtypes = _a

N_THREADS = os.cpu_count() or 1


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def convert(to_dt, src, from_dt):
    out = np.empty(src.shape, NP_OF[to_dt])
    _lib.oracle_convert(to_dt, _p(out), from_dt, _p(src), src.size)
    return out


def to_f32(a, dt):
    return a.astype(np.float32) if dt == FP32 else convert(FP32, a, dt)


def from_f32(a, dt):
    return np.ascontiguousarray(a, np.float32) if dt == FP32 else convert(dt, np.ascontiguousarray(a, np.float32), FP32)


def fill_normal(dt, shape, seed, mean=0.0, std=1.0, threads=None):
    """T(mean + std*z), z ~ N(0,1) a pure function of (seed, flat index)."""
    shape = tuple(shape) if hasattr(shape, "__len__") else (shape,)
    out = np.empty(shape, NP_OF[dt])
    rows = shape[0] if len(shape) > 1 else 1
    per = out.size // max(rows, 1)
    _lib.oracle_fill_normal(dt, _p(out), rows, per, seed, mean, std, threads or N_THREADS)
    return out


def fill_labels(n, seed, n_classes):
    out = np.empty(n, np.uint32)
    _lib.oracle_fill_labels(_p(out), n, seed, n_classes)
    return out


def rms_norm(dt, eps, w, X, threads=None):
    n_rows, n_cols = X.shape
    out = np.empty_like(X)
    ws = np.empty(n_rows, np.float32)
    rms = np.empty(n_rows, np.float32)
    _lib.oracle_rms_norm(dt, n_rows, n_cols, eps, _p(w), _p(X), _p(out), _p(ws), _p(rms), threads or N_THREADS)
    return out, ws, rms


def rms_norm_bwd_x(fwd_dt, bwd_dt, ws, rms, w, X, dY, dX, fused=True, threads=None):
    """Returns the updated dX (dX is accumulated into; the input array is not modified). fused=True is the single-rounding
    multiply-add the reference binary executes; fused=False rounds product and sum separately."""
    n_rows, n_cols = X.shape
    out = dX.copy()
    _lib.oracle_rms_norm_bwd_x(fwd_dt, bwd_dt, n_rows, n_cols, _p(ws), _p(rms), _p(w), _p(X), _p(dY), _p(out), int(fused), threads or N_THREADS)
    return out


def rms_norm_bwd_w(fwd_dt, bwd_dt, rms, X, dY, dW, n_blocks=0, threads=None):
    n_rows, n_cols = X.shape
    out = dW.copy()
    _lib.oracle_rms_norm_bwd_w(fwd_dt, bwd_dt, n_rows, n_cols, _p(rms), _p(X), _p(dY), _p(out), n_blocks, threads or N_THREADS)
    return out


def rope(dt, model_dim, head_dim, num_kv_heads, theta, pos, Xq, Xk, bwd=False, threads=None):
    q, k = Xq.copy(), Xk.copy()
    N = q.shape[0] * model_dim
    _lib.oracle_rope(dt, N, model_dim, head_dim, num_kv_heads, theta, _p(np.ascontiguousarray(pos, np.int32)), _p(q), _p(k), int(bwd), threads or N_THREADS)
    return q, k


def swiglu(dt, x1, x3, threads=None):
    out = np.empty_like(x1)
    _lib.oracle_swiglu(dt, x1.shape[0], x1.shape[1], _p(x1), _p(x3), _p(out), threads or N_THREADS)
    return out


def swiglu_bwd_x(fwd_dt, bwd_dt, x1, x3, dY, threads=None):
    d1, d3 = np.empty_like(dY), np.empty_like(dY)
    _lib.oracle_swiglu_bwd_x(fwd_dt, bwd_dt, x1.shape[0], x1.shape[1], _p(x1), _p(x3), _p(dY), _p(d1), _p(d3), threads or N_THREADS)
    return d1, d3


def softmax(fwd_dt, bwd_dt, X, threads=None):
    out = np.empty(X.shape, NP_OF[bwd_dt])
    _lib.oracle_softmax(fwd_dt, bwd_dt, X.shape[0], X.shape[1], _p(X), _p(out), threads or N_THREADS)
    return out


def cross_entropy_loss(bwd_dt, pred, labels):
    out = pred.copy()
    _lib.oracle_cross_entropy_loss(bwd_dt, pred.shape[0], pred.shape[1], _p(out), _p(np.ascontiguousarray(labels, np.uint32)))
    return out


def softmax_cross_entropy(fwd_dt, bwd_dt, logits, labels, threads=None):
    """Returns (dlogits, row_loss[n_rows] fp32, loss_sum[2] fp32 = {sum, valid rows})."""
    n_rows, n_cols = logits.shape
    dl = np.empty(logits.shape, NP_OF[bwd_dt])
    row_loss = np.empty(n_rows, np.float32)
    loss_sum = np.zeros(2, np.float32)
    _lib.oracle_softmax_cross_entropy(fwd_dt, bwd_dt, n_rows, n_cols, _p(logits), _p(np.ascontiguousarray(labels, np.uint32)), _p(dl),
                                      _p(row_loss), _p(loss_sum), threads or N_THREADS)
    return dl, row_loss, loss_sum


def quantize_rows_e4m3(X_bf16, col_factors=None, threads=None):
    """Per-row e4m3 quantisation of X * col_factors: returns (codes uint8 [rows, cols], scales fp32 [rows])."""
    Q = np.empty(X_bf16.shape, np.uint8)
    sc = np.empty(X_bf16.shape[0], np.float32)
    cf = None if col_factors is None else np.ascontiguousarray(col_factors, np.float32)
    _lib.oracle_quantize_rows_e4m3(X_bf16.shape[0], X_bf16.shape[1], _p(X_bf16), _p(cf), _p(Q), _p(sc), threads or N_THREADS)
    return Q, sc


def quantize_weight_e4m3(W_f32):
    """Per-output-channel quantisation of a weight matrix [out, in] (fp32): scale = amax / 448 per row."""
    amax = np.abs(W_f32).max(1)
    scale = np.where(amax > 0, amax / 448.0, 1.0).astype(np.float32)
    return from_f32((W_f32 / scale[:, None]).astype(np.float32), E4M3), scale


def gemm_e4m3(A, sa, W, sw, threads=None):
    out = np.empty((A.shape[0], W.shape[0]), np.uint16)
    _lib.oracle_gemm_e4m3(A.shape[0], W.shape[0], A.shape[1], _p(A), _p(sa), _p(W), _p(sw), _p(out), threads or N_THREADS)
    return out


def gemm_e4m3_swiglu(A, sa, Wg, sg, Wu, su, save=False, threads=None):
    """H = silu(g) * u; with save=True also returns the bf16 pre-activations (H, g, u)."""
    out = np.empty((A.shape[0], Wg.shape[0]), np.uint16)
    g = np.empty_like(out) if save else None
    u = np.empty_like(out) if save else None
    _lib.oracle_gemm_e4m3_swiglu(A.shape[0], Wg.shape[0], A.shape[1], _p(A), _p(sa), _p(Wg), _p(sg), _p(Wu), _p(su), _p(out), _p(g), _p(u),
                                 threads or N_THREADS)
    return (out, g, u) if save else out


def gemm_e4m3_swiglu_bwd(dOq, s_rows, WdownT, g_saved, u_saved, threads=None):
    """[dG | dU] (bf16 [M, 2f]) from the quantised output gradient, the transposed down weights and the saved pre-activations."""
    M, f = g_saved.shape
    out = np.empty((M, 2 * f), np.uint16)
    _lib.oracle_gemm_e4m3_swiglu_bwd(M, f, dOq.shape[1], _p(dOq), _p(s_rows), _p(WdownT), _p(g_saved), _p(u_saved), _p(out), threads or N_THREADS)
    return out


def swiglu_ffn_fp8(A_bf16, Wg, sg, Wu, su, Wd, sd, threads=None):
    """The whole forward (dfb200_swiglu_ffn_fp8): quantise rows, gate and up projections (bf16), SwiGLU in bf16, quantise the hidden
    rows, down projection. Returns (out, g, u)."""
    Aq, sa = quantize_rows_e4m3(A_bf16, None, threads)
    g, u = gemm_e4m3(Aq, sa, Wg, sg, threads), gemm_e4m3(Aq, sa, Wu, su, threads)
    Hq, sh = quantize_rows_e4m3(swiglu(BF16, g, u, threads), None, threads)
    return gemm_e4m3(Hq, sh, Wd, sd, threads), g, u


def swiglu_ffn_fp8_bwd(dOut_bf16, g, u, Wg, sg, Wu, su, Wd, sd, threads=None):
    """Input gradient of the FFN (dfb200_swiglu_ffn_fp8_bwd): returns dA bf16 [T, d]."""
    WdT = np.ascontiguousarray(Wd.T)                                           # [f, d]
    WguT = np.ascontiguousarray(np.concatenate([Wg.T, Wu.T], axis=1))          # [d, 2f]
    dOq, s1 = quantize_rows_e4m3(dOut_bf16, sd, threads)
    dH = gemm_e4m3(dOq, s1, WdT, None, threads)
    dg, du = swiglu_bwd_x(BF16, BF16, g, u, dH, threads)
    dGUq, s2 = quantize_rows_e4m3(np.ascontiguousarray(np.concatenate([dg, du], axis=1)), np.concatenate([sg, su]), threads)
    return gemm_e4m3(dGUq, s2, WguT, None, threads)


def transpose_quantize_e4m3(X_bf16):
    """Column-wise quantisation of X [rows, cols] and its transpose: returns (codes uint8 [cols, rows], scales fp32 [cols], amax fp32 [cols])
    with codes = e4m3(x * (448 / amax_col)) and scale = amax_col / 448 (1 for an all-zero column), all in fp32 arithmetic."""
    Xf = to_f32(np.ascontiguousarray(X_bf16), BF16)
    amax = np.abs(Xf).max(0).astype(np.float32)
    pos = amax > 0
    inv = np.where(pos, np.float32(448.0) / np.where(pos, amax, np.float32(1)), np.float32(1)).astype(np.float32)
    q = from_f32(np.ascontiguousarray((Xf * inv[None, :]).astype(np.float32)), E4M3)
    return np.ascontiguousarray(q.T), np.where(pos, amax / np.float32(448.0), np.float32(1)).astype(np.float32), amax


def swiglu_ffn_fp8_wgrad(A_bf16, dOut_bf16, g, u, dGU_bf16, threads=None):
    """Weight gradients of the FFN (dfb200_swiglu_ffn_fp8_wgrad): returns (dWgate [f, d], dWup [f, d], dWdown [d, f]) in bf16."""
    f = g.shape[1]
    H = swiglu(BF16, g, u, threads)
    (dOt, s_do, _), (At, s_a, _), (Ht, s_h, _), (dGUt, s_gu, _) = (transpose_quantize_e4m3(X) for X in (dOut_bf16, A_bf16, H, dGU_bf16))
    dWd = gemm_e4m3(dOt, s_do, Ht, s_h, threads)
    dWg = gemm_e4m3(np.ascontiguousarray(dGUt[:f]), s_gu[:f].copy(), At, s_a, threads)
    dWu = gemm_e4m3(np.ascontiguousarray(dGUt[f:]), s_gu[f:].copy(), At, s_a, threads)
    return dWg, dWu, dWd


def embedding(dt, token_ids, table):
    out = np.empty((len(token_ids), table.shape[1]), table.dtype)
    _lib.oracle_embedding(dt, len(token_ids), table.shape[1], _p(np.ascontiguousarray(token_ids, np.uint32)), _p(table), _p(out))
    return out


def copy_to_seq_context(dt, keys, values, seq_positions, contexts, token_context, context_sizes):
    """contexts: list of writable arrays [2 * size, kv_dim] (keys then values); token_context[t] = index of token t's context.
    Updates the arrays in place."""
    ptrs = np.array([contexts[c].ctypes.data for c in token_context], np.uint64)
    sizes = np.array([context_sizes[c] for c in token_context], np.int32)
    _lib.oracle_copy_to_seq_context(dt, keys.shape[0], keys.shape[1], _p(keys), _p(values), _p(np.ascontiguousarray(seq_positions, np.int32)),
                                    _p(ptrs), _p(sizes))


def select_experts(dt, X_routed, top_k, counts_in=None, threads=None):
    """Returns (weights [T, k] in dt, chosen uint16 [T, k], counts int32 [n_experts + 1], cumsum int32 [n_experts], num_routed int32 [n_experts])."""
    T, ne = X_routed.shape
    w = np.empty((T, top_k), NP_OF[dt])
    ids = np.empty((T, top_k), np.uint16)
    counts = np.zeros(ne + 1, np.int32) if counts_in is None else np.ascontiguousarray(counts_in, np.int32).copy()
    cumsum = np.empty(ne, np.int32)
    routed = np.full(ne, -1, np.int32)
    _lib.oracle_select_experts(dt, T, ne, top_k, _p(X_routed), _p(w), _p(ids), _p(counts), _p(cumsum), _p(routed), threads or N_THREADS)
    return w, ids, counts, cumsum, routed


def sigmoid_score(x):
    return float(_lib.oracle_sigmoid_score(float(x)))


def softmax_fp32_out(fwd_dt, X, threads=None):
    """Returns (probabilities fp32, arg_maxs uint32): the reference's softmax_<f16|bf16>_fp32 kernels."""
    out = np.empty(X.shape, np.float32)
    arg = np.empty(X.shape[0], np.uint32)
    _lib.oracle_softmax_fp32_out(fwd_dt, X.shape[0], X.shape[1], _p(X), _p(out), _p(arg), threads or N_THREADS)
    return out, arg
