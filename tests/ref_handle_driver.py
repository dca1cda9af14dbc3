"""This library's op plug-ins under the REFERENCE's own handle, driven by the reference's own submit_* wrappers.

oracle/_ref/libref_handle.so is als244/dataflow_lib's cuda_dataflow_handle.c, cuda_drv.c, table, fingerprint, datatype,
set_native_op_skeletons.c and the dataflow_ops wrappers compiled unchanged (oracle/Makefile). This script, run as a process of its own
by tests/test_reference_handle_gpu.py, plays the reference caller:

    init_cuda_dataflow_handle            the reference's (a private context from cuCtxCreate, src/dataflow_handle/nvidia/src/cuda_drv.c:35-49)
    set_native_op_skeleton               the reference's skeletons and fingerprints (src/set_ops/src/set_native_op_skeletons.c:234-611)
    handle.register_external_code        the reference's (src/dataflow_handle/nvidia/src/cuda_dataflow_handle.c:181-250), given
                                         libdataflow_b200.so and the dataflow_b200_<op> symbols
    submit_rms_norm ... submit_cross_entropy_loss   the reference's wrappers (src/dataflow_ops/src/*.c), which reach this library's
                                         kernels through the reference's cuda_submit_op (:256-350)
    handle.alloc_mem / submit_*_transfer / sync_stream   the reference's

Results are compared with the CPU oracle. It runs in its own process because the reference's context becomes the thread's current
context, which must not be mixed with a framework that lives in the primary context. No torch tensor is touched here."""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path[:0] = [ROOT, HERE]


def main():
    import oracle as O
    from dataflow_lib_b200 import abi, _lib
    from util import check_f32, check_lowp

    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_handle.so"), mode=os.RTLD_LOCAL | os.RTLD_NOW)
    H, SK = C.POINTER(abi.DataflowHandleStruct), C.POINTER(abi.OpSkeleton)
    vp, i32, f32_, u64 = C.c_void_p, C.c_int, C.c_float, C.c_uint64
    sigs = {
        "init_cuda_dataflow_handle": [H, i32, i32, i32, C.c_uint, i32, vp, vp],
        "set_native_op_skeleton": [SK, C.c_char_p, i32, i32],
        "submit_rms_norm": [H, i32, i32, i32, i32, f32_, vp, vp, vp, vp, vp],
        "submit_rms_norm_bwd_x": [H, i32, i32, i32, i32, i32, f32_, vp, vp, vp, vp, vp, vp],
        "submit_rms_norm_bwd_w": [H, i32, i32, i32, i32, i32, f32_, vp, vp, vp, vp],
        "submit_rope": [H, i32, i32, u64, i32, i32, i32, i32, vp, vp, vp],
        "submit_rope_bwd_x": [H, i32, i32, u64, i32, i32, i32, i32, vp, vp, vp],
        "submit_swiglu": [H, i32, i32, i32, i32, vp, vp, vp],
        "submit_swiglu_bwd_x": [H, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp],
        "submit_softmax": [H, i32, i32, i32, i32, i32, vp, vp],
        "submit_cross_entropy_loss": [H, i32, i32, i32, i32, vp, vp],
    }
    for name, args in sigs.items():
        getattr(ref, name).argtypes = args
        getattr(ref, name).restype = i32

    h = abi.DataflowHandleStruct()
    assert ref.init_cuda_dataflow_handle(C.byref(h), abi.COMPUTE_CUDA, 0, 0, 0, 2, None, None) == 0
    hp = C.byref(h)
    BF, NONE = int(abi.DataflowDatatype.BF16), int(abi.DataflowDatatype.NONE)

    # ---- registration: the reference's skeletons, this library's functions
    families = [("rms_norm", BF, NONE, False), ("rms_norm_bwd_x", BF, BF, False), ("rms_norm_bwd_w", BF, BF, True), ("rope", BF, NONE, False),
                ("rope_bwd_x", NONE, BF, False), ("swiglu", BF, NONE, False), ("swiglu_bwd_x", BF, BF, False), ("softmax", BF, BF, False),
                ("cross_entropy_loss", NONE, BF, False)]
    n = len(families)
    sks = (abi.OpSkeleton * n)()
    for k, (op, fwd, bwd, _) in enumerate(families):
        assert ref.set_native_op_skeleton(C.byref(sks[k]), op.encode(), fwd, bwd) == 0
    syms = (C.c_char_p * n)(*[f"dataflow_b200_{op}".encode() for op, _, _, _ in families])
    inits = (C.c_char_p * n)(*[b"dataflow_b200_workspace_init" if ws else None for _, _, _, ws in families])
    assert h.register_external_code(hp, _lib.LIB_PATH.encode(), n, sks, syms, inits) == n
    assert h.num_ops == n

    # ---- buffers through the reference's alloc_mem and blocking transfers (stream id -1)
    def dev(a):
        a = np.ascontiguousarray(a)
        p = h.alloc_mem(hp, a.nbytes)
        assert p
        assert h.submit_inbound_transfer(hp, -1, p, a.ctypes.data, a.nbytes) == 0
        return p

    def empty(nbytes):
        p = h.alloc_mem(hp, nbytes)
        assert p
        assert h.set_mem(hp, -1, p, 0, nbytes) == 0
        return p

    def host(p, shape, dtype):
        a = np.empty(shape, dtype)
        assert h.submit_outbound_transfer(hp, -1, a.ctypes.data, p, a.nbytes) == 0
        return a

    T, d, nh, nkv, hd, f, V = 96, 1024, 8, 2, 128, 2048, 4128
    X, w, dY = O.fill_normal(O.BF16, (T, d), 1), O.fill_normal(O.BF16, (d,), 2, 1.0, 0.02), O.fill_normal(O.BF16, (T, d), 3)
    Q, K = O.fill_normal(O.BF16, (T, nh * hd), 4), O.fill_normal(O.BF16, (T, nkv * hd), 5)
    g, u, dS = O.fill_normal(O.BF16, (T, f), 6), O.fill_normal(O.BF16, (T, f), 7), O.fill_normal(O.BF16, (T, f), 8)
    logits, labels = O.fill_normal(O.BF16, (T, V), 9, 0.0, 2.0), O.fill_labels(T, 10, V)
    long_rows = O.fill_normal(O.BF16, (6, 128256), 11, 0.0, 2.0)          # a cluster of two CTAs per row, 64 KB of dynamic shared memory each
    pos = np.arange(T, dtype=np.int32)
    dX0 = O.fill_normal(O.BF16, (T, d), 12)

    Xd, wd, dYd, Qd, Kd, gd, ud, dSd, Ld, labd, posd, LRd = map(dev, (X, w, dY, Q, K, g, u, dS, logits, labels, pos, long_rows))
    Yd, dXd, dWd = empty(X.nbytes), dev(dX0), empty(w.nbytes)
    wsd, rmsd = empty(4 * T), empty(4 * T)
    Sd, d1d, d3d, Pd, LPd = empty(g.nbytes), empty(g.nbytes), empty(g.nbytes), empty(logits.nbytes), empty(long_rows.nbytes)

    s = 0
    assert ref.submit_rms_norm(hp, s, BF, T, d, 1e-5, wd, Xd, Yd, wsd, rmsd) == 0
    assert ref.submit_rope(hp, s, BF, T * nh * hd, nh * hd, hd, nkv, 500000, posd, Qd, Kd) == 0
    assert ref.submit_swiglu(hp, s, BF, T, f, gd, ud, Sd) == 0
    assert ref.submit_softmax(hp, s, BF, BF, T, V, Ld, Pd) == 0
    assert ref.submit_cross_entropy_loss(hp, s, BF, T, V, Pd, labd) == 0
    assert ref.submit_softmax(hp, s, BF, BF, long_rows.shape[0], long_rows.shape[1], LRd, LPd) == 0
    assert ref.submit_swiglu_bwd_x(hp, s, BF, BF, T, f, gd, ud, dSd, d1d, d3d) == 0
    assert ref.submit_rms_norm_bwd_x(hp, s, BF, BF, T, d, 1e-5, wsd, rmsd, wd, Xd, dYd, dXd) == 0
    ref.submit_rms_norm_bwd_w(hp, s, BF, BF, T, d, 1e-5, rmsd, Xd, dYd, dWd)     # the reference's wrapper has no return statement on success (norm_ops.c:92-97)
    assert h.sync_stream(hp, s) == 0
    q1, k1 = host(Qd, Q.shape, np.uint16), host(Kd, K.shape, np.uint16)
    assert ref.submit_rope_bwd_x(hp, s, BF, T * nh * hd, nh * hd, hd, nkv, 500000, posd, Qd, Kd) == 0
    assert h.sync_handle(hp) == 0

    # ---- against the oracle
    oY, ows, orms = O.rms_norm(O.BF16, 1e-5, w, X)
    check_lowp(host(Yd, X.shape, np.uint16), oY, O.BF16, "rms_norm")
    check_f32(host(rmsd, (T,), np.float32), orms, "rms_vals")
    check_f32(host(wsd, (T,), np.float32), ows, "weighted_sums", scale=1.0)
    oq, ok = O.rope(O.BF16, nh * hd, hd, nkv, 500000, pos, Q, K)
    check_lowp(q1, oq, O.BF16, "rope q")
    check_lowp(k1, ok, O.BF16, "rope k")
    oq2, ok2 = O.rope(O.BF16, nh * hd, hd, nkv, 500000, pos, oq, ok, bwd=True)
    check_lowp(host(Qd, Q.shape, np.uint16), oq2, O.BF16, "rope_bwd_x q")
    check_lowp(host(Kd, K.shape, np.uint16), ok2, O.BF16, "rope_bwd_x k")
    check_lowp(host(Sd, g.shape, np.uint16), O.swiglu(O.BF16, g, u), O.BF16, "swiglu")
    o1, o3 = O.swiglu_bwd_x(O.BF16, O.BF16, g, u, dS)
    check_lowp(host(d1d, g.shape, np.uint16), o1, O.BF16, "swiglu_bwd_x dX_w1")
    check_lowp(host(d3d, g.shape, np.uint16), o3, O.BF16, "swiglu_bwd_x dX_w3")
    probs = O.cross_entropy_loss(O.BF16, O.softmax(O.BF16, O.BF16, logits), labels)
    got = host(Pd, logits.shape, np.uint16)
    check_lowp(got, probs, O.BF16, "softmax + cross_entropy_loss", scale=1.0 / V)
    neg = O.to_f32(got, O.BF16) < 0
    assert np.array_equal(np.nonzero(neg)[1], labels.astype(np.int64)), "label indexing"
    check_lowp(host(LPd, long_rows.shape, np.uint16), O.softmax(O.BF16, O.BF16, long_rows), O.BF16, "softmax, 128256 columns", scale=1.0 / 128256)
    check_lowp(host(dXd, X.shape, np.uint16), O.rms_norm_bwd_x(O.BF16, O.BF16, ows, orms, w, X, dY, dX0), O.BF16, "rms_norm_bwd_x (accumulating)")
    check_lowp(host(dWd, w.shape, np.uint16), O.rms_norm_bwd_w(O.BF16, O.BF16, orms, X, dY, np.zeros_like(w)), O.BF16, "rms_norm_bwd_w",
               scale=float(np.sqrt(T)))
    words = (C.c_uint * 8)()
    assert _lib.lib.dfb200_read_kernel_status(None, words, 8) == 0, [hex(x) for x in words]
    print(f"reference handle ok: {n} plug-ins registered through the reference's register_external_code, 11 submissions through its submit_* wrappers")


if __name__ == "__main__":
    main()
