"""Mixed operation: the reference's OWN external-op code on this library's handle. oracle/_ref/libref_external_ops.so holds the
reference's submit_matmul wrapper and external skeletons (src/dataflow_ops/src/matmul_op.c, src/set_ops/src/set_external_op_skeletons.c)
linked against this library; oracle/_ref/libref_matmul_helper.so is its cuBLASLt plug-in
(src/ops/nvidia/external/matmul_helper/src/matmul_helper.c), both compiled unchanged by `make -C oracle ref`. The plug-in is registered
with handle->register_external_code and the head of the reference's transformer (RMSNorm -> vocabulary projection -> softmax ->
cross entropy -> projection backward, src/dataflow_models/dataflow_transformer/src/dataflow_transformer.c:300-420) is submitted op by op:
this library's kernels for the native ops, the reference's plug-in for the two GEMMs. Checked against the oracle composition
(bf16 tolerance 1e-2 of max(|ref|, rms))."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle as O
from util import check_lowp, f32, to_dev, to_host

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
EXT_OPS, MATMUL = os.path.join(REF_DIR, "libref_external_ops.so"), os.path.join(REF_DIR, "libref_matmul_helper.so")


@pytest.mark.skipif(not (os.path.exists(EXT_OPS) and os.path.exists(MATMUL)), reason="reference plug-ins not built (make -C oracle ref)")
@pytest.mark.parametrize("wrappers", ["reference", "own"])
def test_reference_matmul_plugin_on_this_handle(wrappers):
    """wrappers = "reference": submit_matmul and the matmul skeleton come from the reference's own compiled code; "own": from this
    library (same identity, same argument list), so the plug-in is found and fed the same way."""
    from dataflow_lib_b200 import DataflowHandle, abi
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    if wrappers == "reference":
        ext = C.CDLL(EXT_OPS)
    else:
        from dataflow_lib_b200 import _lib
        ext = C.CDLL(_lib.LIB_PATH)
        ext.set_external_matmul_skeleton.restype = None
    h = DataflowHandle(device_id=0, num_streams=1)
    sk = abi.OpSkeleton()
    ext.set_external_matmul_skeleton(C.byref(sk))
    assert bytes(sk.identifier.fingerprint).hex() == "2a113b16e997d04b8408f9aa299dd5a80bb77d29c95c8cc78270410ef84f3590"
    assert h.register_external_code(MATMUL, [sk], ["cublas_matmul"], ["cublas_matmul_init"]) == 1
    ext.submit_matmul.argtypes = [C.c_void_p, C.c_int] + [C.c_int] * 5 + [C.c_int] * 2 + [C.c_int] * 3 + [C.c_float] * 2 + [C.c_void_p] * 4 + [C.c_uint64, C.c_void_p]
    hp = C.addressof(h.h)

    T, d, V, eps = 256, 512, 2048, 1e-5
    X, w = O.fill_normal(O.BF16, (T, d), 1), O.fill_normal(O.BF16, (d,), 2, 1.0, 0.05)
    Wv = O.fill_normal(O.BF16, (V, d), 3, 0.0, 0.05)
    labels = O.fill_labels(T, 4, V)
    x_d, w_d, Wv_d = to_dev(X, O.BF16), to_dev(w, O.BF16), to_dev(Wv, O.BF16)
    hn = torch.empty((T, d), dtype=torch.bfloat16, device="cuda")
    ws, rms = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    logits, probs = torch.empty((T, V), dtype=torch.bfloat16, device="cuda"), torch.empty((T, V), dtype=torch.bfloat16, device="cuda")
    dh = torch.empty((T, d), dtype=torch.bfloat16, device="cuda")
    lab_d = torch.from_numpy(labels.astype(np.int32)).cuda()
    BF, FP32, NONE = int(DT.BF16), int(DT.FP32), int(DT.NONE)

    assert h.submit_rms_norm(0, DT.BF16, T, d, eps, w_d, x_d, hn, ws, rms) == 0
    # logits[T, V] = hn[T, d] . Wv[V, d]^T   (in the plug-in's column-major terms: D^T = A^T B with A = Wv stored d x V, B = hn stored d x T)
    assert ext.submit_matmul(hp, 0, BF, BF, NONE, BF, FP32, 1, 0, V, d, T, 1.0, 0.0, Wv_d.data_ptr(), hn.data_ptr(), None, logits.data_ptr(), 0, None) == 0
    assert h.submit_softmax(0, DT.BF16, DT.BF16, T, V, logits, probs) == 0
    assert h.submit_cross_entropy_loss(0, DT.BF16, T, V, probs, lab_d) == 0
    # dh[T, d] = dlogits[T, V] . Wv[V, d]
    assert ext.submit_matmul(hp, 0, BF, BF, NONE, BF, FP32, 0, 0, d, V, T, 1.0, 0.0, Wv_d.data_ptr(), probs.data_ptr(), None, dh.data_ptr(), 0, None) == 0
    assert h.sync_stream(0) == 0

    hn_ref, _, _ = O.rms_norm(O.BF16, eps, w, X)
    assert check_lowp(to_host(hn, O.BF16), hn_ref, O.BF16, "head rms_norm") > 0.99
    lg_ref = O.from_f32((f32(to_host(hn, O.BF16), O.BF16).astype(np.float64) @ f32(Wv, O.BF16).astype(np.float64).T).astype(np.float32), O.BF16)
    assert check_lowp(to_host(logits, O.BF16), lg_ref, O.BF16, "logits from the reference's cuBLASLt plug-in") > 0.98
    dl_ref = O.cross_entropy_loss(O.BF16, O.softmax(O.BF16, O.BF16, to_host(logits, O.BF16)), labels)
    assert check_lowp(to_host(probs, O.BF16), dl_ref, O.BF16, "softmax - onehot") > 0.99
    dh_ref = O.from_f32((f32(to_host(probs, O.BF16), O.BF16).astype(np.float64) @ f32(Wv, O.BF16).astype(np.float64)).astype(np.float32), O.BF16)
    check_lowp(to_host(dh, O.BF16), dh_ref, O.BF16, "projection backward from the reference's plug-in")
    h.close()
