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


@pytest.mark.skipif(not os.path.exists(MATMUL), reason="reference matmul plug-in not built (make -C oracle ref)")
def test_transformer_head_call_with_the_reference_matmul_plugin():
    """submit_transformer_head (include/dataflow_transformer.h), the reference's head as ONE host call: forward only, then forward +
    backward with weight-gradient accumulation and the copy of the head gradient on a second stream. Native ops are this library's,
    the three projections the reference's cuBLASLt plug-in. Each output is checked against the oracle composed step by step from
    the device's own inputs to that step (bf16 tolerance 1e-2 of max(|ref|, rms))."""
    from dataflow_lib_b200 import DataflowHandle, _lib, abi
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    L = _lib.lib
    h = DataflowHandle(device_id=0, num_streams=2)
    sk = abi.OpSkeleton()
    L.set_external_matmul_skeleton(C.byref(sk))
    assert h.register_external_code(MATMUL, [sk], ["cublas_matmul"], ["cublas_matmul_init"]) == 1

    T, d, V, eps = 384, 256, 4096, 1e-5
    bf = torch.bfloat16
    X, w = O.fill_normal(O.BF16, (T, d), 11), O.fill_normal(O.BF16, (d,), 12, 1.0, 0.05)
    Wv = O.fill_normal(O.BF16, (V, d), 13, 0.0, 0.05)
    labels = O.fill_labels(T, 14, V)
    labels[5] = V + 3                                                     # a row without a target
    dW0, dw0, dx0 = O.fill_normal(O.BF16, (V, d), 15, 0.0, 0.01), O.fill_normal(O.BF16, (d,), 16, 0.0, 0.01), O.fill_normal(O.BF16, (T, d), 17)
    x_d, w_d, Wv_d = to_dev(X, O.BF16), to_dev(w, O.BF16), to_dev(Wv, O.BF16)
    lab_d = torch.from_numpy(labels.astype(np.int32)).cuda()
    hn, logits, probs = torch.empty((T, d), dtype=bf, device="cuda"), torch.empty((T, V), dtype=bf, device="cuda"), torch.empty((T, V), dtype=bf, device="cuda")
    ws, rms, row_loss = torch.empty(T, device="cuda"), torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    dhn, dW, dw, dx, dx_copy = torch.empty((T, d), dtype=bf, device="cuda"), to_dev(dW0, O.BF16), to_dev(dw0, O.BF16), to_dev(dx0, O.BF16), torch.zeros((T, d), dtype=bf, device="cuda")
    work = torch.empty(32 << 20, dtype=torch.uint8, device="cuda")
    BF, FP32 = int(DT.BF16), int(DT.FP32)
    p = lambda t: t.data_ptr()
    head = abi.TransformerHead(BF, BF, FP32, eps, abi.EmbeddingConfig(V, d), None, p(w_d), p(Wv_d))
    act = abi.TransformerHeadActivations(T, None, p(hn), p(ws), p(rms), p(logits), p(work), work.numel())
    xin = abi.TransformerBlockTransition(None, p(x_d))
    out = abi.TransformerModelOutput(None, None, p(lab_d), p(probs), p(row_loss), 0.0)
    ghead = abi.TransformerHead(BF, BF, FP32, eps, abi.EmbeddingConfig(V, d), None, p(dw), p(dW))
    gact = abi.TransformerHeadActivations(T, None, p(dhn), None, None, None, p(work), work.numel())
    gs, gs2 = abi.TransformerBlockTransition(None, p(dx)), abi.TransformerBlockTransition(None, p(dx_copy))
    r, hp = C.byref, C.byref(h.h)

    # forward only: probabilities
    assert L.submit_transformer_head(hp, 0, 1, r(xin), r(head), r(act), r(out), None, None, None, None) == 0
    assert h.sync_stream(0) == 0
    hn_ref, _, _ = O.rms_norm(O.BF16, eps, w, X)
    assert check_lowp(to_host(hn, O.BF16), hn_ref, O.BF16, "head rms_norm") > 0.99
    hn_h, mm = to_host(hn, O.BF16), lambda a, b: (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert check_lowp(to_host(logits, O.BF16), O.from_f32(mm(f32(hn_h, O.BF16), f32(Wv, O.BF16).T), O.BF16), O.BF16, "logits") > 0.98
    lg_h = to_host(logits, O.BF16)
    assert check_lowp(to_host(probs, O.BF16), O.softmax(O.BF16, O.BF16, lg_h), O.BF16, "probabilities") > 0.99

    # forward + backward
    assert L.submit_transformer_head(hp, 0, 1, r(xin), r(head), r(act), r(out), r(ghead), r(gact), r(gs), r(gs2)) == 0
    assert h.sync_stream(0) == 0 and h.sync_stream(1) == 0
    dl_ref, loss_ref, _ = O.softmax_cross_entropy(O.BF16, O.BF16, lg_h, labels)
    dl_h = to_host(probs, O.BF16)
    assert check_lowp(dl_h, dl_ref, O.BF16, "softmax - onehot") > 0.99
    np.testing.assert_allclose(row_loss.cpu().numpy(), loss_ref, rtol=1e-5, atol=1e-5)
    assert row_loss[5].item() == 0.0
    dhn_h = to_host(dhn, O.BF16)
    check_lowp(dhn_h, O.from_f32(mm(f32(dl_h, O.BF16), f32(Wv, O.BF16)), O.BF16), O.BF16, "d(head_norm_out)")
    dW_ref = f32(dW0, O.BF16) + mm(f32(dl_h, O.BF16).T, f32(hn_h, O.BF16))
    check_lowp(to_host(dW, O.BF16), O.from_f32(dW_ref, O.BF16), O.BF16, "dW_head (accumulated)")
    ws_h, rms_h = ws.cpu().numpy(), rms.cpu().numpy()
    check_lowp(to_host(dx, O.BF16), O.rms_norm_bwd_x(O.BF16, O.BF16, ws_h, rms_h, w, X, dhn_h, dx0), O.BF16, "dX (accumulated)")
    check_lowp(to_host(dw, O.BF16), O.rms_norm_bwd_w(O.BF16, O.BF16, rms_h, X, dhn_h, dw0), O.BF16, "dW_norm (accumulated)", rel=2e-2)
    assert torch.equal(dx_copy, dx), "the copy on the second stream must see the finished gradient"
    h.close()
