"""softmax of fp16 / bf16 rows into fp32 probabilities with the arg-max index (the reference's softmax_<f16|bf16>_fp32 kernels,
src/ops/nvidia/loss/softmax.cu:965-1249) against the CPU oracle. Probabilities: |d| <= 1e-5 * max(|ref|, 1e-6) -- the
kernel's exponential and reciprocal are the approximate hardware forms the reference's fast-math build uses, a few fp32
ulps from the oracle's libm; arg-max indices bit-exact (the smallest index holding the maximum)."""
import numpy as np
import pytest
import torch

import oracle as O
from util import DT_NAME, check_f32, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", [O.FP16, O.BF16], ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("shape", [(64, 128256), (37, 1000), (5, 8), (3, 40000), (2, 262144), (130, 4096)], ids=str)
def test_softmax_fp32_out(dt, shape):
    from dataflow_lib_b200 import ops
    rows, cols = shape
    X = O.fill_normal(dt, shape, 21, 0.0, 2.0)
    # ties for the maximum: copy each row's maximum to two more places; the smallest index has to win
    Xf = O.to_f32(X, dt)
    am = Xf.argmax(1)
    for r in range(rows):
        for j in (cols // 3, cols - 1):
            X[r, j] = X[r, am[r]]
    ref, arg_ref = O.softmax_fp32_out(dt, X)
    assert np.array_equal(arg_ref, O.to_f32(X, dt).argmax(1))                 # numpy's argmax is also first-occurrence
    out = torch.full(shape, float("nan"), dtype=torch.float32, device="cuda")
    arg = torch.full((rows,), 12345, dtype=torch.int32, device="cuda")
    ops.softmax_fp32_out(rows, cols, to_dev(X, dt), out, arg)
    torch.cuda.synchronize()
    check_f32(out.cpu().numpy(), ref, f"softmax_fp32_out {DT_NAME[dt]} {shape}", rel=1e-5, scale=1e-6)
    assert np.array_equal(arg.cpu().numpy().view(np.uint32), arg_ref)
    # without the arg-max output
    out2 = torch.empty_like(out)
    ops.softmax_fp32_out(rows, cols, to_dev(X, dt), out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


def test_softmax_fp32_out_rejects_other_types():
    from dataflow_lib_b200 import ops
    x = torch.zeros((4, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError):
        ops.softmax_fp32_out(4, 64, x, torch.empty_like(x))


def test_softmax_argmax_through_the_handle():
    from dataflow_lib_b200 import DataflowHandle
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    X = O.fill_normal(O.BF16, (33, 2048), 22)
    ref, arg_ref = O.softmax_fp32_out(O.BF16, X)
    h = DataflowHandle(device_id=0, num_streams=1)
    assert h.num_registered == 96, h.num_registered
    out = torch.empty((33, 2048), dtype=torch.float32, device="cuda")
    arg = torch.zeros(33, dtype=torch.int32, device="cuda")
    assert h.submit_softmax_argmax(0, DT.BF16, 33, 2048, to_dev(X, O.BF16), out, arg) == 0
    h.sync_stream(0)
    check_f32(out.cpu().numpy(), ref, "softmax_argmax via handle", rel=1e-5, scale=1e-6)
    assert np.array_equal(arg.cpu().numpy().view(np.uint32), arg_ref)
    h.close()
