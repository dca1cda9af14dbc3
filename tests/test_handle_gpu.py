"""The handle on a GPU: what a synchronising call reports about the kernels' bounded waits, and the ops' device scratch
(one block per op identity and stream, reserved ahead of time or grown on demand, released with the handle)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from util import check_lowp, to_dev, to_host

pytestmark = pytest.mark.gpu


def test_sync_reports_a_wait_that_gave_up(capfd):
    """A kernel whose bounded wait ran out only leaves a status word behind. The handle's synchronising calls are where a caller
    learns that earlier work is done, so they read the word: the first sync after the give-up fails (-1, message naming the word),
    the word is cleared by that read and the next sync succeeds. The wait is made to run out by the library's self-test kernel (a
    barrier that nothing completes); nothing faults."""
    from dataflow_lib_b200 import DataflowHandle, _lib
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    h = DataflowHandle(device_id=0, num_streams=2)
    assert h.sync_stream(0) == 0 and h.sync_handle() == 0
    assert _lib.lib.dfb200_selftest_bounded_wait(2, ctypes.c_void_p(h.stream_ptr(0))) == 1, _lib.last_error()
    assert h.sync_stream(0) == -1
    assert "gave up a bounded wait" in capfd.readouterr().err
    assert h.sync_stream(0) == 0
    assert _lib.lib.dfb200_selftest_bounded_wait(3, ctypes.c_void_p(h.stream_ptr(1))) == 1
    assert h.sync_handle() == -1 and h.sync_handle() == 0
    # and the handle keeps working
    x = torch.randn(32, 512, device="cuda").bfloat16()
    out = torch.empty_like(x)
    assert h.submit_swiglu(0, int(DT.BF16), 32, 512, x, x, out) == 0 and h.sync_stream(0) == 0
    assert torch.isfinite(out.float()).all()
    h.close()


def test_same_op_on_two_streams_keeps_separate_scratch():
    """rms_norm_bwd_w keeps partial sums in device scratch. Submissions of the same identity on two streams of one handle run
    concurrently here (different inputs, no ordering between the streams) and must each give their own answer: the scratch is keyed by
    (op, stream)."""
    from dataflow_lib_b200 import DataflowHandle, _lib
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    BF = int(DT.BF16)
    h = DataflowHandle(device_id=0, num_streams=2)
    R, Cc = 4096, 4096
    need = _lib.lib.dfb200_rms_norm_bwd_w_workspace_bytes(R, Cc)
    small = torch.ones(16, 256, device="cuda").bfloat16()
    for s in (0, 1):                                           # first launches load the kernels (device memory of their own) and make 1 MiB blocks
        assert h.submit_rms_norm_bwd_w(s, BF, BF, 16, 256, 1e-5, torch.ones(16, device="cuda"), small, small, torch.zeros(256, dtype=torch.bfloat16, device="cuda")) == 0
    assert h.sync_handle() == 0
    free0 = torch.cuda.mem_get_info()[0]
    assert h.reserve_workspace("rms_norm_bwd_w", 0, need, DT.BF16, DT.BF16) == 0
    assert h.reserve_workspace("rms_norm_bwd_w", 1, need, DT.BF16, DT.BF16) == 0
    assert h.reserve_workspace("rms_norm", 0, 1 << 20, DT.BF16) == -1                 # an op without scratch
    assert torch.cuda.mem_get_info()[0] < free0                # the two blocks grew
    data = []
    for s in (0, 1):
        g = torch.Generator(device="cuda").manual_seed(100 + s)
        X = torch.randn(R, Cc, device="cuda", generator=g).bfloat16()
        dY = torch.randn(R, Cc, device="cuda", generator=g).bfloat16()
        rms = torch.rsqrt(X.float().pow(2).mean(1) + 1e-5)
        data.append((X, dY, rms, torch.zeros(Cc, dtype=torch.bfloat16, device="cuda")))
    torch.cuda.synchronize()
    free1 = torch.cuda.mem_get_info()[0]                       # after the inputs exist: the tensor allocator may have grown its pool for them
    for rep in range(8):                                       # interleaved, so that launches of the two streams overlap on the device
        for s in (0, 1):
            X, dY, rms, dW = data[s]
            if rep:
                dW.zero_()
            assert h.submit_rms_norm_bwd_w(s, BF, BF, R, Cc, 1e-5, rms, X, dY, dW) == 0
    assert h.sync_handle() == 0
    assert torch.cuda.mem_get_info()[0] == free1              # reserved blocks were large enough: no submission allocated
    for s in (0, 1):
        X, dY, rms, dW = data[s]
        exact = (dY.float() * X.float() * rms[:, None]).double().sum(0)
        assert ((dW.double() - exact).abs() <= 2.0 ** -8 * exact.abs() + 2e-3).all(), f"stream {s}"
    torch.cuda.synchronize()
    before_close = torch.cuda.mem_get_info()[0]
    h.close()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] > before_close         # destroy released the blocks


def test_unreserved_scratch_grows_on_demand_and_matches_the_oracle():
    from dataflow_lib_b200 import DataflowHandle
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    BF = int(DT.BF16)
    h = DataflowHandle(device_id=0, num_streams=1)
    for (R, Cc) in ((16, 256), (300, 2048), (64, 8192)):       # growing shapes on the default stream id -1 and on stream 0
        X, dY = O.fill_normal(O.BF16, (R, Cc), 5), O.fill_normal(O.BF16, (R, Cc), 6)
        _, _, rms = O.rms_norm(O.BF16, 1e-5, O.fill_normal(O.BF16, (Cc,), 7, 1.0, 0.02), X)
        ref = O.rms_norm_bwd_w(O.BF16, O.BF16, rms, X, dY, np.zeros(Cc, np.uint16))
        for s in (-1, 0):
            dW = torch.zeros(Cc, dtype=torch.bfloat16, device="cuda")
            assert h.submit_rms_norm_bwd_w(s, BF, BF, R, Cc, 1e-5, torch.from_numpy(rms).cuda(), to_dev(X, O.BF16), to_dev(dY, O.BF16), dW) == 0
            torch.cuda.synchronize()
            check_lowp(to_host(dW, O.BF16), ref, O.BF16, f"rms_norm_bwd_w {R}x{Cc} stream {s}", scale=float(np.sqrt(R)))
    h.close()
