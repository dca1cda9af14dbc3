"""Shapes and alignments outside the packet kernels' contract: row lengths that are not multiples of 8 elements (4100, 1004, 36, 2),
tensors whose base is offset by one element from a 16-byte boundary, and rows beyond the on-chip forms. The reference's kernels take
all of these (thread-strided scalar loops: src/ops/nvidia/norm/rms_norm.cu:339-406, activations/swiglu.cu:48-68,
attention/rope.cu:137-171; softmax wants multiples of 32 only, loss/softmax.cu:310-322), so this library does too, through its
general-shape kernels. Checked against the CPU oracle with the tolerances of test_ops_gpu.py."""
import numpy as np
import pytest
import torch

import oracle as O
from util import DT_NAME, TORCH_OF, ULP_REL, check_f32, check_lowp, to_host

pytestmark = pytest.mark.gpu

COLS = [4100, 1004, 36, 2]
PAIRS = [(O.BF16, O.BF16), (O.FP32, O.FP32), (O.FP16, O.FP16), (O.E4M3, O.BF16)]
pair_id = lambda p: f"{DT_NAME[p[0]]}-{DT_NAME[p[1]]}"


@pytest.fixture(scope="module")
def ops():
    from dataflow_lib_b200 import ops as _ops
    return _ops


def rel_for(dt):
    return 1e-5 if dt == O.FP32 else max(1e-2, 1.01 * ULP_REL[dt])


def dev(a, dt, offset):
    """numpy raw-bit array -> CUDA tensor whose first element sits `offset` elements after a fresh allocation's (256-byte aligned) start."""
    a = np.ascontiguousarray(a)
    raw = torch.from_numpy(a.view(np.int16) if dt in (O.FP16, O.BF16) else a).reshape(-1)
    buf = torch.empty(raw.numel() + offset, dtype=raw.dtype, device="cuda")
    buf[offset:].copy_(raw)
    t = buf[offset:].view(a.shape)
    t = t.view(TORCH_OF[dt]) if dt != O.FP32 else t
    assert t.is_contiguous() and (offset == 0 or t.data_ptr() % 16 != 0)
    return t


def empty_like(shape, dt, offset):
    return dev(np.zeros(shape, O.NP_OF[dt]), dt, offset)


@pytest.mark.parametrize("offset", [0, 1], ids=["aligned", "offset_by_one"])
@pytest.mark.parametrize("n_cols", COLS)
@pytest.mark.parametrize("pair", PAIRS, ids=pair_id)
def test_rms_norm_family(ops, pair, n_cols, offset):
    F, B = pair
    R, eps = 37, 1e-5
    X, w = O.fill_normal(F, (R, n_cols), 1), O.fill_normal(F, (n_cols,), 2, 1.0, 0.05)
    dY, dX0, dW0 = O.fill_normal(B, (R, n_cols), 3), O.fill_normal(B, (R, n_cols), 4), O.fill_normal(B, (n_cols,), 5, 0.0, 0.1)
    Xd, wd, dYd, dXd, dWd = dev(X, F, offset), dev(w, F, offset), dev(dY, B, offset), dev(dX0, B, offset), dev(dW0, B, offset)
    Y = empty_like((R, n_cols), F, offset)
    ws, rms = torch.empty(R, device="cuda"), torch.empty(R, device="cuda")
    ops.rms_norm(R, n_cols, eps, wd, Xd, Y, ws, rms)
    ops.rms_norm_bwd_x(R, n_cols, eps, ws, rms, wd, Xd, dYd, dXd)
    ops.rms_norm_bwd_w(R, n_cols, eps, rms, Xd, dYd, dWd)
    sums = torch.full((n_cols + 1,), float("nan"), device="cuda")[1:] if offset else torch.full((n_cols,), float("nan"), device="cuda")
    ops.rms_norm_bwd_w_sums(R, n_cols, eps, rms, Xd, dYd, sums)
    torch.cuda.synchronize()
    oY, ows, orms = O.rms_norm(F, eps, w, X)
    check_lowp(to_host(Y, F), oY, F, "rms_norm", rel=rel_for(F))
    check_f32(rms.cpu().numpy(), orms, "rms_vals")
    check_f32(ws.cpu().numpy(), ows, "weighted_sums", scale=float(np.sqrt(n_cols)))
    # the gradients from the DEVICE's statistics, so that the comparison isolates each op
    check_lowp(to_host(dXd, B), O.rms_norm_bwd_x(F, B, ws.cpu().numpy(), rms.cpu().numpy(), w, X, dY, dX0), B, "rms_norm_bwd_x", rel=max(rel_for(B), 2 * ULP_REL[B]))
    ref_w = O.rms_norm_bwd_w(F, B, rms.cpu().numpy(), X, dY, dW0)
    check_lowp(to_host(dWd, B), ref_w, B, "rms_norm_bwd_w", rel=max(rel_for(B), 2e-5), scale=float(np.sqrt(R)))
    exact = (O.to_f32(dY, B).astype(np.float64) * O.to_f32(X, F) * rms.cpu().numpy()[:, None]).sum(0)
    np.testing.assert_allclose(sums.cpu().numpy(), exact, rtol=2e-5, atol=2e-5 * np.sqrt(R))


@pytest.mark.parametrize("offset", [0, 1], ids=["aligned", "offset_by_one"])
@pytest.mark.parametrize("n_cols", COLS)
@pytest.mark.parametrize("pair", PAIRS, ids=pair_id)
def test_swiglu_family(ops, pair, n_cols, offset):
    F, B = pair
    R = 29                                                      # 29 x n_cols is not a multiple of 8 for 4100, 1004, 36 and 2
    x1, x3, dY = O.fill_normal(F, (R, n_cols), 6), O.fill_normal(F, (R, n_cols), 7), O.fill_normal(B, (R, n_cols), 8)
    a, b, g = dev(x1, F, offset), dev(x3, F, offset), dev(dY, B, offset)
    out, d1, d3 = empty_like((R, n_cols), F, offset), empty_like((R, n_cols), B, offset), empty_like((R, n_cols), B, offset)
    ops.swiglu(R, n_cols, a, b, out)
    ops.swiglu_bwd_x(R, n_cols, a, b, g, d1, d3)
    torch.cuda.synchronize()
    check_lowp(to_host(out, F), O.swiglu(F, x1, x3), F, "swiglu", rel=rel_for(F) if F != O.FP32 else 1e-5)
    o1, o3 = O.swiglu_bwd_x(F, B, x1, x3, dY)
    check_lowp(to_host(d1, B), o1, B, "swiglu_bwd_x dX_w1", rel=rel_for(B) if B != O.FP32 else 2e-5)
    check_lowp(to_host(d3, B), o3, B, "swiglu_bwd_x dX_w3", rel=rel_for(B) if B != O.FP32 else 1e-5)


@pytest.mark.parametrize("offset", [0, 1], ids=["aligned", "offset_by_one"])
@pytest.mark.parametrize("geometry", [(3, 1, 12), (5, 2, 2), (2, 2, 36), (4, 1, 128), (1, 0, 6)], ids=str)      # (q heads, kv heads, head_dim)
@pytest.mark.parametrize("dt", [O.BF16, O.FP32, O.FP16], ids=lambda d: DT_NAME[d])
def test_rope_family(ops, dt, geometry, offset):
    nh, nkv, hd = geometry
    T, theta = 41, 10000
    md, kv = nh * hd, nkv * hd
    Q, K = O.fill_normal(dt, (T, md), 9), O.fill_normal(dt, (T, max(nkv, 1) * hd), 10)
    pos = (np.arange(T, dtype=np.int32) * 7) % 300
    q, k = dev(Q, dt, offset), dev(K, dt, offset)
    pos_d = torch.from_numpy(pos).cuda()
    ops.rope(T * md, md, hd, nkv, theta, pos_d, q, k)
    torch.cuda.synchronize()
    oq, ok = O.rope(dt, md, hd, nkv, theta, pos, Q, K)
    tol = dict(rel=rel_for(dt) if dt != O.FP32 else 2e-4)       # fp32: the angle pos * theta^(-2j/hd) itself carries ~1e-5 rad
    check_lowp(to_host(q, dt), oq, dt, "rope q", **tol)
    if kv:
        check_lowp(to_host(k, dt), ok, dt, "rope k", **tol)
    ops.rope_bwd_x(T * md, md, hd, nkv, theta, pos_d, q, k)
    torch.cuda.synchronize()
    oq2, ok2 = O.rope(dt, md, hd, nkv, theta, pos, oq, ok, bwd=True)
    check_lowp(to_host(q, dt), oq2, dt, "rope_bwd_x q", **tol)
    if kv:
        check_lowp(to_host(k, dt), ok2, dt, "rope_bwd_x k", **tol)


@pytest.mark.parametrize("offset", [0, 1], ids=["aligned", "offset_by_one"])
@pytest.mark.parametrize("n_cols", [4100, 1004, 36, 2, 4096, 300000])
@pytest.mark.parametrize("pair", PAIRS, ids=pair_id)
def test_softmax(ops, pair, n_cols, offset):
    if offset == 0 and n_cols == 4096:
        pytest.skip("the packet kernel's own case (test_ops_gpu.py)")
    F, B = pair
    R = 3 if n_cols > 100000 else 19
    X = O.fill_normal(F, (R, n_cols), 11, 0.0, 2.0)
    x, out = dev(X, F, offset), empty_like((R, n_cols), B, offset)
    ops.softmax(R, n_cols, x, out)
    torch.cuda.synchronize()
    ref = O.softmax(F, B, X)
    check_lowp(to_host(out, B), ref, B, f"softmax {n_cols}", rel=rel_for(B) if B != O.FP32 else 2e-5, scale=1.0 / n_cols)
    if B == O.BF16 and F == O.BF16:
        assert (to_host(out, B) == ref).mean() > 0.97           # the reference's rounding points are kept, up to fp32 summation order
