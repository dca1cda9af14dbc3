"""GPU parity tests: the sm_100a kernels, called through the C-ABI (dataflow_lib_b200.ops -> dfb200_*),
against the CPU oracle on the same seeded inputs. Tolerances (stated per check):
  low-precision outputs   |d| <= 1e-2 * max(|ref|, rms(ref))      (fp32 tensors: 1e-5)
  fp32 statistics / loss  |d| <= 1e-5 * max(|ref|, scale)
  label indexing          bit-exact."""
import numpy as np
import pytest
import torch

import oracle as O
from util import BWD_DTS, DT_NAME, FWD_DTS, PAIRS, ULP_REL, check_f32, check_lowp, f32, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from dataflow_lib_b200 import ops as _ops
    return _ops


def rel_for(dt):
    """1e-5 for fp32, 1e-2 for 16-bit types; fp8 outputs cannot resolve 1e-2, so they get one unit in the last place."""
    if dt == O.FP32:
        return 1e-5
    return max(1e-2, 1.01 * ULP_REL[dt])


def fill(dt, shape, seed, mean=0.0, std=1.0):
    return O.fill_normal(dt, shape, seed, mean, std)


# ------------------------------------------------------------------------------------------ RMSNorm

RMS_SHAPES = [(256, 4096), (17, 1024), (3, 8), (1, 4096), (64, 8192), (5, 16384), (300, 2048), (9, 5120), (2, 32768)]


@pytest.mark.parametrize("dt", FWD_DTS, ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("shape", RMS_SHAPES, ids=str)
def test_rms_norm_fwd(ops, dt, shape):
    n_rows, n_cols = shape
    X, w = fill(dt, shape, 1), fill(dt, (n_cols,), 2, 1.0, 0.02)
    ref_out, ref_ws, ref_rms = O.rms_norm(dt, 1e-5, w, X)
    Xd, wd = to_dev(X, dt), to_dev(w, dt)
    out = torch.empty_like(Xd)
    ws = torch.full((n_rows,), float("nan"), device="cuda")
    rms = torch.full((n_rows,), float("nan"), device="cuda")
    ops.rms_norm(n_rows, n_cols, 1e-5, wd, Xd, out, ws, rms)
    torch.cuda.synchronize()
    check_lowp(to_host(out, dt), ref_out, dt, "rms_norm out", rel=rel_for(dt))
    check_f32(rms.cpu().numpy(), ref_rms, "rms_vals", rel=1e-5)
    # weighted sums cancel (sum of +- terms): scale the tolerance by sqrt(sum (w x)^2), the size of the terms
    term_scale = np.sqrt((f32(X, dt).astype(np.float64) ** 2 * f32(w, dt).astype(np.float64) ** 2).sum(1)).max()
    check_f32(ws.cpu().numpy(), ref_ws, "weighted_sums", rel=1e-5, scale=term_scale)
    # NULL statistics pointers (the recompute calls of the reference's backward pass)
    out2 = torch.empty_like(Xd)
    ops.rms_norm(n_rows, n_cols, 1e-5, wd, Xd, out2, None, None)
    torch.cuda.synchronize()
    assert torch.equal(out2.view(torch.uint8), out.view(torch.uint8))


@pytest.mark.parametrize("pair", PAIRS, ids=lambda p: f"{DT_NAME[p[0]]}_{DT_NAME[p[1]]}")
@pytest.mark.parametrize("shape", [(256, 4096), (17, 1024), (3, 16), (64, 8192), (2, 32768)], ids=str)
@pytest.mark.parametrize("zero_dx", [True, False], ids=["dx0", "dxN"])
def test_rms_norm_bwd_x(ops, pair, shape, zero_dx):
    fdt, bdt = pair
    n_rows, n_cols = shape
    X, w = fill(fdt, shape, 1), fill(fdt, (n_cols,), 2, 1.0, 0.02)
    dY = fill(bdt, shape, 3)
    dX0 = np.zeros(shape, O.NP_OF[bdt]) if zero_dx else fill(bdt, shape, 4)
    _, ws, rms = O.rms_norm(fdt, 1e-5, w, X)
    ref = O.rms_norm_bwd_x(fdt, bdt, ws, rms, w, X, dY, dX0, fused=True)
    dX = to_dev(dX0, bdt)
    ops.rms_norm_bwd_x(n_rows, n_cols, 1e-5, torch.from_numpy(ws).cuda(), torch.from_numpy(rms).cuda(), to_dev(w, fdt), to_dev(X, fdt),
                       to_dev(dY, bdt), dX)
    torch.cuda.synchronize()
    got = to_host(dX, bdt)
    frac = check_lowp(got, ref, bdt, "rms_norm_bwd_x dX", rel=rel_for(bdt))
    assert bdt == O.FP32 or frac > 0.99, f"only {frac:.4f} of dX bit-identical to the oracle"


@pytest.mark.parametrize("pair", PAIRS, ids=lambda p: f"{DT_NAME[p[0]]}_{DT_NAME[p[1]]}")
@pytest.mark.parametrize("shape", [(4096, 4096), (17, 1024), (3, 16), (1000, 8192), (2, 32768), (777, 512)], ids=str)
def test_rms_norm_bwd_w(ops, pair, shape):
    fdt, bdt = pair
    n_rows, n_cols = shape
    X, dY = fill(fdt, shape, 1), fill(bdt, shape, 3)
    rms = (1.0 / np.sqrt((f32(X, fdt).astype(np.float64) ** 2).mean(1) + 1e-5)).astype(np.float32)
    dW0 = fill(bdt, (n_cols,), 5)
    ref = O.rms_norm_bwd_w(fdt, bdt, rms, X, dY, dW0, n_blocks=0)
    dW = to_dev(dW0, bdt)
    ops.rms_norm_bwd_w(n_rows, n_cols, 1e-5, torch.from_numpy(rms).cuda(), to_dev(X, fdt), to_dev(dY, bdt), dW)
    torch.cuda.synchronize()
    got = to_host(dW, bdt)
    # column sums of ~N(0,1) terms: absolute floor = size of a sum, sqrt(n_rows)
    check_lowp(got, ref, bdt, "rms_norm_bwd_w dW", rel=rel_for(bdt) if bdt != O.FP32 else 2e-5, scale=float(np.sqrt(n_rows)))
    # deterministic: a second run gives identical bits
    dW2 = to_dev(dW0, bdt)
    ops.rms_norm_bwd_w(n_rows, n_cols, 1e-5, torch.from_numpy(rms).cuda(), to_dev(X, fdt), to_dev(dY, bdt), dW2)
    torch.cuda.synchronize()
    assert np.array_equal(to_host(dW2, bdt), got)


@pytest.mark.parametrize("pair", PAIRS, ids=lambda p: f"{DT_NAME[p[0]]}_{DT_NAME[p[1]]}")
@pytest.mark.parametrize("shape", [(4096, 4096), (17, 1024), (3, 16), (1000, 8192), (64, 16384), (2, 32768), (777, 512), (301, 2056), (37, 4100)], ids=str)
@pytest.mark.parametrize("sums", [False, True], ids=["dW", "sums"])
def test_rms_norm_bwd_x_w(ops, pair, shape, sums):
    """Both gradients of the norm in one pass over X and dY (no reference counterpart): dX must be what rms_norm_bwd_x gives, bit for
    bit, and dW (or the fp32 column sums) what the oracle's rms_norm_bwd_w gives within the tolerance of the separate op. The shapes
    cover the staged kernel (rows of 16-byte multiples that fit the shared-memory ring with 1, 2 or 4 row groups), the register kernel
    (32768 columns: a row slot does not fit twice) and the general-shape fallback (4100 columns)."""
    fdt, bdt = pair
    n_rows, n_cols = shape
    X, w = fill(fdt, shape, 1), fill(fdt, (n_cols,), 2, 1.0, 0.02)
    dY, dX0 = fill(bdt, shape, 3), fill(bdt, shape, 4)
    _, ws, rms = O.rms_norm(fdt, 1e-5, w, X)
    wsd, rmsd, wd, Xd, dYd = torch.from_numpy(ws).cuda(), torch.from_numpy(rms).cuda(), to_dev(w, fdt), to_dev(X, fdt), to_dev(dY, bdt)
    dX_sep, dX = to_dev(dX0, bdt), to_dev(dX0, bdt)
    ops.rms_norm_bwd_x(n_rows, n_cols, 1e-5, wsd, rmsd, wd, Xd, dYd, dX_sep)
    dW0 = fill(bdt, (n_cols,), 5)
    if sums:
        dW = torch.full((n_cols,), float("nan"), device="cuda")                  # overwritten, nothing read
    else:
        dW = to_dev(dW0, bdt)
        ref = O.rms_norm_bwd_w(fdt, bdt, rms, X, dY, dW0, n_blocks=0)
    ops.rms_norm_bwd_x_w(n_rows, n_cols, 1e-5, wsd, rmsd, wd, Xd, dYd, dX, dW, sums=sums)
    torch.cuda.synchronize()
    assert torch.equal(dX.view(torch.uint8), dX_sep.view(torch.uint8)), "dX differs from rms_norm_bwd_x"
    if sums:
        exact = (f32(dY, bdt).astype(np.float64) * f32(X, fdt).astype(np.float64) * rms.astype(np.float64)[:, None]).sum(0)
        got = dW.cpu().numpy()
        assert np.all(np.abs(got - exact) <= 2e-5 * np.maximum(np.abs(exact), np.sqrt(n_rows))), float(np.abs(got - exact).max())
    else:
        check_lowp(to_host(dW, bdt), ref, bdt, "rms_norm_bwd_x_w dW", rel=rel_for(bdt) if bdt != O.FP32 else 2e-5, scale=float(np.sqrt(n_rows)))
    # deterministic: a second run gives identical bits
    dX2, dW2 = to_dev(dX0, bdt), (torch.empty_like(dW) if sums else to_dev(dW0, bdt))
    ops.rms_norm_bwd_x_w(n_rows, n_cols, 1e-5, wsd, rmsd, wd, Xd, dYd, dX2, dW2, sums=sums)
    torch.cuda.synchronize()
    assert torch.equal(dW2.view(torch.uint8), dW.view(torch.uint8)) and torch.equal(dX2.view(torch.uint8), dX.view(torch.uint8))


# ------------------------------------------------------------------------------------------ RoPE

ROPE_CASES = [  # tokens, n_heads, n_kv_heads, head_dim, theta, max_pos
    (64, 32, 8, 128, 500000, 8192), (7, 4, 1, 64, 10000, 4096), (1, 1, 1, 8, 10000, 10), (129, 8, 8, 128, 500000, 131072),
    (33, 16, 2, 256, 1000000, 8192), (5, 3, 0, 32, 10000, 100),
]


@pytest.mark.parametrize("bwd", [False, True], ids=["fwd", "bwd"])
@pytest.mark.parametrize("dt", FWD_DTS, ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("case", ROPE_CASES, ids=str)
def test_rope(ops, dt, case, bwd):
    if bwd and dt not in BWD_DTS:
        pytest.skip("rope_bwd_x exists for fp32/fp16/bf16 only")
    tokens, nh, nkv, hd, theta, max_pos = case
    model_dim, kv_dim = nh * hd, max(nkv, 1) * hd
    rng = np.random.default_rng(7)
    pos = rng.integers(0, max_pos, tokens).astype(np.int32)
    Xq, Xk = fill(dt, (tokens, model_dim), 1), fill(dt, (tokens, kv_dim), 2)
    rq, rk = O.rope(dt, model_dim, hd, nkv, theta, pos, Xq, Xk, bwd=bwd)
    q, k = to_dev(Xq, dt), to_dev(Xk, dt)
    fn = ops.rope_bwd_x if bwd else ops.rope
    fn(tokens * model_dim, model_dim, hd, nkv, theta, torch.from_numpy(pos).cuda(), q, k)
    torch.cuda.synchronize()
    # a rotated pair mixes two ~N(0,1) values: absolute floor = rms of the tensor (default scale)
    check_lowp(to_host(q, dt), rq, dt, "rope q", rel=rel_for(dt) if dt != O.FP32 else 1e-4)
    if nkv:
        check_lowp(to_host(k, dt), rk, dt, "rope k", rel=rel_for(dt) if dt != O.FP32 else 1e-4)
    else:
        assert np.array_equal(to_host(k, dt), Xk), "K must be untouched when num_kv_heads == 0"


# ------------------------------------------------------------------------------------------ SwiGLU

SWIGLU_SHAPES = [(64, 14336), (7, 1000), (1, 8), (33, 4104), (0, 128)]


@pytest.mark.parametrize("dt", FWD_DTS, ids=lambda d: DT_NAME[d])
@pytest.mark.parametrize("shape", SWIGLU_SHAPES, ids=str)
def test_swiglu_fwd(ops, dt, shape):
    x1, x3 = fill(dt, shape, 1), fill(dt, shape, 2)
    ref = O.swiglu(dt, x1, x3)
    out = torch.empty_like(to_dev(x1, dt))
    ops.swiglu(shape[0], shape[1], to_dev(x1, dt), to_dev(x3, dt), out)
    torch.cuda.synchronize()
    if shape[0]:
        check_lowp(to_host(out, dt), ref, dt, "swiglu out", rel=rel_for(dt))


@pytest.mark.parametrize("pair", PAIRS, ids=lambda p: f"{DT_NAME[p[0]]}_{DT_NAME[p[1]]}")
@pytest.mark.parametrize("shape", SWIGLU_SHAPES, ids=str)
def test_swiglu_bwd_x(ops, pair, shape):
    fdt, bdt = pair
    x1, x3, dY = fill(fdt, shape, 1), fill(fdt, shape, 2), fill(bdt, shape, 3)
    r1, r3 = O.swiglu_bwd_x(fdt, bdt, x1, x3, dY)
    d1 = torch.empty_like(to_dev(dY, bdt))
    d3 = torch.empty_like(d1)
    ops.swiglu_bwd_x(shape[0], shape[1], to_dev(x1, fdt), to_dev(x3, fdt), to_dev(dY, bdt), d1, d3)
    torch.cuda.synchronize()
    if shape[0]:
        check_lowp(to_host(d1, bdt), r1, bdt, "swiglu dX_w1", rel=rel_for(bdt))
        check_lowp(to_host(d3, bdt), r3, bdt, "swiglu dX_w3", rel=rel_for(bdt))


# ------------------------------------------------------------------------------------------ softmax / cross entropy

SOFTMAX_SHAPES = [(16, 128256), (33, 1024), (4, 32000), (2, 64), (3, 8), (5, 4104), (1, 200000), (2, 262144), (7, 50304)]


@pytest.mark.parametrize("pair", PAIRS, ids=lambda p: f"{DT_NAME[p[0]]}_{DT_NAME[p[1]]}")
@pytest.mark.parametrize("shape", SOFTMAX_SHAPES, ids=str)
def test_softmax(ops, pair, shape):
    fdt, bdt = pair
    X = fill(fdt, shape, 11, 0.0, 2.0)
    ref = O.softmax(fdt, bdt, X)
    out = torch.empty(shape, dtype=to_dev(np.zeros(1, O.NP_OF[bdt]), bdt).dtype, device="cuda")
    ops.softmax(shape[0], shape[1], to_dev(X, fdt), out)
    torch.cuda.synchronize()
    # probabilities span many decades: the floor is the smallest normal step the type resolves near 1/n_cols
    frac = check_lowp(to_host(out, bdt), ref, bdt, "softmax out", rel=rel_for(bdt) if bdt != O.FP32 else 1e-4, scale=1.0 / shape[1])
    assert bdt == O.FP32 or frac > 0.9, f"only {frac:.3f} of the probabilities are bit-identical to the oracle"


@pytest.mark.parametrize("bdt", BWD_DTS, ids=lambda d: DT_NAME[d])
def test_cross_entropy_step_is_bit_exact(ops, bdt):
    n_rows, n_cols = 257, 4104
    P = O.softmax(bdt, bdt, fill(bdt, (n_rows, n_cols), 5, 0.0, 2.0))
    labels = O.fill_labels(n_rows, 9, n_cols)
    labels[3] = n_cols - 1
    labels[4] = 0
    ref = O.cross_entropy_loss(bdt, P, labels)
    pd = to_dev(P, bdt)
    ops.cross_entropy_loss(n_rows, n_cols, pd, torch.from_numpy(labels.view(np.int32)).cuda())
    torch.cuda.synchronize()
    got = to_host(pd, bdt)
    assert np.array_equal(got, ref), "cross-entropy step must touch exactly pred[r, labels[r]]"
    changed = np.argwhere(got != P)
    assert len(changed) == n_rows and np.array_equal(changed[:, 1], labels.astype(np.int64))


@pytest.mark.parametrize("pair", [(O.BF16, O.BF16), (O.FP16, O.FP16), (O.FP32, O.FP32), (O.E4M3, O.BF16)],
                         ids=lambda p: f"{DT_NAME[p[0]]}_{DT_NAME[p[1]]}")
@pytest.mark.parametrize("shape", [(64, 128256), (33, 1024), (5, 4104), (3, 8), (4, 32000)], ids=str)
def test_fused_softmax_cross_entropy(ops, pair, shape):
    fdt, bdt = pair
    n_rows, n_cols = shape
    X = fill(fdt, shape, 21, 0.0, 2.0)
    labels = O.fill_labels(n_rows, 22, n_cols)
    if n_rows > 2:
        labels[1] = n_cols + 5          # out-of-range label: row is left as plain softmax and not counted
    ref_dl, ref_rl, ref_ls = O.softmax_cross_entropy(fdt, bdt, X, labels)
    Xd, ld = to_dev(X, fdt), torch.from_numpy(labels.view(np.int32)).cuda()
    tdt = to_dev(np.zeros(1, O.NP_OF[bdt]), bdt).dtype
    dl = torch.empty(shape, dtype=tdt, device="cuda")
    row_loss = torch.full((n_rows,), float("nan"), device="cuda")
    loss_sum = torch.full((2,), float("nan"), device="cuda")
    ops.softmax_cross_entropy(n_rows, n_cols, Xd, ld, dl, row_loss, loss_sum)
    # the two-kernel path of the reference API must give the same bits
    two = torch.empty(shape, dtype=tdt, device="cuda")
    ops.softmax(n_rows, n_cols, Xd, two)
    ops.cross_entropy_loss(n_rows, n_cols, two, ld)
    torch.cuda.synchronize()
    assert torch.equal(dl.view(torch.uint8), two.view(torch.uint8)), "fused result differs from softmax + cross_entropy_loss"
    check_lowp(to_host(dl, bdt), ref_dl, bdt, "dlogits", rel=rel_for(bdt) if bdt != O.FP32 else 1e-4, scale=1.0 / n_cols)
    # label indexing, bit-exact: the only negative entries are at [r, labels[r]]
    neg = np.argwhere(f32(to_host(dl, bdt), bdt) < 0)
    valid = labels < n_cols
    assert np.array_equal(neg[:, 0], np.nonzero(valid)[0]) and np.array_equal(neg[:, 1], labels[valid].astype(np.int64))
    check_f32(row_loss.cpu().numpy(), ref_rl, "row_loss", rel=1e-5, scale=1.0)
    ls = loss_sum.cpu().numpy()
    assert ls[1] == ref_ls[1] == valid.sum()
    check_f32(ls[:1], ref_ls[:1], "loss_sum", rel=1e-5)
    # loss only (row_loss = NULL uses the workspace), and gradient only (both NULL)
    loss_sum2 = torch.zeros(2, device="cuda")
    dl2 = torch.empty_like(dl)
    ops.softmax_cross_entropy(n_rows, n_cols, Xd, ld, dl2, None, loss_sum2)
    dl3 = torch.empty_like(dl)
    ops.softmax_cross_entropy(n_rows, n_cols, Xd, ld, dl3, None, None)
    torch.cuda.synchronize()
    assert torch.equal(loss_sum2, loss_sum) and torch.equal(dl2.view(torch.uint8), dl.view(torch.uint8)) and torch.equal(dl3.view(torch.uint8), dl.view(torch.uint8))


# ------------------------------------------------------------------------------------------ argument checking

def test_bad_arguments_are_rejected(ops):
    import ctypes
    from dataflow_lib_b200 import _lib
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    pos = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="must be even"):
        ops.rope(4 * 63, 63, 63, 0, 10000, pos, x, x)                          # pairs need an even head_dim
    with pytest.raises(RuntimeError, match="datatype"):
        ops.swiglu_bwd_x(4, 64, x, x, x.float(), x.float(), x.float())
    with pytest.raises(RuntimeError, match="workspace"):
        ops.rms_norm_bwd_w(4, 64, 1e-5, torch.ones(4, device="cuda"), x, x, w.clone(), workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(RuntimeError, match="bad shape"):
        ops.rms_norm(4, 0, 1e-5, w, x, x.clone())
    # a pointer that is not even aligned to its element (an odd address for a 16-bit tensor) is refused before anything is launched
    L, BF = _lib.lib, 5
    odd = x.data_ptr() + 1
    assert L.dfb200_swiglu(BF, 1, 8, odd, x.data_ptr(), x.data_ptr(), None) == -1 and "element size" in _lib.last_error()
    assert L.dfb200_rms_norm(BF, 1, 8, ctypes.c_float(1e-5), w.data_ptr(), odd, x.data_ptr(), None, None, None) == -1
    assert L.dfb200_softmax(BF, BF, 1, 8, odd, x.data_ptr(), None) == -1
    torch.cuda.synchronize()


def test_no_bounded_wait_gave_up(ops):
    """Kernels that wait on asynchronous copies record a status word when a wait runs out; after all the tests above it is 0."""
    from dataflow_lib_b200 import _lib
    import ctypes
    words = (ctypes.c_uint * 8)()
    rc = _lib.lib.dfb200_read_kernel_status(None, words, 8)
    assert rc == 0, (rc, list(words), _lib.last_error())


def test_bounded_wait_gives_up_and_reports():
    """A device-side wait that can never complete returns at its limit, the kernel ends, the status word names the wait, and the context
    keeps working afterwards (no trap, no hang: the failure is made by leaving a barrier without its arrival)."""
    import ctypes
    import time
    from dataflow_lib_b200 import _lib, ops as _ops
    L = _lib.lib
    words = (ctypes.c_uint * 8)()
    assert L.dfb200_read_kernel_status(None, words, 8) == 0                  # clean before
    t0 = time.time()
    assert L.dfb200_selftest_bounded_wait(7, None) == 1, _lib.last_error()
    assert 1.0 < time.time() - t0 < 20.0                                      # the limit is two seconds
    assert L.dfb200_read_kernel_status(None, words, 8) == 0x7e57 and words[7] == 0x7e57 and not any(words[i] for i in range(7))
    assert L.dfb200_read_kernel_status(None, words, 8) == 0                  # cleared by the read
    x = torch.randn(64, 256, device="cuda").bfloat16()
    out = torch.empty_like(x)
    _ops.swiglu(64, 256, x, x, out)                                           # the context is still usable
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
