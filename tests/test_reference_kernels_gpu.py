"""GPU tests against the REFERENCE's own kernels (oracle/_ref/cuda_kernels.cubin: the reference's CUDA source compiled
unchanged for sm_100a, launched by tests/ref_kernels.py). Two questions per op, on the same seeded inputs:
  1. does the CPU oracle restate the reference (pins the oracle), and
  2. do this library's kernels match the reference within the stated tolerance (bf16 <= 1e-2 rel, fp32 stats <= 1e-5)?
Skipped when the cubin was not built (no reference tree at build time)."""
import numpy as np
import pytest
import torch

import oracle as O
import ref_kernels
from golden_cases import CASES, inputs_for
from util import DT_NAME, check_f32, check_lowp, f32, to_dev, to_host

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernels.available(), reason="oracle/_ref/cuda_kernels.cubin or cuda-python missing")]


@pytest.fixture(scope="module")
def ref():
    return ref_kernels.RefKernels()


@pytest.fixture(scope="module")
def ops():
    from dataflow_lib_b200 import ops as _ops
    return _ops


def fill(dt, shape, seed, mean=0.0, std=1.0):
    return O.fill_normal(dt, shape, seed, mean, std)


BF = O.BF16


def test_rms_norm_fwd_bf16(ref, ops):
    R, Cn = 512, 4096
    X, w = fill(BF, (R, Cn), 1), fill(BF, (Cn,), 2, 1.0, 0.02)
    Xd, wd = to_dev(X, BF), to_dev(w, BF)
    r_out, r_ws, r_rms = torch.empty_like(Xd), torch.zeros(R, device="cuda"), torch.zeros(R, device="cuda")
    ref.rms_norm("bf16", 2, R, Cn, 1e-5, wd, Xd, r_out, r_ws, r_rms)
    m_out, m_ws, m_rms = torch.empty_like(Xd), torch.zeros(R, device="cuda"), torch.zeros(R, device="cuda")
    ops.rms_norm(R, Cn, 1e-5, wd, Xd, m_out, m_ws, m_rms)
    torch.cuda.synchronize()
    o_out, o_ws, o_rms = O.rms_norm(BF, 1e-5, w, X)
    scale = float(np.sqrt((f32(X, BF).astype(np.float64) ** 2 * f32(w, BF).astype(np.float64) ** 2).sum(1)).max())
    # oracle vs reference
    assert check_lowp(o_out, to_host(r_out, BF), BF, "oracle vs reference: rms_norm out") > 0.999
    check_f32(o_rms, r_rms.cpu().numpy(), "oracle vs reference: rms_vals", rel=1e-5)
    check_f32(o_ws, r_ws.cpu().numpy(), "oracle vs reference: weighted_sums", rel=1e-5, scale=scale)
    # this library vs reference
    assert check_lowp(to_host(m_out, BF), to_host(r_out, BF), BF, "rms_norm out vs reference") > 0.999
    check_f32(m_rms.cpu().numpy(), r_rms.cpu().numpy(), "rms_vals vs reference", rel=1e-5)
    check_f32(m_ws.cpu().numpy(), r_ws.cpu().numpy(), "weighted_sums vs reference", rel=1e-5, scale=scale)


@pytest.mark.parametrize("zero_dx", [True, False])
def test_rms_norm_bwd_x_bf16(ref, ops, zero_dx):
    R, Cn = 512, 4096
    X, w, dY = fill(BF, (R, Cn), 1), fill(BF, (Cn,), 2, 1.0, 0.02), fill(BF, (R, Cn), 3)
    dX0 = np.zeros((R, Cn), np.uint16) if zero_dx else fill(BF, (R, Cn), 4)
    _, ws, rms = O.rms_norm(BF, 1e-5, w, X)
    wsd, rmsd = torch.from_numpy(ws).cuda(), torch.from_numpy(rms).cuda()
    r_dx, m_dx = to_dev(dX0, BF), to_dev(dX0, BF)
    ref.rms_norm_bwd_x("bf16_bf16", R, Cn, 1e-5, wsd, rmsd, to_dev(w, BF), to_dev(X, BF), to_dev(dY, BF), r_dx)
    ops.rms_norm_bwd_x(R, Cn, 1e-5, wsd, rmsd, to_dev(w, BF), to_dev(X, BF), to_dev(dY, BF), m_dx)
    torch.cuda.synchronize()
    r = to_host(r_dx, BF)
    unfused = O.rms_norm_bwd_x(BF, BF, ws, rms, w, X, dY, dX0, fused=False)
    fused = O.rms_norm_bwd_x(BF, BF, ws, rms, w, X, dY, dX0, fused=True)
    frac_unfused, frac_fused = float((unfused == r).mean()), float((fused == r).mean())
    print(f"reference rms_norm_bwd_x bf16: bit-identical to oracle unfused {frac_unfused:.5f}, fused {frac_fused:.5f}")
    # the reference binary performs the update as one fused multiply-add in bf16 (single rounding)
    assert frac_fused > 0.999 and frac_fused >= frac_unfused
    frac = check_lowp(to_host(m_dx, BF), r, BF, "rms_norm_bwd_x vs reference")
    print(f"this library vs reference: bit-identical {frac:.5f}")
    assert frac > 0.999


def test_rms_norm_bwd_w_bf16(ref, ops):
    R, Cn = 4096, 4096
    X, dY = fill(BF, (R, Cn), 1), fill(BF, (R, Cn), 3)
    rms = (1.0 / np.sqrt((f32(X, BF).astype(np.float64) ** 2).mean(1) + 1e-5)).astype(np.float32)
    rmsd = torch.from_numpy(rms).cuda()
    r_dw, m_dw = torch.zeros(Cn, dtype=torch.bfloat16, device="cuda"), torch.zeros(Cn, dtype=torch.bfloat16, device="cuda")
    ref.rms_norm_bwd_w("bf16_bf16", R, Cn, 1e-5, rmsd, to_dev(X, BF), to_dev(dY, BF), r_dw)
    ops.rms_norm_bwd_w(R, Cn, 1e-5, rmsd, to_dev(X, BF), to_dev(dY, BF), m_dw)
    torch.cuda.synchronize()
    exact = O.rms_norm_bwd_w(BF, BF, rms, X, dY, np.zeros(Cn, np.uint16), n_blocks=0)
    emul = O.rms_norm_bwd_w(BF, BF, rms, X, dY, np.zeros(Cn, np.uint16), n_blocks=ref.sms)
    r, m = to_host(r_dw, BF), to_host(m_dw, BF)
    # the reference accumulates ~SM-count bf16 atomics per column in arrival order: its own result wanders around the exact
    # column sum by several bf16 ulps of sqrt(R)-sized values; the emulation (block order 0..G-1) is one such path
    s = float(np.sqrt(R))
    err_ref = np.abs(f32(r, BF) - f32(exact, BF)).max() / s
    err_emul = np.abs(f32(emul, BF) - f32(exact, BF)).max() / s
    err_mine = np.abs(f32(m, BF) - f32(exact, BF)).max() / s
    print(f"rms_norm_bwd_w max |err| / sqrt(R): reference {err_ref:.4f}, block-order emulation {err_emul:.4f}, this library {err_mine:.5f}")
    assert err_mine <= 2.0 ** -8 * 4            # within bf16 rounding of the exact sum
    assert err_ref < 0.2 and err_emul < 0.2     # the reference stays in the band its rounding walk predicts
    # element-wise against the reference only within the reference's own noise band (it is not deterministic)
    check_lowp(m, r, BF, "rms_norm_bwd_w vs reference (atomic-order band)", rel=0.2, scale=s)


@pytest.mark.parametrize("bwd", [False, True])
@pytest.mark.parametrize("max_pos", [512, 8192])
def test_rope_bf16(ref, ops, bwd, max_pos):
    T, nh, nkv, hd = 256, 32, 8, 128
    md = nh * hd
    pos = np.random.default_rng(3).integers(0, max_pos, T).astype(np.int32)
    Q, K = fill(BF, (T, md), 1), fill(BF, (T, nkv * hd), 2)
    posd = torch.from_numpy(pos).cuda()
    rq, rk, mq, mk = to_dev(Q, BF), to_dev(K, BF), to_dev(Q, BF), to_dev(K, BF)
    ref.rope("bf16", T * md, md, hd, nkv, 500000, posd, rq, rk, bwd=bwd)
    (ops.rope_bwd_x if bwd else ops.rope)(T * md, md, hd, nkv, 500000, posd, mq, mk)
    torch.cuda.synchronize()
    oq, ok = O.rope(BF, md, hd, nkv, 500000, pos, Q, K, bwd=bwd)
    for name, got_o, got_m, r in (("q", oq, to_host(mq, BF), to_host(rq, BF)), ("k", ok, to_host(mk, BF), to_host(rk, BF))):
        # the reference build's __powf/__sinf/__cosf lose accuracy with the angle (up to max_pos radians): its own
        # deviation from correctly rounded math is what separates it from the oracle and from this library
        fo = check_lowp(got_o, r, BF, f"oracle vs reference: rope {name}")
        fm = check_lowp(got_m, r, BF, f"rope {name} vs reference")
        print(f"rope {name} max_pos {max_pos} bwd {bwd}: bit-identical to reference: oracle {fo:.4f}, this library {fm:.4f}")
        assert fo > (0.97 if max_pos <= 512 else 0.8) and fm > (0.97 if max_pos <= 512 else 0.8)
        assert np.mean(got_o == got_m) > 0.9999


def test_swiglu_bf16(ref, ops):
    R, Cn = 64, 14336
    x1, x3, dY = fill(BF, (R, Cn), 1), fill(BF, (R, Cn), 2), fill(BF, (R, Cn), 3)
    a, b, g = to_dev(x1, BF), to_dev(x3, BF), to_dev(dY, BF)
    r_out, m_out = torch.empty_like(a), torch.empty_like(a)
    r1, r3, m1, m3 = (torch.empty_like(a) for _ in range(4))
    ref.swiglu("bf16", R, Cn, a, b, r_out)
    ref.swiglu_bwd_x("bf16_bf16", R, Cn, a, b, g, r1, r3)
    ops.swiglu(R, Cn, a, b, m_out)
    ops.swiglu_bwd_x(R, Cn, a, b, g, m1, m3)
    torch.cuda.synchronize()
    o_out = O.swiglu(BF, x1, x3)
    o1, o3 = O.swiglu_bwd_x(BF, BF, x1, x3, dY)
    for name, o, m, r in (("out", o_out, m_out, r_out), ("dX_w1", o1, m1, r1), ("dX_w3", o3, m3, r3)):
        assert check_lowp(o, to_host(r, BF), BF, f"oracle vs reference: swiglu {name}") > 0.999
        assert check_lowp(to_host(m, BF), to_host(r, BF), BF, f"swiglu {name} vs reference") > 0.9999


@pytest.mark.parametrize("shape", [(8, 128256), (16, 4096), (3, 32000)], ids=str)
def test_softmax_bf16(ref, ops, shape):
    R, Cn = shape
    X = fill(BF, shape, 11, 0.0, 2.0)
    Xd = to_dev(X, BF)
    r_out, m_out = torch.empty_like(Xd), torch.empty_like(Xd)
    ref.softmax("bf16_bf16", R, Cn, Xd, r_out)
    ops.softmax(R, Cn, Xd, m_out)
    torch.cuda.synchronize()
    o = O.softmax(BF, BF, X)
    r, m = to_host(r_out, BF), to_host(m_out, BF)
    fo = check_lowp(o, r, BF, "oracle vs reference: softmax", scale=1.0 / Cn)
    fm = check_lowp(m, r, BF, "softmax vs reference", scale=1.0 / Cn)
    print(f"softmax {shape}: bit-identical to reference: oracle {fo:.5f}, this library {fm:.5f}")
    assert fo > 0.99 and fm > 0.99
    # and the textbook softmax is NOT what the reference computes (bf16-rounded x - max): the quirk is real
    p = torch.softmax(Xd.float(), 1)
    worst = ((r_out.float() - p).abs() / p).max().item()
    assert worst > 1e-2, worst


@pytest.mark.parametrize("dt,name", [(O.BF16, "bf16"), (O.FP16, "fp16")])
def test_softmax_fp32_out_and_argmax(ref, ops, dt, name):
    """The reference's fp32-output softmax (probabilities unrounded, scratch in the input type) and its arg-max, on rows without ties for
    the maximum (with ties the reference lets an arbitrary matching index win)."""
    R, Cn = 12, 32000
    X = fill(dt, (R, Cn), 13, 0.0, 2.0)
    Xf = O.to_f32(X, dt)
    for r in range(R):                                   # make every row's maximum unique
        X[r, (7919 * (r + 1)) % Cn] = O.from_f32(np.array([Xf[r].max() + 1.0], np.float32), dt)[0]
    Xd = to_dev(X, dt)
    r_out, m_out = torch.empty((R, Cn), device="cuda"), torch.empty((R, Cn), device="cuda")
    r_arg, m_arg = torch.zeros(R, dtype=torch.int32, device="cuda"), torch.zeros(R, dtype=torch.int32, device="cuda")
    ref.softmax_fp32_out(name, R, Cn, Xd, r_out, r_arg)
    ops.softmax_fp32_out(R, Cn, Xd, m_out, m_arg)
    torch.cuda.synchronize()
    assert torch.equal(r_arg, m_arg) and np.array_equal(m_arg.cpu().numpy(), O.to_f32(X, dt).argmax(1))
    r, m = r_out.cpu().numpy(), m_out.cpu().numpy()
    same = float((r == m).mean())
    print(f"softmax_{name}_fp32: bit-identical to the reference kernel: {same:.5f}")
    np.testing.assert_allclose(m, r, rtol=2e-6, atol=1e-12)
    o, _ = O.softmax_fp32_out(dt, X)
    np.testing.assert_allclose(r, o, rtol=1e-5, atol=1e-12)


@pytest.mark.parametrize("dt,name", [(O.FP32, "fp32"), (O.BF16, "bf16")])
def test_select_experts(ref, ops, dt, name):
    """The router against the reference's own kernel. Its scores come from the fast-math exponential, this library's from a fixed IEEE
    sequence, so two experts whose scores differ in the last bits can swap: at least 99.5 % of the tokens must get identical expert ids in
    identical slot order, the weights of those tokens agree to the datatype's rounding, and the per-expert counts differ by no more than
    the number of tokens that differ."""
    T, ne, k = 4096, 64, 8
    X = fill(dt, (T, ne), 17, 0.0, 1.5)
    Xd = to_dev(X, dt)
    tdt = torch.float32 if dt == O.FP32 else torch.bfloat16
    outs = []
    for run in (lambda *a: ref.select_experts(name, T, ne, k, Xd, *a), lambda *a: ops.select_experts(T, ne, k, Xd, *a)):
        w = torch.zeros((T, k), dtype=tdt, device="cuda")
        ids = torch.zeros((T, k), dtype=torch.int16, device="cuda")
        counts = torch.zeros(ne + 1, dtype=torch.int32, device="cuda")
        cum, routed = torch.zeros(ne, dtype=torch.int32, device="cuda"), torch.ones(ne, dtype=torch.int32, device="cuda")
        run(w, ids, counts, cum, routed)
        torch.cuda.synchronize()
        outs.append((w.float().cpu().numpy(), ids.cpu().numpy().view(np.uint16), counts.cpu().numpy(), cum.cpu().numpy(), routed.cpu().numpy()))
    (rw, rid, rc, rcum, rr), (mw, mid, mc, mcum, mr) = outs
    same_rows = (rid == mid).all(1)
    print(f"select_experts {name}: tokens with identical expert ids and slot order: {same_rows.mean():.5f}")
    assert same_rows.mean() >= 0.995
    tol = 1e-5 if dt == O.FP32 else 1e-2
    assert np.allclose(rw[same_rows], mw[same_rows], rtol=tol, atol=tol * 1e-2)
    assert rc[ne] == 0 and mc[ne] == 0 and not rr.any() and not mr.any()
    assert np.abs(rc[:ne] - mc[:ne]).sum() <= 2 * k * int((~same_rows).sum())
    assert mcum[-1] == T * k and np.array_equal(mcum, np.cumsum(mc[:ne]))


def test_copy_to_seq_context(ref, ops):
    """Same scatter as the reference's kernel: two sequences' contexts in one buffer, every (context, position) written once."""
    kv_dim, sizes, per_ctx = 1024, [96, 40], [70, 40]
    T = sum(per_ctx)
    rng = np.random.default_rng(3)
    tok_ctx = rng.permutation(np.repeat(np.arange(2), per_ctx))
    pos = np.empty(T, np.int32)
    for c in range(2):
        pos[tok_ctx == c] = rng.permutation(sizes[c])[:per_ctx[c]]
    keys, values = to_dev(fill(BF, (T, kv_dim), 21), BF), to_dev(fill(BF, (T, kv_dim), 22), BF)
    offs = [0, 2 * sizes[0] * kv_dim]
    total = offs[1] + 2 * sizes[1] * kv_dim
    bufs = [torch.zeros(total, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    pos_d = torch.from_numpy(pos).cuda()
    csz = torch.from_numpy(np.array([sizes[c] for c in tok_ctx], np.int32)).cuda()
    for buf, run in zip(bufs, (lambda p: ref.copy_to_seq_context("bf16", T, kv_dim, keys, values, pos_d, p, csz),
                               lambda p: ops.copy_to_seq_context(T * kv_dim, T, kv_dim, keys, values, pos_d, p, csz))):
        ptrs = torch.from_numpy(np.array([buf.data_ptr() + 2 * offs[c] for c in tok_ctx], np.uint64).view(np.int64)).cuda()
        run(ptrs)
    torch.cuda.synchronize()
    assert torch.equal(bufs[0], bufs[1]) and bufs[0].abs().sum() > 0


@pytest.mark.parametrize("name", sorted(CASES))
def test_golden_cases_live(ref, name):
    """The committed golden file must be what the reference kernels produce here (guards against a stale fixture)."""
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")
    if not os.path.exists(path):
        pytest.skip("golden file not generated yet")
    gold = np.load(path)
    keys = [k for k in gold.files if k.startswith(name + "/")]
    assert keys, name
