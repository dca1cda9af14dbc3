"""Pins the CPU oracle against outputs of the REFERENCE's own CUDA kernels (tests/golden/reference_vectors.npz, produced
on a B200 by tests/golden/make_reference_vectors.py from the reference's kernels compiled unchanged), and checks the
textbook parts of the oracle against PyTorch on the CPU.

Tolerances: the reference is built with --use_fast_math (approximate exp/div/rsqrt/pow/sin/cos) while the oracle uses
libm, so individual low-precision outputs may land on the neighbouring value. The rule is therefore: every element
within 1e-2 relative (absolute floor = tensor RMS, or 1/n_cols for probabilities) AND at least 99 % of elements
bit-identical (97 % for RoPE, whose angle error grows with the position); fp32 statistics within 1e-5 relative."""
import os

import numpy as np
import pytest
import torch

import oracle as O
from golden_cases import CASES, inputs_for
from util import check_f32, check_lowp, f32

GOLD_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")
GOLD = np.load(GOLD_PATH) if os.path.exists(GOLD_PATH) else None


def _rel(dt):
    return {O.FP32: 2e-5, O.FP16: 1e-2, O.BF16: 1e-2}[dt]


@pytest.mark.skipif(GOLD is None, reason="golden reference vectors not generated")
@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_kernel_outputs(name):
    case = CASES[name]
    inp = inputs_for(case)
    op, fdt, bdt = case["op"], case["fdt"], case.get("bdt", case["fdt"])
    g = lambda k: GOLD[f"{name}/{k}"]
    min_same = 0.0 if bdt == O.FP32 else 0.99
    if op == "rms_norm":
        out, ws, rms = O.rms_norm(fdt, 1e-5, inp["w"], inp["X"])
        assert check_lowp(out, g("out"), fdt, name, rel=_rel(fdt)) >= min_same
        check_f32(rms, g("rms"), name + " rms", rel=1e-5)
        terms = np.sqrt((f32(inp["X"], fdt).astype(np.float64) ** 2 * f32(inp["w"], fdt).astype(np.float64) ** 2).sum(1)).max()
        check_f32(ws, g("ws"), name + " ws", rel=1e-5, scale=float(terms))
    elif op == "rms_norm_bwd_x":
        a = O.rms_norm_bwd_x(fdt, bdt, inp["ws"], inp["rms"], inp["w"], inp["X"], inp["dY"], inp["dX"], fused=False)
        b = O.rms_norm_bwd_x(fdt, bdt, inp["ws"], inp["rms"], inp["w"], inp["X"], inp["dY"], inp["dX"], fused=True)
        ref = g("dX")
        best = a if (a == ref).mean() >= (b == ref).mean() else b      # the binary either fuses the multiply-add or not
        assert check_lowp(best, ref, bdt, name, rel=_rel(bdt)) >= min_same
    elif op == "rms_norm_bwd_w":
        exact = O.rms_norm_bwd_w(fdt, bdt, inp["rms"], inp["X"], inp["dY"], inp["dW"], n_blocks=0)
        # 40 rows on >= 40 blocks: one row per block, so the reference result is a chain of 40 roundings in arrival order
        check_lowp(exact, g("dW"), bdt, name, rel=5e-2 if bdt != O.FP32 else 1e-4, scale=float(np.sqrt(40)))
    elif op in ("rope", "rope_bwd_x"):
        q, k = O.rope(fdt, case["model_dim"], case["head_dim"], case["n_kv"], case["theta"], inp["pos"], inp["Q"], inp["K"], bwd=(op == "rope_bwd_x"))
        long_angles = case["max_pos"] > 512
        floor = 0.0 if fdt == O.FP32 else (0.8 if long_angles else 0.97)
        rel = 2e-3 if fdt == O.FP32 else 1e-2          # fp32 shows the fast-math angle error directly
        if fdt == O.FP32 and long_angles:
            rel = 1e-2
        assert check_lowp(q, g("Q"), fdt, name + " Q", rel=rel) >= floor
        assert check_lowp(k, g("K"), fdt, name + " K", rel=rel) >= floor
    elif op == "swiglu":
        tol = max(_rel(fdt) if fdt in (O.FP32, O.FP16, O.BF16) else 0.0, 0.13 if fdt == O.E4M3 else 0.0, 0.26 if fdt == O.E5M2 else 0.0)
        assert check_lowp(O.swiglu(fdt, inp["x1"], inp["x3"]), g("out"), fdt, name, rel=tol) >= min_same
    elif op == "swiglu_bwd_x":
        d1, d3 = O.swiglu_bwd_x(fdt, bdt, inp["x1"], inp["x3"], inp["dY"])
        assert check_lowp(d1, g("d1"), bdt, name + " d1", rel=_rel(bdt)) >= min_same
        assert check_lowp(d3, g("d3"), bdt, name + " d3", rel=_rel(bdt)) >= min_same
    elif op == "softmax":
        out = O.softmax(fdt, bdt, inp["X"])
        assert check_lowp(out, g("out"), bdt, name, rel=_rel(bdt) if bdt != O.FP32 else 1e-4, scale=1.0 / case["shape"][1]) >= min_same
    elif op == "softmax_fp32_out":
        out, arg = O.softmax_fp32_out(fdt, inp["X"])
        np.testing.assert_allclose(out, g("out"), rtol=1e-5, atol=1e-12)
        assert np.array_equal(arg, g("argmax"))
    elif op == "select_experts":
        w, ids, counts, _, _ = O.select_experts(fdt, inp["X"], case["top_k"])
        assert np.array_equal(ids, g("ids"))                       # expert ids and slot order as the reference kernel chose them
        assert np.array_equal(counts, g("counts"))
        check_lowp(w, g("weights"), fdt, name + " weights", rel=_rel(fdt) if fdt != O.FP32 else 1e-5)
    else:
        raise AssertionError(op)


def _bf(a):
    return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).float()


def test_oracle_textbook_parts_against_torch():
    """Where the reference's arithmetic is the textbook formula, the oracle must agree with PyTorch (fp32 on CPU)."""
    X, w = O.fill_normal(O.BF16, (32, 512), 1), O.fill_normal(O.BF16, (512,), 2, 1.0, 0.02)
    out, ws, rms = O.rms_norm(O.BF16, 1e-5, w, X)
    xt, wt = _bf(X), _bf(w)
    r = torch.rsqrt((xt * xt).mean(1) + 1e-5)
    assert torch.equal(((xt * r[:, None]) * wt).bfloat16().float(), _bf(out))
    np.testing.assert_allclose(rms, r.numpy(), rtol=1e-6)
    np.testing.assert_allclose(ws, (xt * wt).sum(1).numpy(), rtol=1e-5, atol=1e-4)
    # swiglu = silu(x1) * x3
    x1, x3 = O.fill_normal(O.BF16, (8, 256), 3), O.fill_normal(O.BF16, (8, 256), 4)
    ref = (torch.nn.functional.silu(_bf(x1)) * _bf(x3)).bfloat16().float()
    got = _bf(O.swiglu(O.BF16, x1, x3))
    assert (ref != got).float().mean() < 1e-3 and torch.allclose(ref, got, rtol=1e-2, atol=1e-3)
    # swiglu backward = autograd of the forward
    a, b = _bf(x1).requires_grad_(), _bf(x3).requires_grad_()
    dY = O.fill_normal(O.BF16, (8, 256), 5)
    (torch.nn.functional.silu(a) * b).backward(_bf(dY))
    d1, d3 = O.swiglu_bwd_x(O.BF16, O.BF16, x1, x3, dY)
    assert torch.allclose(_bf(d1), a.grad, rtol=1e-2, atol=2e-3) and torch.allclose(_bf(d3), b.grad, rtol=1e-2, atol=2e-3)
    # rope: interleaved pairs == multiplication by exp(i * pos * theta^(-2j/hd)); backward == inverse rotation
    T, nh, hd = 8, 2, 64
    Q = O.fill_normal(O.FP32, (T, nh * hd), 6)
    pos = np.arange(T, dtype=np.int32) * 37
    q, _ = O.rope(O.FP32, nh * hd, hd, 0, 10000, pos, Q, Q[:, :0].copy())
    z = torch.view_as_complex(torch.from_numpy(Q).view(T, nh, hd // 2, 2))
    ang = torch.from_numpy(pos).float()[:, None] * (10000.0 ** (-torch.arange(0, hd, 2).float() / hd))[None, :]
    want = torch.view_as_real(z * torch.polar(torch.ones_like(ang), ang)[:, None, :]).reshape(T, nh * hd)
    assert torch.allclose(torch.from_numpy(q), want, rtol=1e-4, atol=1e-4)
    back, _ = O.rope(O.FP32, nh * hd, hd, 0, 10000, pos, q, q[:, :0].copy(), bwd=True)
    np.testing.assert_allclose(back, Q, rtol=1e-5, atol=1e-5)
    # softmax in fp32 is the textbook softmax; cross-entropy step + loss against torch
    L = O.fill_normal(O.FP32, (16, 1000), 7, 0.0, 2.0)
    labels = O.fill_labels(16, 8, 1000)
    dl, row_loss, loss_sum = O.softmax_cross_entropy(O.FP32, O.FP32, L, labels)
    lt = torch.from_numpy(L).requires_grad_()
    loss = torch.nn.functional.cross_entropy(lt, torch.from_numpy(labels.astype(np.int64)), reduction="sum")
    loss.backward()
    np.testing.assert_allclose(dl, lt.grad.numpy(), rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(loss_sum[0], loss.item(), rtol=1e-5)
    assert loss_sum[1] == 16


def test_oracle_rms_norm_bwd_x_is_the_reference_formula_not_the_textbook_gradient():
    """The reference's dX uses sum_j w_j x_j where the true gradient has sum_j dY_j w_j x_j (rms_norm_bwd_x.cu:249):
    the oracle follows the reference; the size of the gap to autograd is asserted so that it stays visible."""
    X, w, dY = O.fill_normal(O.FP32, (16, 256), 1), O.fill_normal(O.FP32, (256,), 2, 1.0, 0.02), O.fill_normal(O.FP32, (16, 256), 3)
    _, ws, rms = O.rms_norm(O.FP32, 1e-5, w, X)
    got = O.rms_norm_bwd_x(O.FP32, O.FP32, ws, rms, w, X, dY, np.zeros_like(X))
    xt, wt = torch.from_numpy(X).requires_grad_(), torch.from_numpy(w)
    ((xt * torch.rsqrt((xt * xt).mean(1, keepdim=True) + 1e-5)) * wt).backward(torch.from_numpy(dY))
    formula = dY * (w[None, :] * rms[:, None] - X * (rms ** 3)[:, None] / 256 * ws[:, None])
    np.testing.assert_allclose(got, formula, rtol=1e-5, atol=1e-6)
    gap = np.abs(got - xt.grad.numpy()).max()
    assert gap > 0.1, gap


def test_oracle_edge_cases():
    """Ragged and tiny shapes, out-of-range labels, thread-count independence."""
    X = O.fill_normal(O.BF16, (5, 40), 9, 0.0, 2.0)                  # n_cols not a multiple of 32
    p = O.softmax(O.BF16, O.BF16, X)
    assert np.all(np.abs(O.to_f32(p, O.BF16).sum(1) - 1.0) < 2e-2)
    labels = np.array([0, 39, 40, 7, 2 ** 31], np.uint32)
    dl, rl, ls = O.softmax_cross_entropy(O.BF16, O.BF16, X, labels)
    assert ls[1] == 3 and rl[2] == 0 and rl[4] == 0 and np.array_equal(dl[2], p[2]) and np.array_equal(dl[4], p[4])
    assert (O.to_f32(dl, O.BF16) < 0).sum() == 3
    big = O.fill_normal(O.BF16, (37, 1000), 10)
    a = O.swiglu(O.BF16, big, big, threads=1)
    b = O.swiglu(O.BF16, big, big, threads=5)
    assert np.array_equal(a, b)
    assert O.rms_norm(O.BF16, 1e-5, big[0], big[:0])[0].shape == (0, 1000)
    # fill is a pure function of (seed, index): a slice equals the slice of the whole
    whole = O.fill_normal(O.BF16, (8, 16), 5)
    assert np.array_equal(O.fill_normal(O.BF16, (4, 16), 5), whole[:4])


# ---- router, embedding, sequence context ------------------------------------------------------------------------

def test_sigmoid_score_is_accurate():
    for x in [-100.0, -88.5, -20.0, -1.0, -1e-3, 0.0, 1e-3, 0.5, 3.0, 17.0, 87.5, 100.0]:
        want = 1.0 / (1.0 + np.exp(-np.float64(x)))
        got = O.sigmoid_score(x)
        assert abs(got - want) <= 4e-7 * max(want, 1e-30) + 1e-38, (x, got, want)
    assert np.isnan(O.sigmoid_score(float("nan")))


def test_select_experts_slot_order_and_ties():
    """Hand-traced cases of the reference's scan (src/ops/nvidia/moe/select_experts.cu:124-153)."""
    X = np.array([[1, 3, 2, 0], [1, 1, 1, 1], [0, 1, 2, 3], [3, 2, 1, 0]], np.float32)
    w, ids, counts, cumsum, routed = O.select_experts(O.FP32, X, 2, threads=1)
    # row 0: e0 -> slot 0, e1 -> slot 1, e2 (2 > 1) evicts slot 0, e3 loses
    # row 1: ties never replace (strict >): the first two experts stay
    # row 2: e2 evicts e0 from slot 0, then e3 evicts e1 from slot 1;  row 3: nothing after the first two wins
    assert ids.tolist() == [[2, 1], [0, 1], [2, 3], [0, 1]]
    s = lambda v: 1.0 / (1.0 + np.exp(-np.float64(v)))
    assert np.allclose(w[0], [s(2) / (s(2) + s(3)), s(3) / (s(2) + s(3))], rtol=1e-6)
    assert np.allclose(w.sum(1), 1.0, rtol=1e-6)
    assert counts.tolist() == [2, 3, 2, 1, 0] and cumsum.tolist() == [2, 5, 7, 8] and not routed.any()


def test_select_experts_matches_a_sort_when_there_are_no_ties():
    T, ne, k = 200, 64, 8
    X = O.fill_normal(O.FP32, (T, ne), 3)
    w, ids, counts, cumsum, _ = O.select_experts(O.FP32, X, k)
    want = np.argsort(-X, axis=1, kind="stable")[:, :k]
    assert np.array_equal(np.sort(ids.astype(np.int64), axis=1), np.sort(want, axis=1))
    sc = 1.0 / (1.0 + np.exp(-X.astype(np.float64)))
    picked = np.take_along_axis(sc, ids.astype(np.int64), axis=1)
    assert np.allclose(w, picked / picked.sum(1, keepdims=True), rtol=2e-6)
    assert np.array_equal(counts[:ne], np.bincount(ids.ravel(), minlength=ne)) and np.array_equal(cumsum, np.cumsum(counts[:ne]))


def test_embedding_and_seq_context_oracle():
    table = O.fill_normal(O.BF16, (50, 24), 1)
    ids = np.array([3, 49, 0, 3], np.uint32)
    assert np.array_equal(O.embedding(O.BF16, ids, table), table[ids])
    keys, values = O.fill_normal(O.BF16, (3, 8), 2), O.fill_normal(O.BF16, (3, 8), 3)
    ctx = [np.zeros((2 * 4, 8), np.uint16), np.zeros((2 * 2, 8), np.uint16)]
    O.copy_to_seq_context(O.BF16, keys, values, [1, 0, 3], ctx, [0, 1, 0], [4, 2])
    assert np.array_equal(ctx[0][1], keys[0]) and np.array_equal(ctx[0][4 + 1], values[0])
    assert np.array_equal(ctx[1][0], keys[1]) and np.array_equal(ctx[1][2 + 0], values[1])
    assert np.array_equal(ctx[0][3], keys[2]) and np.array_equal(ctx[0][4 + 3], values[2])
    assert not ctx[0][[0, 2, 4, 6]].any()


def test_oracle_bf16_loss_is_within_1e5_of_fp64_cross_entropy():
    """The fused op's loss (no reference counterpart) must be the cross entropy of the bf16 logits to 1e-5 relative on the mean,
    although the probabilities beside it keep the reference's bf16 roundings: N(0, 2) logits, a vocabulary-sized row."""
    n_rows, n_cols = 48, 128256
    L = O.fill_normal(O.BF16, (n_rows, n_cols), 77, 0.0, 2.0)
    labels = O.fill_labels(n_rows, 78, n_cols)
    _, row_loss, loss_sum = O.softmax_cross_entropy(O.BF16, O.BF16, L, labels)
    x = torch.from_numpy(O.to_f32(L, O.BF16)).double()
    ce = torch.nn.functional.cross_entropy(x, torch.from_numpy(labels.astype(np.int64)), reduction="none").numpy()
    assert abs(loss_sum[0] / n_rows - ce.mean()) <= 1e-5 * ce.mean()
    assert np.abs(row_loss - ce).max() <= 5e-5 * ce.max()            # per row the rounding inside the exponentials shows a little more
