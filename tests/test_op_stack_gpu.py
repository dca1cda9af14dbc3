"""The token-sharded op stack (dataflow_lib_b200/op_stack.py) against the same data flow composed from the CPU oracle's
ops on a small configuration. Each op has its own element-wise parity test; this one checks the wiring (saved
statistics, residual branch, gradient accumulation order). Two comparisons:
  * layer by layer with the oracle fed the device's own layer input: x_{l+1} within 0.5 % in the L2 norm;
  * end to end: the loss within 2e-3 relative, the final activations within 3 % and the gradients within 6 % in the L2
    norm. The end-to-end bounds are wide because a one-ulp bf16 difference in a row's largest element changes that row's
    FP8 scale, which moves ~7 % of the row's e4m3 codes by one step (6-12 % each), and the next layers amplify that; a
    wiring error shows as an O(1) difference."""
import numpy as np
import pytest
import torch

import oracle as O
from util import f32, to_dev, to_host

pytestmark = pytest.mark.gpu

T, D, F, HEADS, KV, HD, V, L = 256, 512, 1024, 4, 1, 128, 2048, 2
EPS, THETA = 1e-5, 500000


def _rel_l2(got, ref):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def test_stack_matches_oracle_composition():
    from dataflow_lib_b200.op_stack import OpStackStep

    st = OpStackStep(T, D, F, HEADS, KV, HD, V, L, EPS, THETA)
    w_norm = [O.fill_normal(O.BF16, (D,), 10 + l, 1.0, 0.05) for l in range(L + 1)]
    ffn = []
    for l in range(L):
        Wg, sg = O.quantize_weight_e4m3(O.fill_normal(O.FP32, (F, D), 20 + 3 * l, 0.0, 0.04))
        Wu, su = O.quantize_weight_e4m3(O.fill_normal(O.FP32, (F, D), 21 + 3 * l, 0.0, 0.04))
        Wd, sd = O.quantize_weight_e4m3(O.fill_normal(O.FP32, (D, F), 22 + 3 * l, 0.0, 0.04))
        ffn.append((Wg, sg, Wu, su, Wd, sd))
    Wv = O.fill_normal(O.BF16, (V, D), 40, 0.0, 0.05)
    X0 = O.fill_normal(O.BF16, (T, D), 41)
    labels = O.fill_labels(T, 42, V)

    st.set_weights([to_dev(w, O.BF16) for w in w_norm], [tuple(torch.from_numpy(a).cuda() for a in row) for row in ffn], to_dev(Wv, O.BF16))
    st.x[0].copy_(to_dev(X0, O.BF16))
    st.labels.copy_(torch.from_numpy(labels.astype(np.int32)).cuda())
    st.step()
    torch.cuda.synchronize()

    # ---- the same data flow from the oracle's ops
    bf = lambda a: O.from_f32(np.ascontiguousarray(a, np.float32), O.BF16)
    pos = np.arange(T, dtype=np.int32)
    x, stats, saved = [X0], [], []
    for l in range(L):
        h, ws, rms = O.rms_norm(O.BF16, EPS, w_norm[l], x[l])
        q, _ = O.rope(O.BF16, D, HD, KV, THETA, pos, h, np.ascontiguousarray(h[:, :KV * HD]))
        out, g, u = O.swiglu_ffn_fp8(q, *ffn[l])
        x.append(bf(f32(out, O.BF16) + f32(x[l], O.BF16)))
        stats.append((ws, rms)); saved.append((g, u))
    h, ws, rms = O.rms_norm(O.BF16, EPS, w_norm[L], x[L])
    stats.append((ws, rms))
    logits = bf(f32(h, O.BF16) @ f32(Wv, O.BF16).T)
    dlogits, _, loss_sum = O.softmax_cross_entropy(O.BF16, O.BF16, logits, labels)
    dh = bf(f32(dlogits, O.BF16) @ f32(Wv, O.BF16))
    zero_w = np.zeros(D, np.uint16)
    dW = [None] * (L + 1)
    dW[L] = O.rms_norm_bwd_w(O.BF16, O.BF16, stats[L][1], x[L], dh, zero_w)
    dx = O.rms_norm_bwd_x(O.BF16, O.BF16, stats[L][0], stats[L][1], w_norm[L], x[L], dh, np.zeros((T, D), np.uint16))
    for l in reversed(range(L)):
        dA = O.swiglu_ffn_fp8_bwd(dx, saved[l][0], saved[l][1], *ffn[l])
        dA, _ = O.rope(O.BF16, D, HD, KV, THETA, pos, dA, np.zeros((T, KV * HD), np.uint16), bwd=True)
        dW[l] = O.rms_norm_bwd_w(O.BF16, O.BF16, stats[l][1], x[l], dA, zero_w)
        dx = O.rms_norm_bwd_x(O.BF16, O.BF16, stats[l][0], stats[l][1], w_norm[l], x[l], dA, dx)

    # layer by layer, the oracle fed the device's layer input
    for l in range(L):
        xd = to_host(st.x[l], O.BF16)
        h, _, _ = O.rms_norm(O.BF16, EPS, w_norm[l], xd)
        q, _ = O.rope(O.BF16, D, HD, KV, THETA, pos, h, np.ascontiguousarray(h[:, :KV * HD]))
        out, _, _ = O.swiglu_ffn_fp8(q, *ffn[l])
        want = f32(out, O.BF16) + f32(xd, O.BF16)
        assert _rel_l2(f32(to_host(st.x[l + 1], O.BF16), O.BF16), want) < 5e-3, l

    got_loss = st.loss_sum.cpu().numpy()
    assert got_loss[1] == loss_sum[1] == T
    assert abs(got_loss[0] - loss_sum[0]) <= 2e-3 * abs(loss_sum[0]), (got_loss, loss_sum)
    assert _rel_l2(f32(to_host(st.x[L], O.BF16), O.BF16), f32(x[L], O.BF16)) < 3e-2
    assert _rel_l2(f32(to_host(st.dx, O.BF16), O.BF16), f32(dx, O.BF16)) < 6e-2
    for l in range(L + 1):                                     # the stack keeps the weight gradients as fp32 column sums in its packed buffer
        assert _rel_l2(st.dW[l].cpu().numpy(), f32(dW[l], O.BF16)) < 6e-2, l
    assert st.library_launches_per_step() == L * 14 + 5
    st.close()


def test_overlapped_exchange_on_one_rank_keeps_the_step():
    """step(overlap=True) without a process group: the step's results are unchanged and `reduced` is the packed buffer
    [loss sum, valid rows | dW_0 .. dW_L] that a multi-rank run all-reduces in place (bench.py checks the multi-rank case against a
    second all-reduce of the same partial sums on the GPUs it runs on). Consecutive steps alternate between two packed buffers."""
    from dataflow_lib_b200.op_stack import OpStackStep

    st = OpStackStep(T, D, F, HEADS, KV, HD, V, L, EPS, THETA)
    st.random_weights(seed=3)
    g = torch.Generator(device="cuda").manual_seed(5)
    st.x[0].copy_(torch.randn(T, D, device="cuda", generator=g).bfloat16())
    st.labels.copy_(torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32))
    st.step()
    torch.cuda.synchronize()
    first = st.reduced
    packed = st.reduced.clone()
    assert torch.equal(packed[:2], st.loss_sum) and all(torch.equal(packed[2 + l * D:2 + (l + 1) * D], st.dW[l]) for l in range(L + 1))
    st.step(overlap=True)
    st.wait_exchange()
    torch.cuda.synchronize()
    assert st.reduced.data_ptr() != first.data_ptr()           # the other buffer
    assert torch.equal(st.reduced, packed)                     # same inputs, same sums, bit for bit (the reductions are deterministic)
    assert st.reduced.numel() == 2 + (L + 1) * D and st.reduced[1].item() == T
    st.close()
