"""Full-size checks at the benchmark configurations (C1 RMSNorm 4096x4096, C2 the 8192-token Llama-3-8B chain,
C3 fused softmax + cross entropy 16384 x 128256), where the CPU oracle would take too long: size-independent
properties of the ops, plus PyTorch fp32 re-computations on the GPU that model the reference's rounding points.
Inputs: seeded torch normals of the configs' shapes and distributions (synthetic stand-ins for activations)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from dataflow_lib_b200 import ops as _ops
    return _ops


def _randn(shape, seed, std=1.0, mean=0.0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (mean + std * torch.randn(shape, device="cuda", generator=g)).to(dtype)


def _close(got, ref, rel=1e-2, scale=None, flipped_frac=0.0):
    """|got - ref| <= rel * max(|ref|, scale). `flipped_frac` > 0 names the share of elements allowed between rel and 2 rel: those
    whose bf16 INPUT differs by one unit between the device and this fp32 model (two fp32 sums in different orders that straddle a
    rounding boundary), which moves the output by that unit on top of its own rounding."""
    got, ref = got.float(), ref.float()
    assert torch.isfinite(got).all(), "non-finite output"
    s = ref.pow(2).mean().sqrt() if scale is None else scale
    tol = rel * torch.maximum(ref.abs(), torch.as_tensor(s, device=ref.device))
    err = (got - ref).abs()
    bad = err > tol
    if flipped_frac:
        assert bad.float().mean().item() <= flipped_frac, f"{int(bad.sum())}/{bad.numel()} outside {rel} rel"
        bad = err > 2 * tol
    assert not bad.any(), f"{int(bad.sum())}/{bad.numel()} outside {rel} rel"


def test_c1_rms_norm_fwd_bwd(ops):
    R, C, eps = 4096, 4096, 1e-5
    X, w, dY = _randn((R, C), 0), _randn((C,), 1, 0.02, 1.0), _randn((R, C), 2)
    Y, ws, rms = torch.empty_like(X), torch.empty(R, device="cuda"), torch.empty(R, device="cuda")
    ops.rms_norm(R, C, eps, w, X, Y, ws, rms)
    xf, wf, gf = X.float(), w.float(), dY.float()
    r = torch.rsqrt(xf.pow(2).mean(1) + eps)
    assert torch.allclose(rms, r, rtol=1e-5, atol=0)
    assert torch.allclose(ws, (xf * wf).sum(1), rtol=1e-5, atol=1e-3)
    same = (Y == ((xf * r[:, None]) * wf).bfloat16()).float().mean().item()
    assert same > 0.999, same                              # one rounding of an fp32 product: bit-identical up to 1-ulp rsqrt effects
    # backward-x: dX accumulates; reference formula dX += dY * bf16(w r - x r^3 / n * ws), fused multiply-add in bf16
    for dX0 in (torch.zeros_like(X), _randn((R, C), 3)):
        dX = dX0.clone()
        ops.rms_norm_bwd_x(R, C, eps, ws, rms, w, X, dY, dX)
        deriv = (wf * rms[:, None] - (xf * (rms ** 3)[:, None] / C) * ws[:, None]).bfloat16().float()
        want = (dX0.double() + gf.double() * deriv.double()).float().bfloat16()       # exact then one rounding
        assert (dX == want).float().mean().item() > 0.999
        _close(dX, want, rel=2e-2)        # where this fp32 model and the kernel round bf16(deriv) differently, the product moves by ulp(deriv)*|dY|
    # backward-w: exact column sums (fp64) within bf16 rounding; linear in dY (x2 is exact in bf16); accumulates into dW
    dW = torch.zeros(C, dtype=torch.bfloat16, device="cuda")
    ops.rms_norm_bwd_w(R, C, eps, rms, X, dY, dW)
    exact = (gf * xf * rms[:, None]).double().sum(0)
    assert ((dW.double() - exact).abs() <= 2.0 ** -8 * exact.abs() + 2e-3).all()      # bf16 rounding + fp32 summation of 4096 O(1) terms
    dW2 = torch.zeros_like(dW)
    ops.rms_norm_bwd_w(R, C, eps, rms, X, (dY.float() * 2).bfloat16(), dW2)
    assert torch.equal(dW2.float(), dW.float() * 2)
    dW3 = dW.clone()
    ops.rms_norm_bwd_w(R, C, eps, rms, X, dY, dW3)
    assert ((dW3.double() - 2 * exact).abs() <= 2.0 ** -7 * exact.abs() * 2 + 4e-3).all()
    # both gradients in one pass over X and dY (rms_norm_bwd_x_w): dX is the separate op's bit for bit, the weight gradient is the same
    # exact column sum within bf16 rounding, its fp32 form (written, not accumulated) within 2e-5; linear in dY like the separate op
    dX0 = _randn((R, C), 3)
    dX_sep, dX_one, dX_sums = dX0.clone(), dX0.clone(), dX0.clone()
    ops.rms_norm_bwd_x(R, C, eps, ws, rms, w, X, dY, dX_sep)
    dW4, sums = torch.zeros_like(dW), torch.full((C,), float("nan"), device="cuda")
    ops.rms_norm_bwd_x_w(R, C, eps, ws, rms, w, X, dY, dX_one, dW4)
    ops.rms_norm_bwd_x_w(R, C, eps, ws, rms, w, X, dY, dX_sums, sums, sums=True)
    assert torch.equal(dX_one.view(torch.int16), dX_sep.view(torch.int16)) and torch.equal(dX_sums.view(torch.int16), dX_sep.view(torch.int16))
    assert ((dW4.double() - exact).abs() <= 2.0 ** -8 * exact.abs() + 2e-3).all()
    assert ((sums.double() - exact).abs() <= 2e-5 * exact.abs() + 2e-5 * R ** 0.5).all()
    dW5, scratch = torch.zeros_like(dW), dX0.clone()
    ops.rms_norm_bwd_x_w(R, C, eps, ws, rms, w, X, (dY.float() * 2).bfloat16(), scratch, dW5)
    assert torch.equal(dW5.float(), dW4.float() * 2)


def test_c2_rope_roundtrip_and_swiglu(ops):
    T, NH, NKV, HD, F, theta = 8192, 32, 8, 128, 14336, 500000
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    Q, K = _randn((T, NH * HD), 4), _randn((T, NKV * HD), 5)
    q, k = Q.clone(), K.clone()
    ops.rope(T * NH * HD, NH * HD, HD, NKV, theta, pos, q, k)
    # textbook check in fp32: interleaved pairs times exp(i pos theta^(-2j/hd))
    ang = pos.double()[:, None] * (float(theta) ** (-torch.arange(0, HD, 2, device="cuda").double() / HD))[None, :]
    cs, sn = ang.cos().float(), ang.sin().float()
    def rot(x, n_heads):
        x = x.float().view(T, n_heads, HD // 2, 2)
        e, o = x[..., 0], x[..., 1]
        return torch.stack((cs[:, None] * e - sn[:, None] * o, cs[:, None] * o + sn[:, None] * e), -1).view(T, n_heads * HD)
    _close(q, rot(Q, NH).bfloat16())
    _close(k, rot(K, NKV).bfloat16())
    # rotations preserve the norm of every pair (up to two bf16 roundings)
    n0 = Q.float().view(T, -1, 2).pow(2).sum(-1).sqrt()
    n1 = q.float().view(T, -1, 2).pow(2).sum(-1).sqrt()
    assert ((n1 - n0).abs() <= 1.5e-2 * n0 + 1e-2).all()
    # backward is the inverse rotation: fwd then bwd gives the input back within two bf16 roundings
    ops.rope_bwd_x(T * NH * HD, NH * HD, HD, NKV, theta, pos, q, k)
    _close(q, Q, rel=1.6e-2)
    _close(k, K, rel=1.6e-2)
    # swiglu forward/backward against the formulas in fp32
    x1, x3, dY = _randn((T, F), 6), _randn((T, F), 7), _randn((T, F), 8)
    out, d1, d3 = torch.empty_like(x1), torch.empty_like(x1), torch.empty_like(x1)
    ops.swiglu(T, F, x1, x3, out)
    ops.swiglu_bwd_x(T, F, x1, x3, dY, d1, d3)
    a, b, g = x1.float(), x3.float(), dY.float()
    e = torch.exp(-a)
    silu = a / (1 + e)
    assert (out == (silu * b).bfloat16()).float().mean().item() > 0.9999
    _close(out, (silu * b).bfloat16())
    _close(d3, (g * silu).bfloat16())
    _close(d1, (g * (b * (1 + e + a * e)) / ((1 + e) * (1 + e))).bfloat16())


def test_c3_fused_softmax_cross_entropy(ops):
    T, V = 16384, 128256
    g = torch.Generator(device="cuda").manual_seed(9)
    logits = torch.empty(T, V, dtype=torch.bfloat16, device="cuda")
    for i in range(0, T, 2048):                                     # N(0, 2) in slabs to bound temporary memory
        logits[i:i + 2048] = (2.0 * torch.randn(2048, V, device="cuda", generator=g)).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32)
    dl = torch.empty_like(logits)
    row_loss, loss = torch.empty(T, device="cuda"), torch.zeros(2, device="cuda")
    ops.softmax_cross_entropy(T, V, logits, labels, dl, row_loss, loss)
    torch.cuda.synchronize()
    assert loss[1].item() == T
    lab = labels.long()
    worst_sum, neg_count = 0.0, 0
    model_loss = torch.empty(T, device="cuda", dtype=torch.float64)
    for i in range(0, T, 1024):                                     # model of the reference's rounding points, in slabs
        x = logits[i:i + 1024].float()
        d = (x - x.max(1, keepdim=True).values).bfloat16().float()  # x - max rounded to bf16
        e = torch.exp(d)
        pad = (-V) % 1024
        ep = torch.nn.functional.pad(e, (0, pad)).view(1024, -1, 32, 32)            # [row, k, partial index, lane]
        partial = ep.sum(dim=(1, 3)).bfloat16().float()                               # 32 interleaved sums, each rounded to bf16
        total = partial.sum(1).bfloat16().float()                                      # rounded again
        p = (e / total[:, None]).bfloat16()
        want = p.clone()
        rows = torch.arange(1024, device="cuda")
        want[rows, lab[i:i + 1024]] = (p[rows, lab[i:i + 1024]].float() - 1.0).bfloat16()
        got = dl[i:i + 1024]
        frac = (got == want).float().mean().item()
        assert frac > 0.995, (i, frac)
        _close(got, want, rel=1e-2, scale=1.0 / V)
        gf = got.float()
        neg = gf < 0
        neg_count += int(neg.sum())
        assert torch.equal(neg.nonzero()[:, 1], lab[i:i + 1024])                       # label indexing, bit-exact
        worst_sum = max(worst_sum, gf.sum(1).abs().max().item())                       # softmax - onehot sums to ~0 per row
        # the loss keeps none of those roundings but the one inside the exponentials: fp32 sum of the unrounded partials, fp32 x_label - max
        total32 = ep.sum(dim=(1, 3)).sum(1)
        model_loss[i:i + 1024] = (torch.log(total32) - (x - x.max(1, keepdim=True).values)[rows, lab[i:i + 1024]]).double()
    assert neg_count == T and worst_sum < 2e-2
    assert torch.allclose(row_loss.double(), model_loss, rtol=1e-5, atol=0)
    mean_got = loss[0].item() / T
    assert abs(loss[0].item() - row_loss.double().sum().item()) <= 1e-6 * abs(loss[0].item())   # fp64 fixed-order sum of the fp32 row losses
    # the configuration's bound: the mean loss within 1e-5 relative of the cross entropy of these bf16 logits computed in fp64
    ce = 0.0
    for i in range(0, T, 1024):
        ce += torch.nn.functional.cross_entropy(logits[i:i + 1024].double(), lab[i:i + 1024], reduction="sum").item()
    ce /= T
    assert abs(mean_got - ce) <= 1e-5 * abs(ce), (mean_got, ce)


def test_c4_swiglu_ffn_fp8(ops):
    """FP8-weight SwiGLU FFN at 16384 x 4096 x 14336: forward, input gradient and weight gradients. The reference has no such op;
    the checker is the same composition of the quantised arithmetic in fp32 on the GPU (torch matmul, TF32 off, in row slabs):
    every GEMM of the three passes is re-computed from the codes and scales that went into it -- produced by the row / column
    quantisers, which are checked bit for bit against the CPU oracle at small sizes -- and its bf16 output must be within 1e-2 of
    max(|ref|, rms(ref)). At this size every walker of the persistent GEMM takes 24 to 48 tiles."""
    import ctypes
    from dataflow_lib_b200 import _lib
    torch.backends.cuda.matmul.allow_tf32 = False
    T, d, f = 16384, 4096, 14336
    u8 = lambda *s: torch.empty(s, dtype=torch.uint8, device="cuda")
    f32v = lambda n: torch.empty(n, device="cuda")
    bf = lambda *s: torch.full(s, float("nan"), dtype=torch.bfloat16, device="cuda")
    e4 = lambda q: q.view(torch.float8_e4m3fn).float()

    def weight(n_out, n_in, seed):                              # N(0, 0.02) quantised with one fp32 scale per output channel
        g = torch.Generator(device="cuda").manual_seed(seed)
        W = 0.02 * torch.randn(n_out, n_in, device="cuda", generator=g)
        s = W.abs().amax(1) / 448.0
        return (W / s[:, None]).to(torch.float8_e4m3fn).view(torch.uint8), s

    def check_gemm(got, Aq, sa, Wq, sw, what, add=None, post=None, slab=2048):
        """got[m, :] against bf16( post( (Aq Wq^T)[m, :] * sa[m] * sw[:] ) + add[m, :] ), slab by slab."""
        wf = e4(Wq)
        for i in range(0, Aq.shape[0], slab):
            ref = (e4(Aq[i:i + slab]) @ wf.T) * sa[i:i + slab, None]
            if sw is not None:
                ref = ref * sw[None, :]
            if add is not None:
                ref = ref + add[i:i + slab].float()
            _close(got[i:i + slab], ref.bfloat16(), rel=1e-2)
        del wf

    A, dOut, res = _randn((T, d), 21), _randn((T, d), 22), _randn((T, d), 23)
    Wg, sg = weight(f, d, 24)
    Wu, su = weight(f, d, 25)
    Wd, sd = weight(d, f, 26)
    # ---- forward: saved pre-activations and the output with the residual added in the down projection's epilogue
    out, G, U = bf(T, d), bf(T, f), bf(T, f)
    ops.swiglu_ffn_fp8(T, d, f, A, Wg, sg, Wu, su, Wd, sd, out, G, U, residual=res)
    Aq, sa = u8(T, d), f32v(T)
    ops.quantize_rows_e4m3(T, d, A, Aq, sa)
    check_gemm(G, Aq, sa, Wg, sg, "gate")
    check_gemm(U, Aq, sa, Wu, su, "up")
    Hq, sh = u8(T, f), f32v(T)
    ops.swiglu_quantize_rows_e4m3(T, f, G, U, Hq, sh)
    check_gemm(out, Hq, sh, Wd, sd, "down + residual", add=res)
    del Aq, Hq
    # ---- input gradient
    WguT, WdT = u8(d, 2 * f), u8(f, d)
    ops.ffn_fp8_prepare_bwd_weights(d, f, Wg, Wu, Wd, WguT, WdT)
    dA, dGU = bf(T, d), bf(T, 2 * f)
    sgu = torch.cat([sg, su])
    ops.swiglu_ffn_fp8_bwd(T, d, f, dOut, G, U, WdT, sd, WguT, sgu, dA, dgate_dup=dGU)
    dOq, s1 = u8(T, d), f32v(T)
    ops.quantize_rows_e4m3(T, d, dOut, dOq, s1, col_factors=sd)
    wdt = e4(WdT)
    for i in range(0, T, 2048):                                 # dH = bf16(GEMM), then the SwiGLU backward formulas of swiglu_bwd_x
        dh = ((e4(dOq[i:i + 2048]) @ wdt.T) * s1[i:i + 2048, None]).bfloat16().float()
        gf, uf = G[i:i + 2048].float(), U[i:i + 2048].float()
        e = torch.exp(-gf)
        _close(dGU[i:i + 2048, :f], (dh * (uf * (1 + e + gf * e)) / ((1 + e) * (1 + e))).bfloat16(), rel=1e-2, flipped_frac=1e-4)
        _close(dGU[i:i + 2048, f:], (dh * (gf / (1 + e))).bfloat16(), rel=1e-2, flipped_frac=1e-4)
    del wdt, dOq
    dGUq, s2 = u8(T, 2 * f), f32v(T)
    ops.quantize_rows_e4m3(T, 2 * f, dGU, dGUq, s2, col_factors=sgu)
    check_gemm(dA, dGUq, s2, WguT, None, "input gradient")
    del dGUq, WguT, WdT
    # ---- weight gradients: operands are the transposes, quantised with one scale per row of the transpose
    dWg, dWu, dWd = bf(f, d), bf(f, d), bf(d, f)
    ops.swiglu_ffn_fp8_wgrad(T, d, f, A, dOut, G, U, dGU, dWg, dWu, dWd)
    H = bf(T, f)
    ops.swiglu(T, f, G, U, H)

    def transposed(X, cols):
        amax, Qt, sc = f32v(cols), u8(cols, T), f32v(cols)
        ops.col_amax_bf16(T, cols, X, amax)
        ops.transpose_quantize_e4m3(T, cols, X, amax, Qt, sc)
        return Qt, sc

    dOt, s_do = transposed(dOut, d)
    Ht, s_h = transposed(H, f)
    check_gemm(dWd, dOt, s_do, Ht, s_h, "dWdown")
    del dOt, Ht, H
    At, s_a = transposed(A, d)
    dGUt, s_gu = transposed(dGU, 2 * f)
    check_gemm(dWg, dGUt[:f], s_gu[:f], At, s_a, "dWgate")
    check_gemm(dWu, dGUt[f:], s_gu[f:], At, s_a, "dWup")
    torch.cuda.synchronize()
    words = (ctypes.c_uint * 8)()
    assert _lib.lib.dfb200_read_kernel_status(None, words, 8) == 0, [hex(w) for w in words]
