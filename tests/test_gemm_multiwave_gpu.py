"""The persistent FP8 GEMM where every walker takes several tiles: accumulator-stage parity, the hand-back of an
accumulator from the epilogue to the MMA warp, the load ring running on across tiles, the 16-row-group raster and
ragged last tiles in both directions. Each epilogue mode, in the CTA-pair form and in the one-CTA-per-tile form.

Checker: fp32 matmul on the GPU (torch, TF32 off) of the e4m3 codes, times the scales -- the same arithmetic contract as
the CPU oracle's oracle_gemm_e4m3 (products of e4m3 values are exact in fp32, accumulation in fp32), which is too slow
at these sizes and stays the checker for the small shapes of test_ffn_fp8_gpu.py.
Tolerance: bf16 outputs within 1e-2 of max(|ref|, rms(ref))."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

E4M3_MAX = 448.0


@pytest.fixture(scope="module")
def ops():
    from dataflow_lib_b200 import ops as _ops
    torch.backends.cuda.matmul.allow_tf32 = False
    return _ops


@pytest.fixture(params=["cta_pair", "single_cta"])
def form(request):
    old = os.environ.get("DFB200_GEMM_SINGLE_CTA")
    if request.param == "single_cta":
        os.environ["DFB200_GEMM_SINGLE_CTA"] = "1"
    else:
        os.environ.pop("DFB200_GEMM_SINGLE_CTA", None)
    yield request.param
    if old is None:
        os.environ.pop("DFB200_GEMM_SINGLE_CTA", None)
    else:
        os.environ["DFB200_GEMM_SINGLE_CTA"] = old


def _codes(rows, cols, seed, std=1.0):
    """Random e4m3 codes (as uint8) with one fp32 scale per row, the way the row quantiser makes them."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = std * torch.randn(rows, cols, device="cuda", generator=g)
    amax = x.abs().amax(1).clamp_min(1e-30)
    q = (x * (E4M3_MAX / amax)[:, None]).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), (amax / E4M3_MAX).float()


def _bf16(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(rows, cols, device="cuda", generator=g).bfloat16()


def _acc(Aq, Wq):
    return Aq.view(torch.float8_e4m3fn).float() @ Wq.view(torch.float8_e4m3fn).float().T


def _close(got, ref, what, rel=1e-2):
    got, ref = got.float(), ref.float()
    assert torch.isfinite(got).all(), f"{what}: non-finite output (an unwritten tile?)"
    s = ref.pow(2).mean().sqrt()
    tol = rel * torch.maximum(ref.abs(), s)
    bad = (got - ref).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} outside {rel} rel, first at {bad.nonzero()[0].tolist()}"


def _status_clean():
    import ctypes
    from dataflow_lib_b200 import _lib
    words = (ctypes.c_uint * 8)()
    assert _lib.lib.dfb200_read_kernel_status(None, words, 8) == 0, [hex(w) for w in words]


# (M, N, K): 17 x 17 pair tiles = 289 on <= 74 pairs (4 per walker), 33 x 17 = 561 one-CTA tiles on 148 CTAs; ragged in M and N;
# the second shape has more row tiles than one raster group (16) in both forms and a k-loop shorter than the ring.
PLAIN_SHAPES = [(4096 + 40, 4096 + 24, 512), (8192 + 136, 1024 + 8, 256), (2048, 8192, 1024 + 16)]


@pytest.mark.parametrize("mnk", PLAIN_SHAPES, ids=str)
@pytest.mark.parametrize("residual", [False, True], ids=["plain", "residual"])
def test_plain_many_tiles_per_walker(ops, form, mnk, residual):
    M, N, K = mnk
    Aq, sa = _codes(M, K, 1)
    Wq, sw = _codes(N, K, 2, 0.02)
    ref = (_acc(Aq, Wq) * sa[:, None]) * sw[None, :]
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    if residual:
        res = _bf16(M, N, 3)
        out.copy_(res)                                        # in place on the residual buffer, as the FFN's down projection does
        ops.gemm_e4m3(M, N, K, Aq, sa, Wq, sw, out, residual=out)
        ref = ref + res.float()
    else:
        ops.gemm_e4m3(M, N, K, Aq, sa, Wq, sw, out)
    torch.cuda.synchronize()
    _close(out, ref.bfloat16(), f"gemm_e4m3 {form} {mnk} residual={residual}")
    _status_clean()


@pytest.mark.parametrize("mnk", [(4096 + 40, 2048 + 24, 512), (8192 + 136, 1024 + 8, 256)], ids=str)
@pytest.mark.parametrize("save", [False, True], ids=["h_only", "save_g_u"])
def test_swiglu_many_tiles_per_walker(ops, form, mnk, save):
    M, N, K = mnk
    Aq, sa = _codes(M, K, 4)
    Wg, sg = _codes(N, K, 5, 0.05)
    Wu, su = _codes(N, K, 6, 0.05)
    g = (_acc(Aq, Wg) * sa[:, None]) * sg[None, :]
    u = (_acc(Aq, Wu) * sa[:, None]) * su[None, :]
    ref = (g / (1 + torch.exp(-g))) * u
    nan = lambda: torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    H, G, U = nan(), nan() if save else None, nan() if save else None
    ops.gemm_e4m3_swiglu(M, N, K, Aq, sa, Wg, sg, Wu, su, H, G, U)
    torch.cuda.synchronize()
    _close(H, ref.bfloat16(), f"gemm_e4m3_swiglu {form} {mnk}")
    if save:
        _close(G, g.bfloat16(), f"saved gate {form} {mnk}")
        _close(U, u.bfloat16(), f"saved up {form} {mnk}")
    _status_clean()


@pytest.mark.parametrize("mnk", [(4096 + 40, 2048 + 24, 512), (8192 + 136, 1024 + 8, 256)], ids=str)
def test_swiglu_bwd_many_tiles_per_walker(ops, form, mnk):
    M, N, K = mnk                                             # N = hidden width f, K = model width d
    dOq, s1 = _codes(M, K, 7)
    WdT, _ = _codes(N, K, 8, 0.02)
    g, u = _bf16(M, N, 9), _bf16(M, N, 10)
    dh = _acc(dOq, WdT) * s1[:, None]
    gf, uf = g.float(), u.float()
    e = torch.exp(-gf)
    dgate = dh * ((uf * (1 + e + gf * e)) / ((1 + e) * (1 + e)))
    dup = dh * (gf / (1 + e))
    out = torch.full((M, 2 * N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_e4m3_swiglu_bwd(M, N, K, dOq, s1, WdT, g, u, out)
    torch.cuda.synchronize()
    _close(out[:, :N], dgate.bfloat16(), f"gate gradient {form} {mnk}")
    _close(out[:, N:], dup.bfloat16(), f"up gradient {form} {mnk}")
    _status_clean()


def test_both_forms_agree(ops):
    """The CTA-pair form and the one-CTA form accumulate the same fp32 products in the same k order: the outputs agree to the bit
    (asserted for 99.9 % of the elements, the rest within one bf16 unit, in case the two instruction shapes sum a k-block differently)."""
    M, N, K = 2048 + 40, 2048 + 24, 768
    Aq, sa = _codes(M, K, 11)
    Wq, sw = _codes(N, K, 12, 0.02)
    outs = []
    old = os.environ.get("DFB200_GEMM_SINGLE_CTA")
    try:
        for single in ("0", "1"):
            os.environ["DFB200_GEMM_SINGLE_CTA"] = single
            out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
            ops.gemm_e4m3(M, N, K, Aq, sa, Wq, sw, out)
            torch.cuda.synchronize()
            outs.append(out)
    finally:
        if old is None:
            os.environ.pop("DFB200_GEMM_SINGLE_CTA", None)
        else:
            os.environ["DFB200_GEMM_SINGLE_CTA"] = old
    assert (outs[0] == outs[1]).float().mean().item() > 0.999
    _close(outs[0], outs[1], "pair form against one-CTA form", rel=2.0 ** -7)
