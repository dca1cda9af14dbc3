"""Times the REFERENCE's own kernels (oracle/_ref/cuda_kernels.cubin: its cuda_kernels.cu compiled unchanged for sm_100a with
its own flags) beside this library's on the same B200, same shapes, same inputs: the 8192-token layer chain and a 4096-row
slice of the 128256-column softmax. Checker-side tooling (it launches the reference's kernels): it lives with the oracle and is
what profiles/reference_kernels_vs_library_bf16_8192tok.md was made with; run as

    python oracle/time_reference_kernels.py [--iters 20]

Each op is launched `iters` times back to back between two CUDA events after one warm-up launch (inputs are far larger than
L2). cross_entropy_loss is left out: the reference kernel only touches row 0. Prints a markdown table."""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))            # ref_kernels.py: the launcher of the reference cubin that the tests use

from dataflow_lib_b200 import ops          # noqa: E402
from ref_kernels import RefKernels, available   # noqa: E402

T, D, NH, NKV, HD, F, V, THETA, EPS = 8192, 4096, 32, 8, 128, 14336, 128256, 500000, 1e-5


def timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3      # microseconds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    assert available(), "needs oracle/_ref/cuda_kernels.cubin (make -C oracle ref) and a GPU"
    R = RefKernels()
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g).bfloat16()
    X, dY, dX, Y = rn(T, D), rn(T, D), torch.zeros(T, D, device="cuda", dtype=torch.bfloat16), torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.02 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    dW = torch.zeros(D, device="cuda", dtype=torch.bfloat16)
    ws, rms = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    Q, K, pos = rn(T, NH * HD), rn(T, NKV * HD), torch.arange(T, device="cuda", dtype=torch.int32)
    x1, x3, dS = rn(T, F), rn(T, F), rn(T, F)
    S, d1, d3 = torch.empty_like(x1), torch.empty_like(x1), torch.empty_like(x1)
    rows_sm = 4096
    logits, probs = (2 * torch.randn(rows_sm, V, device="cuda", generator=g)).bfloat16(), torch.empty(rows_sm, V, device="cuda", dtype=torch.bfloat16)
    ops.rms_norm(T, D, EPS, w, X, Y, ws, rms)
    N = T * NH * HD
    e = 2
    cases = [
        ("rms_norm", 2 * T * D * e, lambda: R.rms_norm("bf16", 2, T, D, EPS, w, X, Y, ws, rms), lambda: ops.rms_norm(T, D, EPS, w, X, Y, ws, rms)),
        ("rope", 2 * T * (NH + NKV) * HD * e, lambda: R.rope("bf16", N, NH * HD, HD, NKV, THETA, pos, Q, K), lambda: ops.rope(N, NH * HD, HD, NKV, THETA, pos, Q, K)),
        ("swiglu", 3 * T * F * e, lambda: R.swiglu("bf16", T, F, x1, x3, S), lambda: ops.swiglu(T, F, x1, x3, S)),
        ("swiglu_bwd_x", 5 * T * F * e, lambda: R.swiglu_bwd_x("bf16_bf16", T, F, x1, x3, dS, d1, d3), lambda: ops.swiglu_bwd_x(T, F, x1, x3, dS, d1, d3)),
        ("rope_bwd_x", 2 * T * (NH + NKV) * HD * e, lambda: R.rope("bf16", N, NH * HD, HD, NKV, THETA, pos, Q, K, bwd=True),
         lambda: ops.rope_bwd_x(N, NH * HD, HD, NKV, THETA, pos, Q, K)),
        ("rms_norm_bwd_x", 4 * T * D * e, lambda: R.rms_norm_bwd_x("bf16_bf16", T, D, EPS, ws, rms, w, X, dY, dX),
         lambda: ops.rms_norm_bwd_x(T, D, EPS, ws, rms, w, X, dY, dX)),
        ("rms_norm_bwd_w", 2 * T * D * e, lambda: R.rms_norm_bwd_w("bf16_bf16", T, D, EPS, rms, X, dY, dW), lambda: ops.rms_norm_bwd_w(T, D, EPS, rms, X, dY, dW)),
        (f"softmax {rows_sm}x{V}", 2 * rows_sm * V * e, lambda: R.softmax("bf16_bf16", rows_sm, V, logits, probs), lambda: ops.softmax(rows_sm, V, logits, probs)),
    ]
    print("| op (bf16) | reference kernel on B200, us | this library, us | speed-up | this library GB/s (algorithmic) |")
    print("|---|---|---|---|---|")
    tot_ref = tot_own = 0.0
    for name, nbytes, ref_fn, own_fn in cases:
        t_ref, t_own = timed(ref_fn, a.iters), timed(own_fn, a.iters)
        if not name.startswith("softmax"):
            tot_ref, tot_own = tot_ref + t_ref, tot_own + t_own
        print(f"| {name} | {t_ref:.1f} | {t_own:.1f} | {t_ref / t_own:.1f}x | {nbytes / t_own / 1e3:.0f} |")
    print(f"| chain of the 7 ops, 8192 tokens | {tot_ref:.1f} | {tot_own:.1f} | {tot_ref / tot_own:.1f}x | |")
    print(f"| tokens/s, chain | {T / tot_ref * 1e6:.3g} | {T / tot_own * 1e6:.3g} | | |")


if __name__ == "__main__":
    main()
