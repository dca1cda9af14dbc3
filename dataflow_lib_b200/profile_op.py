"""Runs ONE op a few times on synthetic data, for profilers (ncu) and quick timing:

    python -m dataflow_lib_b200.profile_op swiglu_bwd_x --tokens 2048 --iters 3
    ncu --set full --clock-control none -k regex:swiglu_bwd_x -c 3 -o prof python -m dataflow_lib_b200.profile_op swiglu_bwd_x --tokens 2048

Shapes are the Llama-3-8B layer's (d_model 4096, 32 q / 8 kv heads x 128, ffn 14336, vocab 128256); --tokens sets the rows.
Prints the event-timed mean of the launches after the first (the first one warms up)."""
import argparse

import torch

from . import ops

D, NH, NKV, HD, F, V = 4096, 32, 8, 128, 14336, 128256


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["rms_norm", "rms_norm_bwd_x", "rms_norm_bwd_w", "rms_norm_bwd_x_w", "rope", "rope_bwd_x", "swiglu", "swiglu_bwd_x",
                                   "softmax", "softmax_cross_entropy", "swiglu_ffn_fp8", "swiglu_ffn_fp8_bwd", "swiglu_ffn_fp8_wgrad", "gemm_e4m3_swiglu", "gemm_e4m3",
                                   "fp8_peak"])
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--vocab", type=int, default=V, help="softmax ops: columns per row (default: the Llama-3 vocabulary)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32", "fp8e4m3", "fp8e5m2"],
                    help="datatype of the forward tensors; with an fp8 type the gradients are bf16 (the registered fp8 x bf16 pairs)")
    a = ap.parse_args()
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "fp8e4m3": torch.float8_e4m3fn, "fp8e5m2": torch.float8_e5m2}[a.dtype]
    bdt = torch.bfloat16 if a.dtype.startswith("fp8") else dt        # datatype of gradients
    T = a.tokens
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g).to(dt)
    rnb = lambda *s: torch.randn(*s, device="cuda", generator=g).to(bdt)
    es, bes = torch.empty(0, dtype=dt).element_size(), torch.empty(0, dtype=bdt).element_size()
    if a.op == "fp8_peak":
        # the tensor-core ceiling for the FFN numbers: a library e4m3 GEMM (torch._scaled_mm -> cuBLASLt). Burst = best single launch
        # of 8192^3; sustained = the FFN's own shapes, 5 launches back to back (what profile_op reports for this library's kernels)
        one = torch.ones((), device="cuda")

        def lib_gemm(m, n, k):
            A8 = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
            B8 = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn).t()
            return lambda: torch._scaled_mm(A8, B8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        f8 = lib_gemm(8192, 8192, 8192)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); f8(); e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        print(f"fp8_peak burst: library e4m3 GEMM 8192^3 best of 10: {best * 1e3:.1f} us, {2 * 8192 ** 3 / (best * 1e-3) / 1e12:.0f} TFLOP/s")
        for name, (m, n, k) in {"gate or up projection": (T, F, D), "down projection": (T, D, F)}.items():
            fn = lib_gemm(m, n, k)
            fn(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.iters
            print(f"fp8_peak sustained: library e4m3 GEMM {m}x{n}x{k} ({name}), {a.iters} back to back: {ms * 1e3:.1f} us, {2 * m * n * k / (ms * 1e-3) / 1e12:.0f} TFLOP/s")
        return
    if a.op in ("swiglu_ffn_fp8", "swiglu_ffn_fp8_bwd", "swiglu_ffn_fp8_wgrad", "gemm_e4m3_swiglu", "gemm_e4m3"):
        def qw(n_out, n_in):
            W = 0.02 * torch.randn(n_out, n_in, device="cuda", generator=g)
            sc = W.abs().amax(1) / 448.0
            return (W / sc[:, None]).to(torch.float8_e4m3fn).view(torch.uint8), sc.float()
        A = rn(T, D)
        Wg, sg = qw(F, D)
        Wu, su = qw(F, D)
        Wd, sd = qw(D, F)
        out, H = torch.empty(T, D, device="cuda", dtype=torch.bfloat16), torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
        Aq, sa = torch.empty(T, D, device="cuda", dtype=torch.uint8), torch.empty(T, device="cuda")
        Hq, sh = torch.empty(T, F, device="cuda", dtype=torch.uint8), torch.empty(T, device="cuda")
        ops.quantize_rows_e4m3(T, D, A, Aq, sa)
        ops.gemm_e4m3_swiglu(T, F, D, Aq, sa, Wg, sg, Wu, su, H)
        ops.quantize_rows_e4m3(T, F, H, Hq, sh)
        G, U = torch.empty_like(H), torch.empty_like(H)
        WguT, WdT = torch.empty(D, 2 * F, device="cuda", dtype=torch.uint8), torch.empty(F, D, device="cuda", dtype=torch.uint8)
        ops.ffn_fp8_prepare_bwd_weights(D, F, Wg, Wu, Wd, WguT, WdT)
        ops.swiglu_ffn_fp8(T, D, F, A, Wg, sg, Wu, su, Wd, sd, out, G, U)
        dOut, dA, sgu = rn(T, D), torch.empty(T, D, device="cuda", dtype=torch.bfloat16), torch.cat([sg, su])
        dGU = torch.empty(T, 2 * F, device="cuda", dtype=torch.bfloat16)
        ops.swiglu_ffn_fp8_bwd(T, D, F, dOut, G, U, WdT, sd, WguT, sgu, dA, dgate_dup=dGU)
        dWg, dWu, dWd = (torch.empty(s_, device="cuda", dtype=torch.bfloat16) for s_ in ((F, D), (F, D), (D, F)))
        fn = {"swiglu_ffn_fp8": lambda: ops.swiglu_ffn_fp8(T, D, F, A, Wg, sg, Wu, su, Wd, sd, out, G, U),
              "swiglu_ffn_fp8_bwd": lambda: ops.swiglu_ffn_fp8_bwd(T, D, F, dOut, G, U, WdT, sd, WguT, sgu, dA),
              "swiglu_ffn_fp8_wgrad": lambda: ops.swiglu_ffn_fp8_wgrad(T, D, F, A, dOut, G, U, dGU, dWg, dWu, dWd),
              "gemm_e4m3_swiglu": lambda: ops.gemm_e4m3_swiglu(T, F, D, Aq, sa, Wg, sg, Wu, su, H),
              "gemm_e4m3": lambda: ops.gemm_e4m3(T, D, F, Hq, sh, Wd, sd, out)}[a.op]
        flops = {"swiglu_ffn_fp8": 6.0, "swiglu_ffn_fp8_bwd": 6.0, "swiglu_ffn_fp8_wgrad": 6.0, "gemm_e4m3_swiglu": 4.0, "gemm_e4m3": 2.0}[a.op] * T * D * F
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        print(f"{a.op} tokens={T} d={D} f={F}: {ms * 1e3:.1f} us/launch, {flops / (ms * 1e-3) / 1e12:.0f} TFLOP/s ({flops / 1e12:.2f} TFLOP)")
        return
    if a.op.startswith("rms_norm"):
        X, w, dY, dX = rn(T, D), (1 + 0.02 * torch.randn(D, device="cuda", generator=g)).to(dt), rnb(T, D), torch.zeros(T, D, device="cuda", dtype=bdt)
        Y, dW = torch.empty_like(X), torch.zeros(D, device="cuda", dtype=bdt)
        ws, rms = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
        ops.rms_norm(T, D, 1e-5, w, X, Y, ws, rms)
        fn = {"rms_norm": lambda: ops.rms_norm(T, D, 1e-5, w, X, Y, ws, rms),
              "rms_norm_bwd_x": lambda: ops.rms_norm_bwd_x(T, D, 1e-5, ws, rms, w, X, dY, dX),
              "rms_norm_bwd_w": lambda: ops.rms_norm_bwd_w(T, D, 1e-5, rms, X, dY, dW),
              "rms_norm_bwd_x_w": lambda: ops.rms_norm_bwd_x_w(T, D, 1e-5, ws, rms, w, X, dY, dX, dW)}[a.op]
        nbytes = T * D * {"rms_norm": 2 * es, "rms_norm_bwd_x": es + 3 * bes, "rms_norm_bwd_w": es + bes, "rms_norm_bwd_x_w": es + 3 * bes}[a.op]
    elif a.op.startswith("rope"):
        rdt = dt if a.op == "rope" else bdt                      # the backward op works on gradients
        Q, K = (torch.randn(T, n * HD, device="cuda", generator=g).to(rdt) for n in (NH, NKV))
        pos = torch.arange(T, device="cuda", dtype=torch.int32)
        f = ops.rope if a.op == "rope" else ops.rope_bwd_x
        fn = lambda: f(T * NH * HD, NH * HD, HD, NKV, 500000, pos, Q, K)
        nbytes = 2 * T * (NH + NKV) * HD * Q.element_size()
    elif a.op.startswith("swiglu"):
        x1, x3, dY = rn(T, F), rn(T, F), rnb(T, F)
        out, d1, d3 = torch.empty_like(x1), torch.empty_like(dY), torch.empty_like(dY)
        fn = (lambda: ops.swiglu(T, F, x1, x3, out)) if a.op == "swiglu" else (lambda: ops.swiglu_bwd_x(T, F, x1, x3, dY, d1, d3))
        nbytes = T * F * (3 * es if a.op == "swiglu" else 2 * es + 3 * bes)
    else:
        vocab = a.vocab
        L = (2 * torch.randn(T, vocab, device="cuda", generator=g)).to(dt)
        out = torch.empty(T, vocab, device="cuda", dtype=bdt)
        labels = torch.randint(0, vocab, (T,), device="cuda", generator=g, dtype=torch.int32)
        loss = torch.zeros(2, device="cuda")
        fn = (lambda: ops.softmax(T, vocab, L, out)) if a.op == "softmax" else (lambda: ops.softmax_cross_entropy(T, vocab, L, labels, out, None, loss))
        nbytes = T * vocab * (es + bes)
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    print(f"{a.op} {a.dtype} tokens={T}: {ms * 1e3:.1f} us/launch back to back, {nbytes / (ms * 1e-3) / 1e9:.0f} GB/s algorithmic ({nbytes / 2**20:.0f} MiB)")


if __name__ == "__main__":
    main()
