"""The block callers (include/dataflow_transformer.h: submit_transformer_block, _bwd_x, _bwd_w) on the GPU: every native op of a
block runs from this library, the seven projections and their gradients through the reference's cuBLASLt plug-in
(oracle/_ref/libref_matmul_helper.so, built unchanged), attention through a stand-in plug-in written for this test
(tests/c_caller/attention_standin.c: copies only, so that the wiring of every attention buffer shows in the results).
Each buffer the chains leave behind is checked against the oracle composed step by step from the device's own inputs to that step
where those survive (bf16 tolerance: 1e-2 of max(|ref|, rms))."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle as O
from util import check_f32, check_lowp, f32, to_dev, to_host

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MATMUL = os.path.join(ROOT, "oracle", "_ref", "libref_matmul_helper.so")


@pytest.fixture(scope="module")
def standin(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("standin") / "libattention_standin.so")
    cmd = ["gcc", "-O1", "-std=gnu11", "-Wall", "-Wextra", "-Werror", "-Wno-unused-parameter", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "c_caller", "attention_standin.c"), "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def _mm(a_bits, b_bits, c_bits=None, transpose_b=True):
    """bf16( a . b^T + c ) with exact products and one rounding, as a GEMM with fp32 accumulation gives it up to summation order."""
    a, b = f32(a_bits, O.BF16).astype(np.float64), f32(b_bits, O.BF16).astype(np.float64)
    acc = a @ (b.T if transpose_b else b)
    if c_bits is not None:
        acc = acc + f32(c_bits, O.BF16)
    return O.from_f32(acc.astype(np.float32), O.BF16)


@pytest.mark.skipif(not os.path.exists(MATMUL), reason="reference matmul plug-in not built (make -C oracle ref)")
def test_block_forward_and_backward_chains(standin):
    from dataflow_lib_b200 import DataflowHandle, _lib, abi
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    L = _lib.lib
    h = DataflowHandle(device_id=0, num_streams=2)
    sks = [abi.OpSkeleton() for _ in range(3)]
    L.set_external_matmul_skeleton(C.byref(sks[0]))
    L.set_external_flash3_attention_fwd_skeleton(C.byref(sks[1]))
    L.set_external_flash3_attention_bwd_skeleton(C.byref(sks[2]))
    assert h.register_external_code(MATMUL, [sks[0]], ["cublas_matmul"], ["cublas_matmul_init"]) == 1
    assert h.register_external_code(standin, sks[1:], ["standin_attention_fwd", "standin_attention_bwd"], [None, None]) == 2

    T, nq, nkv, hd, f, eps, theta = 256, 4, 2, 64, 512, 1e-5, 10000
    d, kv = nq * hd, nkv * hd
    BF, FP32 = int(DT.BF16), int(DT.FP32)
    bf = torch.bfloat16
    fill = lambda shape, seed, std=1.0, mean=0.0: O.fill_normal(O.BF16, shape, seed, mean, std)
    host = {"X": fill((T, d), 1), "w_an": fill((d,), 2, 0.05, 1.0), "w_fn": fill((d,), 3, 0.05, 1.0),
            "Wq": fill((d, d), 4, 0.06), "Wk": fill((kv, d), 5, 0.06), "Wv": fill((kv, d), 6, 0.06), "Wo": fill((d, d), 7, 0.06),
            "W1": fill((f, d), 8, 0.06), "W2": fill((d, f), 9, 0.04), "W3": fill((f, d), 10, 0.06), "dOut": fill((T, d), 11)}
    dev = {k: to_dev(v, O.BF16) for k, v in host.items()}
    pos = np.arange(T, dtype=np.int32)
    pos_d = torch.from_numpy(pos).cuda()
    z = lambda *s: torch.zeros(s, dtype=bf, device="cuda")
    zf = lambda n: torch.zeros(n, device="cuda")
    keep = []

    def one(t):
        keep.append((C.c_void_p * 1)(t.data_ptr()))
        return C.cast(keep[-1], C.POINTER(C.c_void_p))

    def containers(weights):
        """(block, activations, tensors): fresh activation buffers; `weights` maps member -> tensor."""
        blk = abi.TransformerBlock()
        c = blk.config
        c.block_dt, c.compute_dt, c.eps, c.theta = BF, FP32, eps, theta
        c.num_q_heads, c.num_kv_heads, c.head_dim, c.model_dim, c.kv_dim, c.ffn_dim = nq, nkv, hd, d, kv, f
        blk.w_attn_norm, blk.w_ffn_norm = weights["w_an"].data_ptr(), weights["w_fn"].data_ptr()
        blk.w_q, blk.w_k, blk.w_v, blk.w_o = (weights[k].data_ptr() for k in ("Wq", "Wk", "Wv", "Wo"))
        blk.w_1, blk.w_2, blk.w_3 = one(weights["W1"]), one(weights["W2"]), one(weights["W3"])
        t = {"sums_a": zf(T), "rms_a": zf(T), "x_q": z(T, d), "x_k": z(T, kv), "x_v": z(T, kv), "lse": zf(T * nq), "attn_out": z(T, d), "x_o": z(T, d),
             "sums_f": zf(T), "rms_f": zf(T), "x_1": z(T, f), "x_2": z(T, d), "x_3": z(T, f), "x_temp": z(T, d), "x_mlp": z(T, f),
             "re_attn": z(T, d), "re_ffn": z(T, d), "work": torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")}
        bc = abi.SeqBatchConfig(1, T, T, pos_d.data_ptr(), None, None, T, None, None, T)
        sv = abi.SeqBatchSavedActivations()
        sv.attn_norm_weighted_sums, sv.attn_norm_rms_vals, sv.x_q, sv.x_k_local, sv.x_v_local = (t[k].data_ptr() for k in ("sums_a", "rms_a", "x_q", "x_k", "x_v"))
        sv.softmax_lse, sv.x_attn_out, sv.x_o, sv.ffn_norm_weighted_sums, sv.ffn_norm_rms_vals = (t[k].data_ptr() for k in ("lse", "attn_out", "x_o", "sums_f", "rms_f"))
        sv.x_1, sv.x_2, sv.x_3 = one(t["x_1"]), one(t["x_2"]), one(t["x_3"])
        ctx = abi.SeqBatchContext(None, None, 0, t["x_k"].data_ptr(), t["x_v"].data_ptr())      # one sequence, no cache: the attention reads the local K, V
        ws = abi.SeqBatchActivationWorkspace(None, None, 0, t["x_temp"].data_ptr(), t["x_mlp"].data_ptr(), t["re_attn"].data_ptr(),
                                             t["re_ffn"].data_ptr(), t["work"].data_ptr(), t["work"].numel())
        act = abi.TransformerBlockActivations(C.pointer(blk), C.pointer(bc), C.pointer(sv), C.pointer(ctx), C.pointer(ws))
        keep.extend([blk, bc, sv, ctx, ws, act])
        return blk, act, t

    blk, act, a = containers(dev)
    out_copy = z(T, d)
    xin, xout = abi.TransformerBlockTransition(None, dev["X"].data_ptr()), abi.TransformerBlockTransition(None, out_copy.data_ptr())
    r, hp = C.byref, C.byref(h.h)
    B = lambda t: to_host(t, O.BF16)

    # ---------------- forward
    assert L.submit_transformer_block(hp, 0, 1, r(xin), r(blk), r(act), r(xout)) == 0
    assert h.sync_stream(0) == 0 and h.sync_stream(1) == 0
    hn, ws_a, rms_a = O.rms_norm(O.BF16, eps, host["w_an"], host["X"])
    check_f32(a["rms_a"].cpu().numpy(), rms_a, "attention norm rms")
    check_f32(a["sums_a"].cpu().numpy(), ws_a, "attention norm weighted sums", scale=1.0)
    q_ref, k_ref = O.rope(O.BF16, d, hd, nkv, theta, pos, _mm(hn, host["Wq"]), _mm(hn, host["Wk"]))
    check_lowp(B(a["x_q"]), q_ref, O.BF16, "x_q after RoPE")
    check_lowp(B(a["x_k"]), k_ref, O.BF16, "x_k_local after RoPE")
    check_lowp(B(a["x_v"]), _mm(hn, host["Wv"]), O.BF16, "x_v_local")
    assert torch.equal(a["attn_out"], a["x_q"]), "the stand-in attention copies x_q"
    check_lowp(B(a["x_o"]), _mm(B(a["attn_out"]), host["Wo"], host["X"]), O.BF16, "x_o = attention projection + input")
    fn, ws_f, rms_f = O.rms_norm(O.BF16, eps, host["w_fn"], B(a["x_o"]))
    check_lowp(B(a["x_temp"]), fn, O.BF16, "FFN norm output")
    check_f32(a["rms_f"].cpu().numpy(), rms_f, "FFN norm rms")
    check_lowp(B(a["x_1"]), _mm(B(a["x_temp"]), host["W1"]), O.BF16, "x_1")
    check_lowp(B(a["x_3"]), _mm(B(a["x_temp"]), host["W3"]), O.BF16, "x_3")
    check_lowp(B(a["x_mlp"]), O.swiglu(O.BF16, B(a["x_1"]), B(a["x_3"])), O.BF16, "swiglu")
    check_lowp(B(a["x_2"]), _mm(B(a["x_mlp"]), host["W2"], B(a["x_o"])), O.BF16, "x_2 = down projection + x_o")
    assert torch.equal(out_copy, a["x_2"]), "the copy on the second stream must see the finished output"

    # ---------------- input gradients
    g0 = {k: fill(host[k].shape, 20 + i, 0.01) for i, k in enumerate(("w_an", "w_fn", "Wq", "Wk", "Wv", "Wo", "W1", "W2", "W3"))}    # gradients accumulate
    gdev = {k: to_dev(v, O.BF16) for k, v in g0.items()}
    gblk, _, _ = containers(gdev)
    _, gact, g = containers(dev)
    dX = dev["dOut"].clone()
    dnext = z(T, d)
    dstream, dnext_t = abi.TransformerBlockTransition(None, dX.data_ptr()), abi.TransformerBlockTransition(None, dnext.data_ptr())
    assert L.submit_transformer_block_bwd_x(hp, 0, 1, r(blk), r(dstream), r(act), r(xin), r(gact), r(gblk), r(dnext_t)) == 0
    assert h.sync_stream(0) == 0 and h.sync_stream(1) == 0
    check_lowp(B(g["x_mlp"]), _mm(host["dOut"], host["W2"], transpose_b=False), O.BF16, "d(swiglu output)")
    d1, d3 = O.swiglu_bwd_x(O.BF16, O.BF16, B(a["x_1"]), B(a["x_3"]), B(g["x_mlp"]))
    check_lowp(B(g["x_1"]), d1, O.BF16, "d(x_1)")
    check_lowp(B(g["x_3"]), d3, O.BF16, "d(x_3)")
    t = _mm(B(g["x_3"]), host["W3"], _mm(B(g["x_1"]), host["W1"], transpose_b=False), transpose_b=False)     # d(FFN norm output)
    dxo_ref = O.rms_norm_bwd_x(O.BF16, O.BF16, a["sums_f"].cpu().numpy(), a["rms_f"].cpu().numpy(), host["w_fn"], B(a["x_o"]), t, host["dOut"])
    # `t` is made here, not read from the device (x_temp is reused later in the chain): where the two GEMMs round an element of it to
    # different bf16 neighbours the product dY * deriv moves by that unit on top of its own rounding, hence 2e-2 for this op's output
    check_lowp(B(g["x_o"]), dxo_ref, O.BF16, "d(x_o) = output gradient + FFN norm path", rel=2e-2)
    check_lowp(B(gdev["w_fn"]), O.rms_norm_bwd_w(O.BF16, O.BF16, a["rms_f"].cpu().numpy(), B(a["x_o"]), t, g0["w_fn"]), O.BF16, "dW_ffn_norm", rel=2e-2)
    u = _mm(B(g["x_o"]), host["Wo"], transpose_b=False)                                   # d(x_attn_out); the stand-in hands it on as d(x_q)
    dq_ref, dk_ref = O.rope(O.BF16, d, hd, nkv, theta, pos, u, B(a["x_k"]), bwd=True)     # ... and x_k as d(x_k), both then rotated back
    check_lowp(B(g["x_q"]), dq_ref, O.BF16, "d(x_q) after the RoPE gradient")
    check_lowp(B(g["x_k"]), dk_ref, O.BF16, "d(x_k_local) after the RoPE gradient")
    assert torch.equal(g["x_v"], a["x_v"]), "the stand-in attention gradient copies x_v into d(x_v)"
    t2 = _mm(B(g["x_q"]), host["Wq"], transpose_b=False)
    t2 = _mm(B(g["x_k"]), host["Wk"], t2, transpose_b=False)
    t2 = _mm(B(g["x_v"]), host["Wv"], t2, transpose_b=False)                               # d(attention norm output)
    dx_ref = O.rms_norm_bwd_x(O.BF16, O.BF16, a["sums_a"].cpu().numpy(), a["rms_a"].cpu().numpy(), host["w_an"], host["X"], t2, B(g["x_o"]))
    check_lowp(B(dX), dx_ref, O.BF16, "gradient with respect to the block input", rel=2e-2)        # t2 is made here too
    check_lowp(B(gdev["w_an"]), O.rms_norm_bwd_w(O.BF16, O.BF16, a["rms_a"].cpu().numpy(), host["X"], t2, g0["w_an"]), O.BF16, "dW_attn_norm", rel=2e-2)
    check_lowp(B(g["re_attn"]), hn, O.BF16, "recomputed attention norm")
    check_lowp(B(g["re_ffn"]), fn, O.BF16, "recomputed FFN norm")
    assert torch.equal(dnext, dX), "the copy on the second stream must see the finished gradient"

    # ---------------- weight gradients (accumulated into the non-zero buffers)
    dout_t = abi.TransformerBlockTransition(None, dev["dOut"].data_ptr())
    assert L.submit_transformer_block_bwd_w(hp, 0, r(dout_t), r(act), r(gact), r(gblk)) == 0
    assert h.sync_stream(0) == 0
    check_lowp(B(g["x_mlp"]), O.swiglu(O.BF16, B(a["x_1"]), B(a["x_3"])), O.BF16, "recomputed swiglu")
    wgrad = lambda dy, x, w0: _mm(np.ascontiguousarray(dy.T), np.ascontiguousarray(x.T), w0)        # dW[out, in] = dy^T x + dW_0
    check_lowp(B(gdev["W2"]), wgrad(host["dOut"], B(g["x_mlp"]), g0["W2"]), O.BF16, "dW_2")
    check_lowp(B(gdev["W1"]), wgrad(B(g["x_1"]), B(g["re_ffn"]), g0["W1"]), O.BF16, "dW_1")
    check_lowp(B(gdev["W3"]), wgrad(B(g["x_3"]), B(g["re_ffn"]), g0["W3"]), O.BF16, "dW_3")
    check_lowp(B(gdev["Wo"]), wgrad(B(g["x_o"]), B(a["attn_out"]), g0["Wo"]), O.BF16, "dW_o")
    check_lowp(B(gdev["Wv"]), wgrad(B(g["x_v"]), B(g["re_attn"]), g0["Wv"]), O.BF16, "dW_v")
    check_lowp(B(gdev["Wk"]), wgrad(B(g["x_k"]), B(g["re_attn"]), g0["Wk"]), O.BF16, "dW_k")
    check_lowp(B(gdev["Wq"]), wgrad(B(g["x_q"]), B(g["re_attn"]), g0["Wq"]), O.BF16, "dW_q")
    h.close()
