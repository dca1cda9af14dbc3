"""The small seeded cases behind tests/golden/reference_vectors.npz (outputs of the reference's own kernels).
Shared by the generator (tests/golden/make_reference_vectors.py, GPU) and the checker (tests/test_oracle_cpu.py)."""
import numpy as np

import oracle as O

BF, FH, F32, E4, E5 = O.BF16, O.FP16, O.FP32, O.E4M3, O.E5M2


def _rms(dt, R, C, tag):
    return {"op": "rms_norm", "fdt": dt, "shape": (R, C), "dts": {"X": dt, "w": dt}, "tag": tag}


CASES = {}
for _dt, _n in ((BF, "bf16"), (FH, "fp16"), (F32, "fp32")):
    CASES[f"rms_norm_{_n}"] = {"op": "rms_norm", "fdt": _dt, "shape": (12, 1024), "dts": {"X": _dt, "w": _dt}}
    CASES[f"rms_norm_bwd_x_{_n}"] = {"op": "rms_norm_bwd_x", "fdt": _dt, "bdt": _dt, "shape": (12, 1024), "dts": {"X": _dt, "w": _dt, "dY": _dt, "dX": _dt}}
    CASES[f"rms_norm_bwd_w_{_n}"] = {"op": "rms_norm_bwd_w", "fdt": _dt, "bdt": _dt, "shape": (40, 512), "dts": {"X": _dt, "dY": _dt, "dW": _dt}}
    CASES[f"rope_{_n}"] = {"op": "rope", "fdt": _dt, "tokens": 16, "model_dim": 512, "head_dim": 128, "n_kv": 2, "theta": 500000, "max_pos": 512,
                           "dts": {"Q": _dt, "K": _dt}}
    CASES[f"rope_bwd_x_{_n}"] = {"op": "rope_bwd_x", "fdt": _dt, "tokens": 16, "model_dim": 512, "head_dim": 128, "n_kv": 2, "theta": 500000,
                                 "max_pos": 512, "dts": {"Q": _dt, "K": _dt}}
    CASES[f"swiglu_{_n}"] = {"op": "swiglu", "fdt": _dt, "shape": (6, 1024), "dts": {"x1": _dt, "x3": _dt}}
    CASES[f"swiglu_bwd_x_{_n}"] = {"op": "swiglu_bwd_x", "fdt": _dt, "bdt": _dt, "shape": (6, 1024), "dts": {"x1": _dt, "x3": _dt, "dY": _dt}}
    CASES[f"softmax_{_n}"] = {"op": "softmax", "fdt": _dt, "bdt": _dt, "shape": (4, 4096), "dts": {"X": _dt}}
CASES["rope_bf16_long"] = {"op": "rope", "fdt": BF, "tokens": 16, "model_dim": 512, "head_dim": 128, "n_kv": 2, "theta": 500000, "max_pos": 8192,
                           "dts": {"Q": BF, "K": BF}}
CASES["softmax_bf16_vocab"] = {"op": "softmax", "fdt": BF, "bdt": BF, "shape": (2, 128256), "dts": {"X": BF}}
CASES["softmax_fp8e4m3_bf16"] = {"op": "softmax", "fdt": E4, "bdt": BF, "shape": (4, 4096), "dts": {"X": E4}}
CASES["swiglu_fp8e4m3"] = {"op": "swiglu", "fdt": E4, "shape": (6, 1024), "dts": {"x1": E4, "x3": E4}}
for _dt, _n in ((F32, "fp32"), (BF, "bf16")):
    CASES[f"select_experts_{_n}"] = {"op": "select_experts", "fdt": _dt, "tokens": 192, "n_experts": 64, "top_k": 8, "dts": {"X": _dt}}
for _dt, _n in ((BF, "bf16"), (FH, "fp16")):
    CASES[f"softmax_{_n}_fp32_argmax"] = {"op": "softmax_fp32_out", "fdt": _dt, "bdt": F32, "shape": (4, 4096), "dts": {"X": _dt}}
CASES["swiglu_bwd_x_fp8e5m2_fp16"] = {"op": "swiglu_bwd_x", "fdt": E5, "bdt": FH, "shape": (6, 1024), "dts": {"x1": E5, "x3": E5, "dY": FH}}


def inputs_for(case):
    """numpy raw-bit inputs of a case (deterministic in the case description)."""
    op, fdt, bdt = case["op"], case["fdt"], case.get("bdt", case["fdt"])
    if op == "rms_norm":
        R, C = case["shape"]
        return {"X": O.fill_normal(fdt, (R, C), 101), "w": O.fill_normal(fdt, (C,), 102, 1.0, 0.02)}
    if op == "rms_norm_bwd_x":
        R, C = case["shape"]
        X, w = O.fill_normal(fdt, (R, C), 101), O.fill_normal(fdt, (C,), 102, 1.0, 0.02)
        _, ws, rms = O.rms_norm(fdt, 1e-5, w, X)
        return {"X": X, "w": w, "dY": O.fill_normal(bdt, (R, C), 103), "dX": O.fill_normal(bdt, (R, C), 104), "ws": ws, "rms": rms}
    if op == "rms_norm_bwd_w":
        R, C = case["shape"]
        X = O.fill_normal(fdt, (R, C), 101)
        rms = (1.0 / np.sqrt((O.to_f32(X, fdt).astype(np.float64) ** 2).mean(1) + 1e-5)).astype(np.float32)
        return {"X": X, "dY": O.fill_normal(bdt, (R, C), 103), "dW": np.zeros(C, O.NP_OF[bdt]), "rms": rms}
    if op in ("rope", "rope_bwd_x"):
        T, md, hd, nkv = case["tokens"], case["model_dim"], case["head_dim"], case["n_kv"]
        pos = (np.arange(T, dtype=np.int64) * 2654435761 % case["max_pos"]).astype(np.int32)
        return {"Q": O.fill_normal(fdt, (T, md), 105), "K": O.fill_normal(fdt, (T, nkv * hd), 106), "pos": pos}
    if op == "swiglu":
        return {"x1": O.fill_normal(fdt, case["shape"], 107), "x3": O.fill_normal(fdt, case["shape"], 108)}
    if op == "swiglu_bwd_x":
        return {"x1": O.fill_normal(fdt, case["shape"], 107), "x3": O.fill_normal(fdt, case["shape"], 108), "dY": O.fill_normal(bdt, case["shape"], 109)}
    if op == "softmax":
        return {"X": O.fill_normal(fdt, case["shape"], 110, 0.0, 2.0)}
    if op == "softmax_fp32_out":
        X = O.fill_normal(fdt, case["shape"], 110, 0.0, 2.0)
        Xf = O.to_f32(X, fdt)
        for r in range(X.shape[0]):                       # a unique maximum per row (with ties the reference's arg-max is arbitrary)
            X[r, (997 * (r + 1)) % X.shape[1]] = O.from_f32(np.array([Xf[r].max() + 1.0], np.float32), fdt)[0]
        return {"X": X}
    if op == "select_experts":
        return {"X": O.fill_normal(fdt, (case["tokens"], case["n_experts"]), 111, 0.0, 1.5)}
    raise KeyError(op)
