"""Generates tests/golden/reference_vectors.npz: outputs of the REFERENCE's own CUDA kernels on small seeded inputs.

Runs on a GPU box. The kernels are oracle/_ref/cuda_kernels.cubin -- als244/dataflow_lib's src/ops/nvidia/cuda_kernels.cu
compiled unchanged (its own flags, -arch sm_100a) by `make -C oracle ref` -- launched by tests/ref_kernels.py with the
reference's launch geometry. Inputs are regenerated from (seed, shape) by oracle.fill_normal, so only outputs are
stored (raw bits). tests/test_oracle_cpu.py checks the CPU oracle against this file on machines without a GPU.

    python tests/golden/make_reference_vectors.py [out.npz]
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle as O  # noqa: E402
from ref_kernels import RefKernels  # noqa: E402
from util import DT_NAME, to_dev, to_host  # noqa: E402
from golden_cases import CASES, inputs_for  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_vectors.npz")
    ref = RefKernels()
    blobs = {}
    for name, case in CASES.items():
        inp = inputs_for(case)
        op, fdt, bdt = case["op"], case["fdt"], case.get("bdt", case["fdt"])
        nf, nb = DT_NAME[fdt], DT_NAME[bdt]
        d = {k: (to_dev(v, case["dts"][k]) if k in case["dts"] else torch.from_numpy(v).cuda()) for k, v in inp.items()}
        if op == "rms_norm":
            R, Cn = inp["X"].shape
            out, ws, rms = torch.empty_like(d["X"]), torch.zeros(R, device="cuda"), torch.zeros(R, device="cuda")
            ref.rms_norm(nf, O.oracle_sizeof(fdt) if hasattr(O, "oracle_sizeof") else {3: 4, 4: 2, 5: 2, 6: 1, 7: 1}[fdt], R, Cn, 1e-5, d["w"], d["X"], out, ws, rms)
            blobs[name + "/out"], blobs[name + "/ws"], blobs[name + "/rms"] = to_host(out, fdt), ws.cpu().numpy(), rms.cpu().numpy()
        elif op == "rms_norm_bwd_x":
            R, Cn = inp["X"].shape
            ref.rms_norm_bwd_x(f"{nf}_{nb}", R, Cn, 1e-5, d["ws"], d["rms"], d["w"], d["X"], d["dY"], d["dX"])
            blobs[name + "/dX"] = to_host(d["dX"], bdt)
        elif op == "rms_norm_bwd_w":
            R, Cn = inp["X"].shape
            ref.rms_norm_bwd_w(f"{nf}_{nb}", R, Cn, 1e-5, d["rms"], d["X"], d["dY"], d["dW"])
            blobs[name + "/dW"] = to_host(d["dW"], bdt)
        elif op in ("rope", "rope_bwd_x"):
            T = inp["Q"].shape[0]
            ref.rope(nf, T * case["model_dim"], case["model_dim"], case["head_dim"], case["n_kv"], case["theta"], d["pos"], d["Q"], d["K"], bwd=(op == "rope_bwd_x"))
            blobs[name + "/Q"], blobs[name + "/K"] = to_host(d["Q"], fdt), to_host(d["K"], fdt)
        elif op == "swiglu":
            R, Cn = inp["x1"].shape
            out = torch.empty_like(d["x1"])
            ref.swiglu(nf, R, Cn, d["x1"], d["x3"], out)
            blobs[name + "/out"] = to_host(out, fdt)
        elif op == "swiglu_bwd_x":
            R, Cn = inp["x1"].shape
            d1, d3 = torch.empty_like(d["dY"]), torch.empty_like(d["dY"])
            ref.swiglu_bwd_x(f"{nf}_{nb}", R, Cn, d["x1"], d["x3"], d["dY"], d1, d3)
            blobs[name + "/d1"], blobs[name + "/d3"] = to_host(d1, bdt), to_host(d3, bdt)
        elif op == "softmax":
            R, Cn = inp["X"].shape
            out = torch.empty((R, Cn), dtype=to_dev(np.zeros(1, O.NP_OF[bdt]), bdt).dtype, device="cuda")
            ref.softmax(f"{nf}_{nb}", R, Cn, d["X"], out)
            blobs[name + "/out"] = to_host(out, bdt)
        elif op == "softmax_fp32_out":
            R, Cn = inp["X"].shape
            out, arg = torch.empty((R, Cn), device="cuda"), torch.zeros(R, dtype=torch.int32, device="cuda")
            ref.softmax_fp32_out(nf, R, Cn, d["X"], out, arg)
            blobs[name + "/out"], blobs[name + "/argmax"] = out.cpu().numpy(), arg.cpu().numpy().view(np.uint32)
        elif op == "select_experts":
            T, ne, k = case["tokens"], case["n_experts"], case["top_k"]
            w = torch.zeros((T, k), dtype=d["X"].dtype, device="cuda")
            ids = torch.zeros((T, k), dtype=torch.int16, device="cuda")
            counts = torch.zeros(ne + 1, dtype=torch.int32, device="cuda")
            cum, routed = torch.zeros(ne, dtype=torch.int32, device="cuda"), torch.ones(ne, dtype=torch.int32, device="cuda")
            ref.select_experts(nf, T, ne, k, d["X"], w, ids, counts, cum, routed)
            torch.cuda.synchronize()
            blobs[name + "/weights"], blobs[name + "/ids"] = to_host(w, fdt), ids.cpu().numpy().view(np.uint16)
            blobs[name + "/counts"] = counts.cpu().numpy()
        torch.cuda.synchronize()
    np.savez_compressed(out_path, **blobs)
    print(f"wrote {len(blobs)} arrays for {len(CASES)} cases to {out_path} ({os.path.getsize(out_path) / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
