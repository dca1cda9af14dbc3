#!/usr/bin/env python
"""Benchmark of the hot path: the Llama-3-8B-shaped elementwise op chain, forward + backward, bf16.

    python bench.py --gpus N --steps K --warmup W            this library on N B200s (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W    the CPU arm: the reference has no host implementation
                                                             of these ops, so the arm times the oracle port of its
                                                             kernels' arithmetic on all host threads

One step = one pass over one batch of 8192 tokens per GPU (weak scaling, token-sharded, no data-path collective;
the RMSNorm weight gradient is all-reduced over NCCL at N > 1):
    fwd  RMSNorm(d=4096) -> RoPE on Q [32 x 128] and K [8 x 128], theta 500000, positions 0..8191 -> SwiGLU [8192 x 14336]
    bwd  SwiGLU bwd_x -> RoPE bwd_x -> RMSNorm bwd_x and bwd_w
The two gradients of the norm run as this library's one-pass op rms_norm_bwd_x_w (X and dY read once; dX bit-identical to
rms_norm_bwd_x); --separate-norm-bwd runs the reference's two identities instead, and either way one region of the other form is
timed in the same run (`norm_backward.other_form`). All ops are submitted through the Dataflow_Handle API (submit_* -> registry lookup -> external op -> C-ABI launcher -> kernel).
Synthetic seeded inputs (N(0,1); weight N(1, 0.02)). The working set of a step (1.7 GiB) is 13x the 126 MB L2.

`value`   tokens/s with inputs resident in HBM, CUDA events on the handle's stream, max over ranks.
`e2e`     the same chain with HOST buffers: every step copies its inputs from pinned host memory through
          handle->submit_inbound_transfer, runs the ops, and reads the weight gradient and the per-row statistics
          back through submit_outbound_transfer.
`roofline` the dominant kernel (swiglu_bwd_x: 5 tensors x 14336 x 2 B per token), timed with events around each launch.

    python bench.py --workload stack [--gpus N]              a second, non-default workload: the 4-layer token-sharded training
                                                             step (FP8 FFN, vocabulary projection, fused softmax + cross entropy)
"""
import argparse
import faulthandler
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, D_MODEL, N_HEADS, N_KV, HEAD_DIM, FFN, THETA, EPS = 8192, 4096, 32, 8, 128, 14336, 500000, 1e-5
WORKLOAD = "llama3-8b layer elementwise chain fwd+bwd (RMSNorm d=4096 -> RoPE 32q/8kv x128 -> SwiGLU 14336), bf16, 8192 tokens/GPU"
METRIC, UNIT = "tokens_per_s_op_chain", "tokens/s"

# algorithmic HBM bytes per token of each op (bf16): what the op must read and write once
BYTES_PER_TOKEN = {
    "rms_norm": 2 * D_MODEL * 2 + 8, "rope": 2 * (N_HEADS + N_KV) * HEAD_DIM * 2 + 4, "swiglu": 3 * FFN * 2,
    "swiglu_bwd_x": 5 * FFN * 2, "rope_bwd_x": 2 * (N_HEADS + N_KV) * HEAD_DIM * 2 + 4,
    "rms_norm_bwd_x": 4 * D_MODEL * 2 + 8, "rms_norm_bwd_w": 2 * D_MODEL * 2 + 4,
    "rms_norm_bwd_x_w": 4 * D_MODEL * 2 + 8,        # both gradients of the norm in one pass: X, dY and dX read once, dX written
}
# The backward of the norm runs as this library's one-pass op (rms_norm_bwd_x_w: 4 d e bytes per token) unless --separate-norm-bwd asks
# for the reference's two identities (rms_norm_bwd_x, then rms_norm_bwd_w reading X and dY again: 6 d e bytes per token).
CHAIN_OPS = ["rms_norm", "rope", "swiglu", "swiglu_bwd_x", "rope_bwd_x", "rms_norm_bwd_x_w"]
CHAIN_OPS_SEPARATE = ["rms_norm", "rope", "swiglu", "swiglu_bwd_x", "rope_bwd_x", "rms_norm_bwd_x", "rms_norm_bwd_w"]
DOMINANT = "swiglu_bwd_x"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu capture summarised in
# profiles/swiglu_bwd_x_bf16_2048x14336.md: reads scale with the rows and equal the algorithmic 704.6 MB; DRAM writes are
# the algorithmic 469.8 MB minus ~51.6 MB that is still dirty in L2 when the kernel ends (size-independent residue). (Inside the
# chain the kernel starts with the tail of x_w1 and x_w3 already in L2, left there by swiglu: up to ~126 MB fewer DRAM reads.)
DOMINANT_DRAM_TRAFFIC_BYTES = 1_122_800_000


def quiet_nccl_banner():
    """NCCL writes its debug output to STDOUT; at the VERSION level (which ignores NCCL_DEBUG_FILE) that is a version banner beside the
    JSON line. VERSION is raised to WARN and the output sent to stderr, unless the caller chose a more verbose level or a file."""
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")


def measured_peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (earlier measurement on this pool)"


# ----------------------------------------------------------------------------------------------- CPU arm

def cpu_chain_tokens_per_s(sample_tokens, threads):
    """The oracle port of the chain on `sample_tokens` tokens; returns (tokens/s, seconds)."""
    import numpy as np
    import oracle as O
    T = sample_tokens
    X, w, dY = O.fill_normal(O.BF16, (T, D_MODEL), 1), O.fill_normal(O.BF16, (D_MODEL,), 2, 1.0, 0.02), O.fill_normal(O.BF16, (T, D_MODEL), 3)
    Q, K = O.fill_normal(O.BF16, (T, N_HEADS * HEAD_DIM), 4), O.fill_normal(O.BF16, (T, N_KV * HEAD_DIM), 5)
    g, u, dS = O.fill_normal(O.BF16, (T, FFN), 6), O.fill_normal(O.BF16, (T, FFN), 7), O.fill_normal(O.BF16, (T, FFN), 8)
    pos = np.arange(T, dtype=np.int32)
    dX, dW = np.zeros_like(X), np.zeros_like(w)
    t0 = time.perf_counter()
    _, ws, rms = O.rms_norm(O.BF16, EPS, w, X, threads=threads)
    q, k = O.rope(O.BF16, N_HEADS * HEAD_DIM, HEAD_DIM, N_KV, THETA, pos, Q, K, threads=threads)
    O.swiglu(O.BF16, g, u, threads=threads)
    O.swiglu_bwd_x(O.BF16, O.BF16, g, u, dS, threads=threads)
    O.rope(O.BF16, N_HEADS * HEAD_DIM, HEAD_DIM, N_KV, THETA, pos, q, k, bwd=True, threads=threads)
    O.rms_norm_bwd_x(O.BF16, O.BF16, ws, rms, w, X, dY, dX, threads=threads)
    O.rms_norm_bwd_w(O.BF16, O.BF16, rms, X, dY, dW, threads=threads)
    dt = time.perf_counter() - t0
    return T / dt, dt


def cpu_baseline(target_seconds=12.0):
    threads = os.cpu_count() or 1
    rate, _ = cpu_chain_tokens_per_s(64, threads)                       # calibration
    sample = int(min(TOKENS, max(64, rate * target_seconds)))
    sample -= sample % 64
    rate, secs = cpu_chain_tokens_per_s(sample, threads)
    passes, total = 1, secs
    while total < target_seconds and passes < 64:                       # the whole batch is short on a many-core host: repeat it
        _, secs = cpu_chain_tokens_per_s(sample, threads)
        passes, total = passes + 1, total + secs
    out = {"value": sample * passes / total, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": f"{passes} passes over {sample} of {TOKENS} tokens of the same chain, oracle/oracle.c on {threads} threads, {total:.1f} s"}
    ref = reference_convert_rate(threads)
    if ref is not None:
        out["reference_convert_datatype"] = ref
    return out


def reference_convert_rate(threads):
    """The one piece of the path the reference implements on the CPU: dataflow_convert_datatype (src/datatype/src/dataflow_datatype.c:81-90),
    used to make bf16 inputs from fp32. Times the reference's own build of it (oracle/_ref/libref_host.so, when present) and this
    library's host implementation on the chain's activation shape [8192, 4096], fp32 -> bf16, same thread count."""
    import ctypes as C
    import numpy as np
    so = os.path.join(ROOT, "oracle", "_ref", "libref_host.so")
    if not os.path.exists(so):
        return None
    try:
        ref = C.CDLL(so)
        from dataflow_lib_b200 import _lib
    except OSError:
        return None
    sig = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_long, C.c_int]
    ref.dataflow_convert_datatype.argtypes = sig
    n = TOKENS * D_MODEL
    src = np.random.default_rng(0).standard_normal(n, dtype=np.float32)
    dst_ref, dst_own = np.empty(n, np.uint16), np.empty(n, np.uint16)
    FP32, BF16 = 3, 5

    def rate(fn, dst):
        fn(dst.ctypes.data, src.ctypes.data, BF16, FP32, n, threads)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 1.0:
            fn(dst.ctypes.data, src.ctypes.data, BF16, FP32, n, threads)
            reps += 1
        return n * reps / (time.perf_counter() - t0)
    r_ref, r_own = rate(ref.dataflow_convert_datatype, dst_ref), rate(_lib.lib.dataflow_convert_datatype, dst_own)
    return {"kind": "reference", "what": f"fp32 -> bf16 of [{TOKENS}, {D_MODEL}] on {threads} threads", "reference_elements_per_s": r_ref,
            "this_library_elements_per_s": r_own, "identical_output": bool(np.array_equal(dst_ref, dst_own))}


def chain_config(world):
    """The `config` object of the JSON line: the same for this library's arm and for the CPU arm, so that the two lines compare."""
    return {"workload": WORKLOAD, "tokens_per_gpu": TOKENS, "l2": "inputs larger than L2 (1.7 GiB touched per step vs 126 MB)",
            "parallelism": f"token-sharded x{world}" + (", NCCL all-reduce (from C) of the packed loss / RMSNorm weight gradient buffer" if world > 1 else "")}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # a step is one pass of the chain over the whole batch of 8192 tokens, as in this library's arm (0.3 - 0.5 s on 16 - 32 host threads)
    for _ in range(args.warmup):
        cpu_chain_tokens_per_s(TOKENS, threads)
    times = []
    for _ in range(args.steps):
        _, secs = cpu_chain_tokens_per_s(TOKENS, threads)
        times.append(secs)
    total = sum(times)
    value = TOKENS * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": chain_config(args.gpus),
        "note": "the reference ships these ops only as CUDA kernels; this arm is the CPU port of their arithmetic (oracle/oracle.c) on all host "
                "threads of rank 0, one full batch per step; it does not grow with --gpus",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"{TOKENS} tokens per step on {threads} threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm

def other_configs(hbm_peak):
    """Untimed extras for the JSON line (N = 1 only, after the timed regions): the other configurations of the hot path, each op
    launched 5 times back to back between two CUDA events after a warm-up launch, through the C-ABI launchers on torch tensors.
    HBM-bound ops report algorithmic GB/s and its fraction of the measured copy ceiling; the FP8 FFN reports TFLOP/s."""
    import torch
    from dataflow_lib_b200 import ops

    def timed(fn, n=5):
        fn(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g).bfloat16()
    hbm = lambda nbytes, ms: {"ms": ms, "GB/s": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / hbm_peak}
    out = {}
    # C1: RMSNorm 4096 x 4096 (32 MiB tensors: partly L2-resident when repeated, as the configuration is defined)
    R, C = 4096, 4096
    X, dY, w = rn(R, C), rn(R, C), (1 + 0.02 * torch.randn(C, device="cuda", generator=g)).bfloat16()
    Y, dX, dW = torch.empty_like(X), torch.zeros_like(X), torch.zeros(C, device="cuda", dtype=torch.bfloat16)
    ws, rms = torch.empty(R, device="cuda"), torch.empty(R, device="cuda")
    def c1_sequence():
        ops.rms_norm(R, C, EPS, w, X, Y, ws, rms)
        ops.rms_norm_bwd_x(R, C, EPS, ws, rms, w, X, dY, dX)
        ops.rms_norm_bwd_w(R, C, EPS, rms, X, dY, dW)
    def c1_one_pass_sequence():
        ops.rms_norm(R, C, EPS, w, X, Y, ws, rms)
        ops.rms_norm_bwd_x_w(R, C, EPS, ws, rms, w, X, dY, dX, dW)
    out["c1_rms_norm_4096x4096"] = {
        "fwd": hbm(2 * R * C * 2, timed(lambda: ops.rms_norm(R, C, EPS, w, X, Y, ws, rms))),
        "bwd_x": hbm(4 * R * C * 2, timed(lambda: ops.rms_norm_bwd_x(R, C, EPS, ws, rms, w, X, dY, dX))),
        "bwd_w": hbm(2 * R * C * 2, timed(lambda: ops.rms_norm_bwd_w(R, C, EPS, rms, X, dY, dW))),
        "bwd_x_w": hbm(4 * R * C * 2, timed(lambda: ops.rms_norm_bwd_x_w(R, C, EPS, ws, rms, w, X, dY, dX, dW))),
        "fwd_bwd_x_bwd_w_sequence": hbm(8 * R * C * 2, timed(c1_sequence, 20)),
        "fwd_bwd_x_w_sequence": hbm(6 * R * C * 2, timed(c1_one_pass_sequence, 20)),
        "note": "the configuration as it is run: forward, input gradient and weight gradient back to back (4 launches, programmatic dependent "
                "launches), 256 MiB algorithmic per sequence -- or, with both gradients in one pass over X and dY (bwd_x_w: same outputs), 3 launches and 192 MiB; the whole working set (4 x 32 MiB) is of the order of the 126 MB L2, so single ops "
                "repeated in isolation partly hit L2 and can read above the DRAM ceiling"}
    del X, dY, Y, dX
    # C3: fused softmax + cross entropy 16384 x 128256
    T3, V = 16384, 128256
    logits = (2 * torch.randn(T3, V, device="cuda", generator=g)).bfloat16()
    dlogits = torch.empty_like(logits)
    labels = torch.randint(0, V, (T3,), device="cuda", generator=g, dtype=torch.int32)
    loss = torch.zeros(2, device="cuda")
    out["c3_softmax_cross_entropy_16384x128256"] = hbm(2 * T3 * V * 2, timed(lambda: ops.softmax_cross_entropy(T3, V, logits, labels, dlogits, None, loss), 3))
    out["c3_softmax_cross_entropy_16384x128256"]["mean_loss"] = float(loss[0] / loss[1])
    del logits, dlogits
    # C4: FP8-weight SwiGLU FFN 16384 x 4096 x 14336, forward and input gradient
    T4 = 16384
    u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device="cuda")
    def qw(n_out, n_in):
        W = rn(n_out, n_in) * 0.02
        Q, sc = u8(n_out, n_in), torch.empty(n_out, device="cuda")
        ops.quantize_rows_e4m3(n_out, n_in, W.contiguous(), Q, sc)
        return Q, sc
    (Wg, sg), (Wu, su), (Wd, sd) = qw(FFN, D_MODEL), qw(FFN, D_MODEL), qw(D_MODEL, FFN)
    WguT, WdT = u8(D_MODEL, 2 * FFN), u8(FFN, D_MODEL)
    ops.ffn_fp8_prepare_bwd_weights(D_MODEL, FFN, Wg, Wu, Wd, WguT, WdT)
    A, dO = rn(T4, D_MODEL), rn(T4, D_MODEL)
    G, U = torch.empty(T4, FFN, device="cuda", dtype=torch.bfloat16), torch.empty(T4, FFN, device="cuda", dtype=torch.bfloat16)
    o, dA, sgu = torch.empty_like(A), torch.empty_like(A), torch.cat([sg, su])
    flops = 6.0 * T4 * D_MODEL * FFN
    ms_f = timed(lambda: ops.swiglu_ffn_fp8(T4, D_MODEL, FFN, A, Wg, sg, Wu, su, Wd, sd, o, G, U))
    ms_b = timed(lambda: ops.swiglu_ffn_fp8_bwd(T4, D_MODEL, FFN, dO, G, U, WdT, sd, WguT, sgu, dA))
    dGU = torch.empty(T4, 2 * FFN, device="cuda", dtype=torch.bfloat16)
    ops.swiglu_ffn_fp8_bwd(T4, D_MODEL, FFN, dO, G, U, WdT, sd, WguT, sgu, dA, dgate_dup=dGU)
    dWg, dWu, dWd = (torch.empty(s_, device="cuda", dtype=torch.bfloat16) for s_ in ((FFN, D_MODEL), (FFN, D_MODEL), (D_MODEL, FFN)))
    ms_w = timed(lambda: ops.swiglu_ffn_fp8_wgrad(T4, D_MODEL, FFN, A, dO, G, U, dGU, dWg, dWu, dWd))
    # the tensor ceiling, measured in this run: the library's e4m3 GEMM (torch._scaled_mm -> cuBLASLt) alone on the GEMM shapes of each
    # pass, without the quantisation passes an FFN op also has to run (MEASURED_PEAKS.json holds no fp8 figure)
    one = torch.ones((), device="cuda")
    def lib_gemm_ms(m, n, k):
        A8 = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
        B8 = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e4m3fn).t()
        return timed(lambda: torch._scaled_mm(A8, B8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
    try:
        g_up, g_down, g_dgrad = lib_gemm_ms(T4, FFN, D_MODEL), lib_gemm_ms(T4, D_MODEL, FFN), lib_gemm_ms(T4, D_MODEL, 2 * FFN)
        g_wdown, g_wup = lib_gemm_ms(D_MODEL, FFN, T4), lib_gemm_ms(FFN, D_MODEL, T4)
        lib = {"fwd": 2 * g_up + g_down, "bwd_input_grad": g_up + g_dgrad, "bwd_weight_grads": g_wdown + 2 * g_wup}
    except Exception as e:                                       # the library lacks an fp8 GEMM here: report without the fraction
        lib = {}
        print(f"note: no library e4m3 GEMM for the in-run ceiling ({e})", file=sys.stderr)
    def entry(name, ms):
        d = {"ms": ms, "TFLOP/s": flops / ms / 1e9}
        if name in lib:
            d["library_gemms_alone_ms"] = lib[name]
            d["library_gemms_alone_TFLOP/s"] = flops / lib[name] / 1e9
            d["frac"] = lib[name] / ms
        return d
    out["c4_swiglu_ffn_fp8_16384x4096x14336"] = {
        "fwd": entry("fwd", ms_f), "bwd_input_grad": entry("bwd_input_grad", ms_b), "bwd_weight_grads": entry("bwd_weight_grads", ms_w),
        "tokens_per_s_fwd_bwd": T4 / ((ms_f + ms_b + ms_w) * 1e-3),
        "frac_is": "time of the library's e4m3 GEMMs (cuBLASLt through torch._scaled_mm) alone on the pass's GEMM shapes / time of the pass, "
                   "both measured in this run; the pass also quantises its activations, which the library figure leaves out"}
    return out


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={uuid}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 8:
                continue
            try:
                sm.append(float(p[0])); mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(names, p[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # idle samples (before/after the kernels) would drag the median down: keep the upper half
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_memory_near_gpu(device_index):
    """Multi-rank runs: prefer this process's host memory on the NUMA node its GPU hangs off, and run on that node's CPUs where the
    allowed CPU set has any, so that eight ranks' pinned buffers are not all served by one socket's memory. Linux only
    (set_mempolicy(MPOL_PREFERRED) for this process; nothing outside it is touched); every failure leaves things as they were. Returns
    what was found and done, for the JSON line."""
    import ctypes
    import platform
    info = {"gpu_numa_node": None, "mempolicy": "unchanged", "cpu_affinity": "unchanged"}
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        if hasattr(p, "pci_bus_id"):
            bus = "%04x:%02x:%02x.0" % (getattr(p, "pci_domain_id", 0), p.pci_bus_id, getattr(p, "pci_device_id", 0))
        else:
            import pynvml
            pynvml.nvmlInit()
            raw = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(device_index)).busId
            raw = raw.decode() if isinstance(raw, bytes) else raw
            bus = raw.lower()[-12:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read())
        info["gpu_numa_node"] = node
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        info["host_numa_nodes"] = len(nodes)
        if node < 0 or len(nodes) < 2:
            return info
        if platform.machine() == "x86_64" and node < 63:
            mask = ctypes.c_ulong(1 << node)
            libc = ctypes.CDLL(None, use_errno=True)
            rc = libc.syscall(238, 1, ctypes.byref(mask), ctypes.c_ulong(64))          # set_mempolicy(MPOL_PREFERRED, {node})
            info["mempolicy"] = f"preferred node {node}" if rc == 0 else f"refused (errno {ctypes.get_errno()})"
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                if part:
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
        both = os.sched_getaffinity(0) & cpus
        if both:
            os.sched_setaffinity(0, both)
            info["cpu_affinity"] = f"{len(both)} allowed CPUs of node {node}"
        else:
            info["cpu_affinity"] = f"none of node {node}'s CPUs is in the allowed set"
    except Exception as e:                                   # placement is an optimisation: report and carry on
        info["error"] = repr(e)
    return info


def seeded_inputs(rank):
    """Host inputs of the chain: seed 0 + rank for the data, identical weights on all ranks. numpy normals rounded to bf16 by torch on the
    CPU; returned as raw 16-bit arrays (what the handle's transfers move)."""
    import numpy as np
    import torch

    def normal_bf16(shape, seed, mean=0.0, std=1.0):
        a = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
        if mean != 0.0 or std != 1.0:
            a = mean + std * a
        return torch.from_numpy(a).bfloat16().view(torch.int16).numpy().view(np.uint16)

    T, seed = TOKENS, 1000 * rank
    return {
        "X": normal_bf16((T, D_MODEL), seed + 1), "w": normal_bf16((D_MODEL,), 2, 1.0, 0.02), "dY": normal_bf16((T, D_MODEL), seed + 3),
        "Q": normal_bf16((T, N_HEADS * HEAD_DIM), seed + 4), "K": normal_bf16((T, N_KV * HEAD_DIM), seed + 5),
        "gate": normal_bf16((T, FFN), seed + 6), "up": normal_bf16((T, FFN), seed + 7), "dS": normal_bf16((T, FFN), seed + 8),
        "pos": np.arange(T, dtype=np.int32),
    }


def run_gpu_arm(args):
    import ctypes as C

    import numpy as np
    import torch
    import torch.distributed as dist

    from dataflow_lib_b200 import DataflowHandle
    from dataflow_lib_b200 import _lib as _dl
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    from dataflow_lib_b200.sharding import Exchange, PackedReduction

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch N > 1 with torchrun)"
    torch.cuda.set_device(local)
    host_numa = host_memory_near_gpu(local) if world > 1 else None      # before any host buffer of this rank exists
    if host_numa is not None:
        print(f"rank {rank}: host memory placement {host_numa}", file=sys.stderr)
    if world > 1:
        quiet_nccl_banner()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    # stream 0 computes; stream 1 (higher priority) carries the exchange; stream 2, in the end-to-end region, the next step's uploads
    h = DataflowHandle(device_id=local, num_streams=3, stream_prios=[0, -1, 0])
    stream = torch.cuda.ExternalStream(h.stream_ptr(0), device=torch.device("cuda", local))
    stream1 = torch.cuda.ExternalStream(h.stream_ptr(1), device=torch.device("cuda", local))
    BF, S0, S1, S2 = int(DT.BF16), 0, 1, 2
    T = TOKENS
    L, hp = _dl.lib, C.byref(h.h)

    # ---- host inputs, pinned through the handle
    host = seeded_inputs(rank)
    for a in host.values():
        assert h.enable_access_to_host_mem(a.ctypes.data, a.nbytes, 0) == 0
    out_host = {"dW": np.zeros(D_MODEL, np.float32 if world > 1 else np.uint16), "rms": np.zeros(T, np.float32), "ws": np.zeros(T, np.float32)}
    for a in out_host.values():
        assert h.enable_access_to_host_mem(a.ctypes.data, a.nbytes, 0) == 0

    def device_set():
        return {k: torch.empty(v.shape, dtype=torch.int32 if k == "pos" else torch.bfloat16, device="cuda") for k, v in host.items()}
    sets = [device_set(), device_set()]           # two input sets: the end-to-end region uploads step s + 1 while step s computes
    Y, dX = torch.empty_like(sets[0]["X"]), torch.zeros_like(sets[0]["X"])
    S, d1, d3 = (torch.empty_like(sets[0]["gate"]) for _ in range(3))
    dW = torch.zeros(D_MODEL, dtype=torch.bfloat16, device="cuda")
    ws, rms = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    # The step's reductions over tokens: [loss sum, valid rows | dW]. At N > 1 the weight-gradient kernel writes its fp32 column sums
    # straight into the dW slot and the packed buffer is all-reduced in place by the library's C exchange (NCCL called from C); the
    # chain has no loss, so those two floats stay zero.
    packed = PackedReduction([D_MODEL], device="cuda")
    exchange = Exchange(h) if world > 1 else None

    def upload(dev, stream_id):
        for k, a in host.items():
            assert h.submit_inbound_transfer(stream_id, dev[k], a.ctypes.data, a.nbytes) == 0

    op_names = CHAIN_OPS_SEPARATE if args.separate_norm_bwd else CHAIN_OPS
    launches_per_step = len(op_names) + 1      # the weight gradient of the norm is two launches (partial sums, final sum) in both forms
    DOM = op_names.index(DOMINANT)
    N = T * N_HEADS * HEAD_DIM

    def bind(dev, separate):
        """The submissions of one step on input set `dev`, bound once: the C entry points (submit_* of include/dataflow_api.h) with plain
        integer pointers, so that the per-step host work is the C path (skeleton + SHA-256 + table lookup + launch)."""
        P = {k: v.data_ptr() for k, v in dev.items()}
        grad = packed.dW[0].data_ptr() if world > 1 else dW.data_ptr()
        calls = [
            lambda: L.submit_rms_norm(hp, S0, BF, T, D_MODEL, EPS, P["w"], P["X"], Y.data_ptr(), ws.data_ptr(), rms.data_ptr()),
            lambda: L.submit_rope(hp, S0, BF, N, N_HEADS * HEAD_DIM, HEAD_DIM, N_KV, THETA, P["pos"], P["Q"], P["K"]),
            lambda: L.submit_swiglu(hp, S0, BF, T, FFN, P["gate"], P["up"], S.data_ptr()),
            lambda: L.submit_swiglu_bwd_x(hp, S0, BF, BF, T, FFN, P["gate"], P["up"], P["dS"], d1.data_ptr(), d3.data_ptr()),
            lambda: L.submit_rope_bwd_x(hp, S0, BF, N, N_HEADS * HEAD_DIM, HEAD_DIM, N_KV, THETA, P["pos"], P["Q"], P["K"]),
        ]
        # The weight gradient: at N > 1 fp32 column sums in their slot of the packed buffer (overwritten every step), at N = 1 the
        # reference's form, accumulated into the bf16 dW.
        norm_args = (hp, S0, BF, BF, T, D_MODEL, EPS, ws.data_ptr(), rms.data_ptr(), P["w"], P["X"], P["dY"], dX.data_ptr())
        if separate:
            calls.append(lambda: L.submit_rms_norm_bwd_x(*norm_args))
            bwd_w = L.submit_rms_norm_bwd_w_sums if world > 1 else L.submit_rms_norm_bwd_w
            calls.append(lambda: bwd_w(hp, S0, BF, BF, T, D_MODEL, EPS, rms.data_ptr(), P["X"], P["dY"], grad))
        else:
            bwd_x_w = L.submit_rms_norm_bwd_x_w_sums if world > 1 else L.submit_rms_norm_bwd_x_w
            calls.append(lambda: bwd_x_w(*norm_args, grad))
        return calls
    bound = [bind(sets[0], args.separate_norm_bwd), bind(sets[1], args.separate_norm_bwd)]
    bound_other = bind(sets[0], not args.separate_norm_bwd)        # the other form of the norm's backward, for one comparison region
    exchange_pending, exchange_due = [False], [False]
    AFTER_OP = op_names.index("rope")          # the exchange of step s is issued behind this op of step s + 1: beside `swiglu`

    def issue_exchange():
        """The data-parallel exchange (one in-place fp32 all-reduce of 16 KB, issued from C) on the handle's second stream, behind a
        dependency on what the compute stream holds so far."""
        assert h.submit_dependency(S1, h.get_stream_state(S0)) == 0
        assert exchange.all_reduce(S1, packed) == 0
        exchange_due[0], exchange_pending[0] = False, True

    def chain(events=None, only=None, which=0, calls=None):
        """One step on input set `which`. `events[i] = (start, end)` are recorded around op i (all ops, or just op `only`)."""
        calls = calls or bound[which]
        for i, call in enumerate(calls):
            timed = events is not None and (only is None or only == i)
            if world > 1 and i == len(calls) - 1 and exchange_pending[0]:
                # the weight-gradient kernel rewrites the packed buffer: it waits for the previous step's exchange on stream 1
                assert h.submit_dependency(S0, h.get_stream_state(S1)) == 0
                exchange_pending[0] = False
            if timed:
                events[i][0].record(stream)
            rc = call()
            if timed:
                events[i][1].record(stream)
            if rc != 0:
                raise RuntimeError(f"submit of op {i} of the chain failed")
            if i == AFTER_OP and exchange_due[0]:
                # The previous step's exchange runs beside this step's `swiglu`, a flat grid of short CTAs that gives up a few SMs for
                # the collective's 30 - 50 us at no measurable cost. Beside a persistent grid (rms_norm, rope: every CTA resident for the
                # whole kernel) the CTAs that the collective displaces run as a second wave: rope 36 -> 47 us at N = 8 when the
                # exchange was issued right after the step.
                issue_exchange()
        if world > 1:
            exchange_due[0] = True

    def join_exchange():
        if world > 1 and exchange_due[0]:
            issue_exchange()
        if world > 1 and exchange_pending[0]:
            assert h.submit_dependency(S0, h.get_stream_state(S1)) == 0
            exchange_pending[0] = False

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    upload(sets[0], S0)
    upload(sets[1], S0)
    assert h.sync_stream(S0) == 0
    for _ in range(max(args.warmup, 3)):
        chain()
    join_exchange()
    barrier()

    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None

    # ---- timed regions 1: inputs resident in HBM; EXACTLY `steps` steps per region, `repeats` regions, each bracketed by a barrier and a
    # synchronize; the median region is reported (with the spread). Only the dominant kernel is bracketed by events (an event pair costs
    # a few microseconds of stream serialisation, which seven pairs per 0.4 ms step would distort).
    new_events = lambda: [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in op_names]
    region_ms, dom_ms_all, enqueue_ms = [], [], []
    for _ in range(max(args.repeats, 1)):
        ev = [new_events() for _ in range(args.steps)]
        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        host_t0 = time.perf_counter()
        t_begin.record(stream)
        for s in range(args.steps):
            chain(ev[s], only=DOM)
        join_exchange()
        t_end.record(stream)
        enqueue_ms.append(1e3 * (time.perf_counter() - host_t0) / args.steps)      # host time to submit one step (no sync)
        barrier()
        region_ms.append(t_begin.elapsed_time(t_end))
        dom_ms_all.append(statistics.mean(ev[s][DOM][0].elapsed_time(ev[s][DOM][1]) for s in range(args.steps)))
    regions = torch.tensor(region_ms, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(regions, op=dist.ReduceOp.MAX)           # per region: the slowest rank
    region_ms = regions.tolist()
    ms_total = statistics.median(region_ms)
    dom_ms = statistics.median(dom_ms_all)
    host_enqueue_ms = statistics.median(enqueue_ms)      # includes waiting for room in the launch queue once the region outruns it
    # the host's own cost of submitting a step: 40 steps (under 300 launches, well inside the queue) submitted to an idle device
    barrier()
    host_t0 = time.perf_counter()
    for s in range(40):
        chain()
    host_submit_ms = 1e3 * (time.perf_counter() - host_t0) / 40
    join_exchange()
    barrier()

    # ---- untimed: the dominant kernel alone, back to back (every launch re-reads its 0.7 GB of inputs from DRAM: it walks the tensors
    # from the end, so what the previous launch left in L2 is the part it reads last)
    iso = [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)]
    bound[0][DOM](); barrier()
    iso[0].record(stream)
    for _ in range(20):
        bound[0][DOM]()
    iso[1].record(stream)
    barrier()
    dom_alone_ms = iso[0].elapsed_time(iso[1]) / 20

    # ---- one region of the OTHER form of the norm's backward (separate identities when the timed regions ran the one-pass op, and
    # the other way round), for a like-for-like step time in the same run
    for _ in range(3):
        chain(calls=bound_other)
    join_exchange(); barrier()
    o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    o0.record(stream)
    for s in range(args.steps):
        chain(calls=bound_other)
    join_exchange()
    o1.record(stream)
    barrier()
    other_ms = torch.tensor([o0.elapsed_time(o1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(other_ms, op=dist.ReduceOp.MAX)
    other_form_ms_per_step = other_ms.item() / args.steps

    # ---- untimed pass: every op bracketed, for the per-op table (event-to-event times include launch latency)
    prof_steps = min(args.steps, 50)
    evp = [new_events() for _ in range(prof_steps)]
    for s in range(prof_steps):
        chain(evp[s])
    join_exchange()
    barrier()
    per_op_ms = {name: statistics.mean(evp[s][i][0].elapsed_time(evp[s][i][1]) for s in range(prof_steps)) for i, name in enumerate(op_names)}

    # ---- untimed check of the multi-rank path: the packed buffer after the C exchange against the same partial sums all-reduced by
    # torch.distributed, and against world x this rank's own sums where every rank holds the same data
    exchange_check = None
    if world > 1:
        local_sums = torch.empty(D_MODEL, device="cuda")
        with torch.cuda.stream(stream):
            if args.separate_norm_bwd:
                assert L.submit_rms_norm_bwd_w_sums(hp, S0, BF, BF, T, D_MODEL, EPS, rms.data_ptr(), sets[0]["X"].data_ptr(), sets[0]["dY"].data_ptr(), local_sums.data_ptr()) == 0
            else:       # the same one-pass op the step runs (its summation order is its own), on a scratch dX
                scratch_dX = torch.zeros_like(dX)
                assert L.submit_rms_norm_bwd_x_w_sums(hp, S0, BF, BF, T, D_MODEL, EPS, ws.data_ptr(), rms.data_ptr(), sets[0]["w"].data_ptr(), sets[0]["X"].data_ptr(),
                                                      sets[0]["dY"].data_ptr(), scratch_dX.data_ptr(), local_sums.data_ptr()) == 0
        chain(); join_exchange()
        barrier()
        want = local_sums.clone()
        dist.all_reduce(want)
        got = packed.dW[0]
        err = ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
        exchange_check = {"max_rel_diff_vs_torch_all_reduce": err, "ok": bool(err <= 1e-6), "loss_slots": packed.loss.tolist()}
        if not exchange_check["ok"]:
            print(f"warning: the C exchange and torch.distributed disagree (max relative difference {err:g})", file=sys.stderr)

    # ---- timed region 2: end to end with host buffers through the handle's transfer calls. Every step's inputs come from pinned host
    # memory (submit_inbound_transfer) and its results go back (submit_outbound_transfer) and are waited for; the uploads of step s + 1
    # run on stream 1 into the other input set while step s computes on stream 0.
    e2e_steps = max(3, min(args.steps, 10))
    h2d = sum(a.nbytes for a in host.values())
    grad_src = packed.dW[0] if world > 1 else dW
    d2h = sum(a.nbytes for a in out_host.values())

    def e2e_region(n_steps):
        upload(sets[0], S2)
        for s in range(n_steps):
            b = s & 1
            assert h.submit_dependency(S0, h.get_stream_state(S2)) == 0      # this step's inputs have arrived
            if s + 1 < n_steps:
                upload(sets[1 - b], S2)                                          # the next step's inputs, beside this step's kernels
            chain(which=b)
            join_exchange()
            assert h.submit_outbound_transfer(S0, out_host["dW"].ctypes.data, grad_src, out_host["dW"].nbytes) == 0
            assert h.submit_outbound_transfer(S0, out_host["rms"].ctypes.data, rms, out_host["rms"].nbytes) == 0
            assert h.submit_outbound_transfer(S0, out_host["ws"].ctypes.data, ws, out_host["ws"].nbytes) == 0
            assert h.sync_stream(S0) == 0                                        # the host consumes the result every step

    e2e_region(2)
    e2e_ms = []
    for _ in range(3):
        e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e_begin.record(stream)
        e2e_region(e2e_steps)
        e_end.record(stream)
        barrier()
        e2e_ms.append(e_begin.elapsed_time(e_end))
    # the host-side ceiling of that region: the same uploads alone, all ranks at once
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    c0.record(stream1)
    for _ in range(3):
        upload(sets[0], S1)
    c1.record(stream1)
    barrier()
    copy_ms = c0.elapsed_time(c1) / 3

    clocks = sampler.stop() if sampler else None

    times = torch.tensor(e2e_ms + [copy_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    *e2e_ms, copy_ms = times.tolist()
    ms_e2e = statistics.median(e2e_ms)

    c5 = None
    if not args.no_stack:
        # configuration C5 on the same GPUs: the token-sharded 4-layer step, after the chain's timed regions
        c5 = stack_step_report(rank, world, local, steps=5, warmup=3, tokens=16384)

    if rank == 0:
        peak, peak_src = measured_peak_hbm()
        dom_bytes = BYTES_PER_TOKEN[DOMINANT] * T
        achieved, alone = dom_bytes / (dom_ms * 1e-3) / 1e9, dom_bytes / (dom_alone_ms * 1e-3) / 1e9
        ops_report = {name: {"ms": per_op_ms[name], "GB/s": BYTES_PER_TOKEN[name] * T / (per_op_ms[name] * 1e-3) / 1e9,
                             "frac_of_peak": BYTES_PER_TOKEN[name] * T / (per_op_ms[name] * 1e-3) / 1e9 / peak} for name in op_names}
        step_bytes = sum(BYTES_PER_TOKEN[name] for name in op_names) * T
        other_names = CHAIN_OPS if args.separate_norm_bwd else CHAIN_OPS_SEPARATE
        other_bytes = sum(BYTES_PER_TOKEN[name] for name in other_names) * T
        cpu = cpu_baseline() if world == 1 else None
        others = other_configs(peak) if (world == 1 and not args.no_other_configs) else {}
        if c5 is not None:
            others = dict(others or {}, c5_stack_4layer=c5)
        line = {
            "metric": METRIC, "value": world * T * args.steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": chain_config(world),
            "timed_regions": {"repeats": len(region_ms), "steps_each": args.steps, "ms": region_ms, "reported": "median",
                              "min_ms_per_step": min(region_ms) / args.steps, "max_ms_per_step": max(region_ms) / args.steps},
            "step_hbm": {"algorithmic_bytes": step_bytes, "GB/s": step_bytes / (ms_total / args.steps * 1e-3) / 1e9,
                         "frac_of_peak": step_bytes / (ms_total / args.steps * 1e-3) / 1e9 / peak},
            "roofline": {"bound": "hbm", "kernel": DOMINANT, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": DOMINANT_DRAM_TRAFFIC_BYTES, "algorithmic_bytes": dom_bytes, "peak_source": peak_src,
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "alone": {"achieved": alone, "frac": alone / peak, "ms": dom_alone_ms,
                                   "what": "the same kernel launched 20 times back to back by itself in this run: every byte comes from DRAM"},
                         "traffic_source": "profiles/swiglu_bwd_x_bf16_2048x14336.md: ncu capture of the kernel alone at 2048 rows, reads scaled by the rows "
                                           "(x4), writes less the size-independent ~52 MB still dirty in L2 at kernel end",
                         "note": "achieved / frac are measured inside the chain, where the kernel follows swiglu on the same x_w1, x_w3 and walks "
                                 "them from the end: the ~126 MB that swiglu left in L2 are not re-read from DRAM, so frac can pass 1; `alone` is the "
                                 "distance to the DRAM roofline"},
            "ops_event_bracketed": ops_report,
            "norm_backward": {"form": "separate rms_norm_bwd_x + rms_norm_bwd_w (the reference's identities)" if args.separate_norm_bwd
                                      else "one pass: rms_norm_bwd_x_w (dX bit-identical to rms_norm_bwd_x, dW summed in fp32)",
                              "other_form": {"ops": other_names, "ms_per_step": other_form_ms_per_step, "algorithmic_bytes": other_bytes,
                                             "tokens_per_s": world * T / (other_form_ms_per_step * 1e-3),
                                             "what": f"one region of {args.steps} steps with the other form of the norm's backward, same run"}},
            "e2e": {"value": world * T * e2e_steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": ms_e2e / e2e_steps, "regions_ms": e2e_ms, "reported": "median of 3 regions",
                    "copy_ms": copy_ms, "compute_ms": ms_total / args.steps,
                    "h2d_GBps_per_rank": h2d / (copy_ms * 1e-3) / 1e9, "h2d_GBps_all_ranks": world * h2d / (copy_ms * 1e-3) / 1e9,
                    "note": "uploads of step s + 1 run on stream 1 beside the kernels of step s; copy_ms is the upload of one step alone with all "
                            "ranks copying at once (slowest rank): the host-side ceiling of this region"},
            "gpu_launches": launches_per_step * args.steps * len(region_ms),
            "host_enqueue_ms_per_step": host_enqueue_ms,
            "host_submit_ms_per_step": host_submit_ms,
            "host_note": "host_submit = wall time per step of submitting 40 steps to an idle device (the C path: skeleton, SHA-256, table lookup, "
                         "launch, through ctypes); host_enqueue = the same inside the timed regions, where the host runs a full launch queue ahead "
                         "of the device and mostly waits for room in it",
            "clocks": clocks,
        }
        if exchange_check is not None:
            line["exchange_check"] = exchange_check
        if host_numa is not None:
            line["host_numa"] = host_numa
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if others:
            line["other_configs"] = others
        print(json.dumps(line), flush=True)

    for a in list(host.values()) + list(out_host.values()):
        h.disable_access_to_host_mem(a.ctypes.data)
    if exchange is not None:
        exchange.close()
    h.close()
    if world > 1:
        dist.destroy_process_group()


def stack_step_report(rank, world, local, steps, warmup, tokens, with_clocks=False):
    """The token-sharded 4-layer training step of dataflow_lib_b200/op_stack.py (configuration C5: 16384 tokens per GPU, d 4096, ffn
    14336, 32/8 heads x 128, vocabulary 128256; bf16 activations, FP8 FFN weights, seed-0 random weights identical on every rank, data
    seeded per rank; loss sum and RMSNorm weight gradients in one packed buffer all-reduced by the library's C exchange). Returns the
    report on rank 0 (None elsewhere); torch.distributed must already be initialised when world > 1."""
    import torch
    import torch.distributed as dist

    from dataflow_lib_b200 import ops
    from dataflow_lib_b200.op_stack import OpStackStep

    T, V, LAYERS = tokens, 128256, 4
    st = OpStackStep(T, D_MODEL, FFN, N_HEADS, N_KV, HEAD_DIM, V, LAYERS, EPS, float(THETA), device=f"cuda:{local}")
    st.random_weights(seed=0)
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    host_x = torch.randn(T, D_MODEL, generator=g, device="cuda").bfloat16().cpu().pin_memory()
    host_labels = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32).cpu().pin_memory()
    host_loss = torch.zeros(2).pin_memory()
    st.x[0].copy_(host_x); st.labels.copy_(host_labels)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(warmup, 3)
    for _ in range(warm):
        st.step()
    barrier()
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid)) if (rank == 0 and with_clocks) else None
    ev = lambda: torch.cuda.Event(enable_timing=True)
    t0, t1 = ev(), ev()
    barrier()
    t0.record(st.stream)
    for _ in range(steps):
        st.step(overlap=True)                     # the all-reduce runs beside the next step; the last one is waited for below
    st.wait_exchange()
    t1.record(st.stream)
    barrier()
    ms_total = t0.elapsed_time(t1)
    exchange_check = None
    if world > 1:
        # untimed check of the C exchange: the step's packed partial sums all-reduced once more by torch.distributed
        st.step(overlap=True); st.wait_exchange()
        barrier()
        got = st.reduced.clone()
        partial = torch.empty_like(got)
        saved_exchange, st._exchange = st._exchange, _NoExchange()
        st.step()                                  # the same step without the collective: this rank's own sums
        barrier()
        partial.copy_(st.reduced)
        st._exchange = saved_exchange
        want = partial.clone()
        dist.all_reduce(want)
        err = ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
        exchange_check = {"max_rel_diff_vs_torch_all_reduce": err, "ok": bool(err <= 1e-6)}
        if not exchange_check["ok"]:
            print(f"warning: stack step: the C exchange and torch.distributed disagree (max relative difference {err:g})", file=sys.stderr)

    # end to end: the step's tokens and labels come from pinned host memory, the loss goes back, every step
    e_steps = max(3, min(steps, 10))
    def e2e_step():
        with torch.cuda.stream(st.stream):
            st.x[0].copy_(host_x, non_blocking=True); st.labels.copy_(host_labels, non_blocking=True)
        st.step()
        with torch.cuda.stream(st.stream):
            host_loss.copy_(st.loss_sum, non_blocking=True)
        st.stream.synchronize()
    e2e_step()
    e0, e1 = ev(), ev()
    barrier()
    e0.record(st.stream)
    for _ in range(e_steps):
        e2e_step()
    e1.record(st.stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    # untimed accounting: three more steps with an event at every segment boundary, and this library's dominant kernel by itself
    st.marks = []
    for _ in range(3):
        st.step()
    torch.cuda.synchronize()
    breakdown = {k: v / 3 for k, v in st.segment_ms().items()}
    st.marks = None

    def timed(fn, n=5):
        fn(); a, b = ev(), ev()
        a.record()
        for _ in range(n):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / n
    Aq = torch.empty(T, D_MODEL, dtype=torch.uint8, device="cuda"); sa = torch.empty(T, device="cuda")
    ops.quantize_rows_e4m3(T, D_MODEL, st.h, Aq, sa)
    # the gate projection as the FFN forward runs it: e4m3 x e4m3 -> bf16 [T, FFN], K = d_model
    ms_gemm = timed(lambda: ops.gemm_e4m3(T, FFN, D_MODEL, Aq, sa, st.Wg[0], st.sg[0], st.G[0]))
    clocks = sampler.stop() if sampler else None
    status = ops.read_kernel_status()
    assert not any(status), f"a device-side wait gave up: {status}"

    times = torch.tensor([ms_total, ms_e2e], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = times.tolist()
    loss = float(st.loss_sum[0]) / max(float(st.loss_sum[1]), 1.0)
    launches = st.library_launches_per_step()
    st.close()
    if rank != 0:
        return None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            bf16_sustained, src = float(json.load(f)["bf16_tflops_sustained"]), "2 x bf16_tflops_sustained of MEASURED_PEAKS.json (it holds no fp8 figure)"
    except (OSError, KeyError, ValueError):
        bf16_sustained, src = 1400.0, "2 x the fallback's sustained bf16 figure"
    flops = 2.0 * T * D_MODEL * FFN
    achieved = flops / (ms_gemm * 1e-3) / 1e12
    return {
        "metric": "tokens_per_s_op_stack_step", "value": world * T * steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": ms_total / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 activations, e4m3 FFN operands with fp32 accumulation", "data": "synthetic",
        "config": {"workload": f"4-layer op stack step fwd+bwd (RMSNorm -> RoPE -> FP8 SwiGLU FFN + residual) x4 + head (RMSNorm -> vocabulary GEMM -> "
                               f"fused softmax+CE), {T} tokens/GPU, d 4096, ffn 14336, vocab 128256",
                   "tokens_per_gpu": T, "l2": "inputs larger than L2 (tens of GB touched per step)",
                   "parallelism": f"token-sharded x{world}" + (", packed loss / RMSNorm weight gradient buffer all-reduced over NCCL from C on a side stream, overlapped with the next step" if world > 1 else "")},
        "roofline": {"bound": "tensor", "kernel": "gemm_e4m3_kernel<PLAIN, CTA pair> (the gate projection of the FFN forward, timed alone after the step)", "achieved": achieved,
                     "peak": 2 * bf16_sustained, "unit": "TFLOP/s", "frac": achieved / (2 * bf16_sustained), "traffic": None, "peak_source": src},
        "step_breakdown_ms": breakdown, "exchange_check": exchange_check,
        "e2e": {"value": world * T * e_steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": host_x.numel() * 2 + host_labels.numel() * 4,
                "d2h_bytes_per_step": 8, "steps": e_steps, "ms_per_step": ms_e2e / e_steps},
        "gpu_launches": launches * steps,
        "loss": loss,
        "clocks": clocks,
    }


class _NoExchange:
    """Stands in for the exchange during the untimed multi-rank check: the step without its collective."""
    def all_reduce(self, stream_id, packed, count=None):
        return 0

    def close(self):
        pass


def run_stack_arm(args):
    """--workload stack: configuration C5 by itself (the default workload reports it under other_configs.c5_stack_4layer). `value` is
    tokens/s of the whole step, the library vocabulary GEMMs included and reported separately in the breakdown."""
    import torch
    import torch.distributed as dist

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch N > 1 with torchrun)"
    torch.cuda.set_device(local)
    if world > 1:
        quiet_nccl_banner()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    line = stack_step_report(rank, world, local, steps=args.steps, warmup=args.warmup, tokens=args.tokens or 16384, with_clocks=True)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    faulthandler.enable()                      # a crash in native code leaves the Python stack on stderr
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="chain", choices=["chain", "stack"],
                    help="chain (default): the elementwise op chain the headline metric is quoted on; stack: the 4-layer token-sharded training step")
    ap.add_argument("--tokens", type=int, default=0, help="stack workload only: tokens per GPU (default 16384)")
    ap.add_argument("--repeats", type=int, default=7, help="chain workload: timed regions of --steps steps each; the median region is reported")
    ap.add_argument("--separate-norm-bwd", action="store_true",
                    help="chain workload: run the norm's backward as the reference's two identities (rms_norm_bwd_x, rms_norm_bwd_w) instead of the one-pass op")
    ap.add_argument("--no-stack", action="store_true", help="chain workload: skip the 4-layer stack step (other_configs.c5_stack_4layer)")
    ap.add_argument("--no-other-configs", action="store_true", help="chain workload, N = 1: skip configurations C1, C3 and C4")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "stack":
        if args.steps == 200:
            args.steps = 10
        run_stack_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
