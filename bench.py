#!/usr/bin/env python
"""Benchmark of the hot path: the Llama-3-8B-shaped elementwise op chain, forward + backward, bf16.

    python bench.py --gpus N --steps K --warmup W            this library on N B200s (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W    the CPU arm: the reference has no host implementation
                                                             of these ops, so the arm times the oracle port of its
                                                             kernels' arithmetic on all host threads

One step = one pass over one batch of 8192 tokens per GPU (weak scaling, token-sharded, no data-path collective;
the RMSNorm weight gradient is all-reduced over NCCL at N > 1):
    fwd  RMSNorm(d=4096) -> RoPE on Q [32 x 128] and K [8 x 128], theta 500000, positions 0..8191 -> SwiGLU [8192 x 14336]
    bwd  SwiGLU bwd_x -> RoPE bwd_x -> RMSNorm bwd_x -> RMSNorm bwd_w
submitted through the Dataflow_Handle API (submit_* -> registry lookup -> external op -> C-ABI launcher -> kernel).
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
}
KERNEL_LAUNCHES_PER_STEP = 8          # 7 ops; rms_norm_bwd_w is two launches
DOMINANT = "swiglu_bwd_x"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu capture summarised in
# profiles/swiglu_bwd_x_bf16_2048x14336.md: reads scale with the rows and equal the algorithmic 704.6 MB; DRAM writes are
# the algorithmic 469.8 MB minus ~41.6 MB that is still dirty in L2 when the kernel ends (size-independent residue). (Inside the
# chain the kernel starts with the tail of x_w1 and x_w3 already in L2, left there by swiglu: up to ~126 MB fewer DRAM reads.)
DOMINANT_DRAM_TRAFFIC_BYTES = 1_132_800_000


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


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rate, _ = cpu_chain_tokens_per_s(64, threads)
    # a step is a bounded sample of the workload: about min(1 s, 150 s / K) of CPU work
    sample = int(max(64, min(TOKENS, rate * min(1.0, 150.0 / max(args.steps, 1)))))
    sample -= sample % 64
    for _ in range(args.warmup):
        cpu_chain_tokens_per_s(sample, threads)
    times = []
    for _ in range(args.steps):
        _, secs = cpu_chain_tokens_per_s(sample, threads)
        times.append(secs)
    total = sum(times)
    value = sample * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": WORKLOAD, "note": "the reference ships these ops only as CUDA kernels; this arm is the CPU port "
                                        "of their arithmetic (oracle/oracle.c), each step a bounded sample of the workload (see cpu_baseline.sample)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"{sample} tokens per step on {threads} threads"},
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
    out["c1_rms_norm_4096x4096"] = {
        "fwd": hbm(2 * R * C * 2, timed(lambda: ops.rms_norm(R, C, EPS, w, X, Y, ws, rms))),
        "bwd_x": hbm(4 * R * C * 2, timed(lambda: ops.rms_norm_bwd_x(R, C, EPS, ws, rms, w, X, dY, dX))),
        "bwd_w": hbm(2 * R * C * 2, timed(lambda: ops.rms_norm_bwd_w(R, C, EPS, rms, X, dY, dW))),
        "note": "64-128 MiB per launch against a 126 MB L2: repeated launches partly hit L2"}
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
    out["c4_swiglu_ffn_fp8_16384x4096x14336"] = {"fwd": {"ms": ms_f, "TFLOP/s": flops / ms_f / 1e9}, "bwd_input_grad": {"ms": ms_b, "TFLOP/s": flops / ms_b / 1e9},
                                                 "bwd_weight_grads": {"ms": ms_w, "TFLOP/s": flops / ms_w / 1e9},
                                                 "tokens_per_s_fwd_bwd": T4 / ((ms_f + ms_b + ms_w) * 1e-3)}
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


def run_gpu_arm(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle as O   # input generation only (seeded fills); the timed path never touches it
    from dataflow_lib_b200 import DataflowHandle
    from dataflow_lib_b200.abi import DataflowDatatype as DT
    from dataflow_lib_b200.sharding import allreduce_step

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch N > 1 with torchrun)"
    torch.cuda.set_device(local)
    if world > 1:
        quiet_nccl_banner()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    h = DataflowHandle(device_id=local, num_streams=2)
    stream = torch.cuda.ExternalStream(h.stream_ptr(0), device=torch.device("cuda", local))
    stream1 = torch.cuda.ExternalStream(h.stream_ptr(1), device=torch.device("cuda", local))
    exchange_state = [None]
    BF, S0 = int(DT.BF16), 0
    T = TOKENS

    # ---- host inputs (seed 0 + rank for data, identical weights on all ranks), pinned through the handle
    seed = 1000 * rank
    host = {
        "X": O.fill_normal(O.BF16, (T, D_MODEL), seed + 1), "w": O.fill_normal(O.BF16, (D_MODEL,), 2, 1.0, 0.02),
        "dY": O.fill_normal(O.BF16, (T, D_MODEL), seed + 3), "Q": O.fill_normal(O.BF16, (T, N_HEADS * HEAD_DIM), seed + 4),
        "K": O.fill_normal(O.BF16, (T, N_KV * HEAD_DIM), seed + 5), "gate": O.fill_normal(O.BF16, (T, FFN), seed + 6),
        "up": O.fill_normal(O.BF16, (T, FFN), seed + 7), "dS": O.fill_normal(O.BF16, (T, FFN), seed + 8),
        "pos": np.arange(T, dtype=np.int32),
    }
    for a in host.values():
        assert h.enable_access_to_host_mem(a.ctypes.data, a.nbytes, 0) == 0
    out_host = {"dW": np.zeros(D_MODEL, np.uint16), "rms": np.zeros(T, np.float32), "ws": np.zeros(T, np.float32)}
    for a in out_host.values():
        assert h.enable_access_to_host_mem(a.ctypes.data, a.nbytes, 0) == 0

    dev = {k: torch.empty(v.shape, dtype=torch.int32 if k == "pos" else torch.bfloat16, device="cuda") for k, v in host.items()}
    Y, dX = torch.empty_like(dev["X"]), torch.zeros_like(dev["X"])
    S, d1, d3 = torch.empty_like(dev["gate"]), torch.empty_like(dev["gate"]), torch.empty_like(dev["gate"])
    dW = torch.zeros(D_MODEL, dtype=torch.bfloat16, device="cuda")
    ws, rms = torch.empty(T, device="cuda"), torch.empty(T, device="cuda")
    step_loss = torch.zeros(2, device="cuda")            # [loss sum, valid rows]: unused by this chain, part of the packed exchange

    def upload():
        for k, a in host.items():
            assert h.submit_inbound_transfer(S0, dev[k], a.ctypes.data, a.nbytes) == 0

    op_names = ["rms_norm", "rope", "swiglu", "swiglu_bwd_x", "rope_bwd_x", "rms_norm_bwd_x", "rms_norm_bwd_w"]

    DOM = op_names.index(DOMINANT)

    # The submissions of one step, bound once: the C entry points (submit_* of include/dataflow_api.h) with plain
    # integer pointers, so that the per-step host work is the C path (skeleton + SHA-256 + table lookup + launch)
    # and not Python argument marshalling.
    import ctypes as C
    from dataflow_lib_b200 import _lib as _dl
    L, hp = _dl.lib, C.byref(h.h)
    P = {k: v.data_ptr() for k, v in dev.items()}
    N = T * N_HEADS * HEAD_DIM
    calls = [
        lambda: L.submit_rms_norm(hp, S0, BF, T, D_MODEL, EPS, P["w"], P["X"], Y.data_ptr(), ws.data_ptr(), rms.data_ptr()),
        lambda: L.submit_rope(hp, S0, BF, N, N_HEADS * HEAD_DIM, HEAD_DIM, N_KV, THETA, P["pos"], P["Q"], P["K"]),
        lambda: L.submit_swiglu(hp, S0, BF, T, FFN, P["gate"], P["up"], S.data_ptr()),
        lambda: L.submit_swiglu_bwd_x(hp, S0, BF, BF, T, FFN, P["gate"], P["up"], P["dS"], d1.data_ptr(), d3.data_ptr()),
        lambda: L.submit_rope_bwd_x(hp, S0, BF, N, N_HEADS * HEAD_DIM, HEAD_DIM, N_KV, THETA, P["pos"], P["Q"], P["K"]),
        lambda: L.submit_rms_norm_bwd_x(hp, S0, BF, BF, T, D_MODEL, EPS, ws.data_ptr(), rms.data_ptr(), P["w"], P["X"], P["dY"], dX.data_ptr()),
        lambda: L.submit_rms_norm_bwd_w(hp, S0, BF, BF, T, D_MODEL, EPS, rms.data_ptr(), P["X"], P["dY"], dW.data_ptr()),
    ]

    def chain(events=None, only=None):
        """One step. `events[i] = (start, end)` are recorded around op i (all ops, or just op `only`)."""
        for i, call in enumerate(calls):
            timed = events is not None and (only is None or only == i)
            if world > 1 and i == len(calls) - 1 and exchange_state[0] is not None:
                # rms_norm_bwd_w rewrites dW: it has to wait for the previous step's exchange, which ran on stream 1
                assert h.submit_dependency(S0, exchange_state[0]) == 0
            if timed:
                events[i][0].record(stream)
            rc = call()
            if timed:
                events[i][1].record(stream)
            if rc != 0:
                raise RuntimeError(f"submit of {op_names[i]} failed")
        if world > 1:
            # the data-parallel exchange (one packed fp32 all-reduce, 16 KB) runs on the handle's second stream behind a
            # dependency on the compute stream, so that it overlaps the next step's kernels
            assert h.submit_dependency(1, h.get_stream_state(S0)) == 0
            with torch.cuda.stream(stream1):
                allreduce_step(step_loss, [dW])
            exchange_state[0] = h.get_stream_state(1)

    def join_exchange():
        if world > 1 and exchange_state[0] is not None:
            assert h.submit_dependency(S0, exchange_state[0]) == 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    upload()
    h.sync_stream(S0)
    for _ in range(max(args.warmup, 3)):
        chain()
    barrier()

    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None

    # ---- timed region 1: inputs resident in HBM. Only the dominant kernel is bracketed by events here (an event
    # pair costs a few microseconds of stream serialisation, which seven pairs per 0.4 ms step would distort).
    new_events = lambda: [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in op_names]
    ev = [new_events() for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    host_t0 = time.perf_counter()
    t_begin.record(stream)
    for s in range(args.steps):
        chain(ev[s], only=DOM)
    join_exchange()
    t_end.record(stream)
    host_enqueue_ms = 1e3 * (time.perf_counter() - host_t0) / args.steps      # host time to submit one step (no sync)
    barrier()
    ms_total = t_begin.elapsed_time(t_end)
    dom_ms = statistics.mean(ev[s][DOM][0].elapsed_time(ev[s][DOM][1]) for s in range(args.steps))

    # ---- untimed pass: every op bracketed, for the per-op table (event-to-event times include launch latency)
    prof_steps = min(args.steps, 50)
    evp = [new_events() for _ in range(prof_steps)]
    for s in range(prof_steps):
        chain(evp[s])
    barrier()
    per_op_ms = {name: statistics.mean(evp[s][i][0].elapsed_time(evp[s][i][1]) for s in range(prof_steps)) for i, name in enumerate(op_names)}

    # ---- timed region 2: end to end with host buffers through the handle's transfer calls
    e2e_steps = max(3, min(args.steps, 10))
    h2d = sum(a.nbytes for a in host.values())
    d2h = sum(a.nbytes for a in out_host.values())

    def e2e_step():
        upload()
        chain()
        join_exchange()
        assert h.submit_outbound_transfer(S0, out_host["dW"].ctypes.data, dW, out_host["dW"].nbytes) == 0
        assert h.submit_outbound_transfer(S0, out_host["rms"].ctypes.data, rms, out_host["rms"].nbytes) == 0
        assert h.submit_outbound_transfer(S0, out_host["ws"].ctypes.data, ws, out_host["ws"].nbytes) == 0
        h.sync_stream(S0)                                # the host consumes the result every step

    e2e_step()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e_begin.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e_end.record(stream)
    barrier()
    ms_e2e = e_begin.elapsed_time(e_end)

    clocks = sampler.stop() if sampler else None

    times = torch.tensor([ms_total, ms_e2e], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = times.tolist()

    if rank == 0:
        peak, peak_src = measured_peak_hbm()
        dom_bytes = BYTES_PER_TOKEN[DOMINANT] * T
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        ops_report = {name: {"ms": per_op_ms[name], "GB/s": BYTES_PER_TOKEN[name] * T / (per_op_ms[name] * 1e-3) / 1e9,
                             "frac_of_peak": BYTES_PER_TOKEN[name] * T / (per_op_ms[name] * 1e-3) / 1e9 / peak} for name in op_names}
        cpu = cpu_baseline() if world == 1 else None
        others = other_configs(peak) if world == 1 else None
        line = {
            "metric": METRIC, "value": world * T * args.steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": T, "l2": "inputs larger than L2 (1.7 GiB touched per step vs 126 MB)",
                       "parallelism": f"token-sharded x{world}" + (", NCCL all-reduce of the RMSNorm weight gradient" if world > 1 else "")},
            "roofline": {"bound": "hbm", "kernel": DOMINANT, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": DOMINANT_DRAM_TRAFFIC_BYTES, "algorithmic_bytes": dom_bytes, "peak_source": peak_src,
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "note": "traffic is from an ncu capture of the kernel run alone; in the chain it follows swiglu on the same x_w1, x_w3 and "
                                 "walks them from the end, so the ~126 MB that swiglu left in L2 are not re-read from DRAM and frac can pass 1"},
            "ops_event_bracketed": ops_report,
            "e2e": {"value": world * T * e2e_steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": ms_e2e / e2e_steps},
            "gpu_launches": KERNEL_LAUNCHES_PER_STEP * args.steps,
            "host_enqueue_ms_per_step": host_enqueue_ms,
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if others is not None:
            line["other_configs"] = others
        print(json.dumps(line), flush=True)

    for a in list(host.values()) + list(out_host.values()):
        h.disable_access_to_host_mem(a.ctypes.data)
    h.close()
    if world > 1:
        dist.destroy_process_group()


def run_stack_arm(args):
    """--workload stack: the token-sharded 4-layer training step of dataflow_lib_b200/op_stack.py (16384 tokens per GPU,
    d 4096, ffn 14336, 32/8 heads x 128, vocabulary 128256; bf16 activations, FP8 FFN weights, seed-0 random weights identical
    on every rank, data seeded per rank; loss sum and RMSNorm weight gradients all-reduced over NCCL). Not the default
    workload: `value` is tokens/s of the whole step, the library vocabulary GEMMs included and reported separately."""
    import torch
    import torch.distributed as dist

    from dataflow_lib_b200 import ops
    from dataflow_lib_b200.op_stack import OpStackStep

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch N > 1 with torchrun)"
    torch.cuda.set_device(local)
    if world > 1:
        quiet_nccl_banner()
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    T, V, LAYERS = args.tokens or 16384, 128256, 4
    st = OpStackStep(T, D_MODEL, FFN, N_HEADS, N_KV, HEAD_DIM, V, LAYERS, EPS, float(THETA))
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

    warm = max(args.warmup, 3)
    for _ in range(warm):
        st.step()
    barrier()
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None
    ev = lambda: torch.cuda.Event(enable_timing=True)
    t0, t1 = ev(), ev()
    barrier()
    t0.record()
    for _ in range(args.steps):
        st.step(overlap=True)                     # the all-reduce runs beside the next step; the last one is waited for below
    st.wait_exchange()
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    if world > 1:
        # untimed check of the overlapped exchange: the same step reduced on the compute stream gives the same buffer
        from dataflow_lib_b200.sharding import pack_reduction
        st.step(overlap=True); st.wait_exchange()
        overlapped = st.reduced.clone()
        st.step()
        in_stream = pack_reduction(st.loss_sum, st.dW)            # that path stores the reduced dW back in bf16
        exchange_check = "identical" if (torch.equal(overlapped[:2], in_stream[:2]) and
                                         torch.equal(overlapped[2:].bfloat16().float(), in_stream[2:])) else "differs"
        if exchange_check != "identical":
            print("warning: the overlapped exchange and the in-stream one gave different sums", file=sys.stderr)
    else:
        exchange_check = None

    # end to end: the step's tokens and labels come from pinned host memory, the loss goes back, every step
    e_steps = max(3, min(args.steps, 10))
    def e2e_step():
        st.x[0].copy_(host_x, non_blocking=True); st.labels.copy_(host_labels, non_blocking=True)
        st.step()
        host_loss.copy_(st.loss_sum, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_step()
    e0, e1 = ev(), ev()
    barrier()
    e0.record()
    for _ in range(e_steps):
        e2e_step()
    e1.record()
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
    if rank == 0:
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                bf16_sustained, src = float(json.load(f)["bf16_tflops_sustained"]), "2 x bf16_tflops_sustained of MEASURED_PEAKS.json (it holds no fp8 figure)"
        except (OSError, KeyError, ValueError):
            bf16_sustained, src = 1400.0, "2 x the fallback's sustained bf16 figure"
        flops = 2.0 * T * D_MODEL * FFN
        achieved = flops / (ms_gemm * 1e-3) / 1e12
        step_ms = ms_total / args.steps
        line = {
            "metric": "tokens_per_s_op_stack_step", "value": world * T * args.steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 activations, e4m3 FFN operands with fp32 accumulation", "data": "synthetic",
            "config": {"workload": f"4-layer op stack step fwd+bwd (RMSNorm -> RoPE -> FP8 SwiGLU FFN + residual) x4 + head (RMSNorm -> vocabulary GEMM -> "
                                   f"fused softmax+CE), {T} tokens/GPU, d 4096, ffn 14336, vocab 128256",
                       "tokens_per_gpu": T, "l2": "inputs larger than L2 (tens of GB touched per step)",
                       "parallelism": f"token-sharded x{world}" + (", NCCL all-reduce of loss and RMSNorm weight gradients on a side stream, overlapped with the next step" if world > 1 else "")},
            "roofline": {"bound": "tensor", "kernel": "gemm_e4m3_kernel<PLAIN, CTA pair> (the gate projection of the FFN forward, timed alone after the step)", "achieved": achieved,
                         "peak": 2 * bf16_sustained, "unit": "TFLOP/s", "frac": achieved / (2 * bf16_sustained), "traffic": None, "peak_source": src},
            "step_breakdown_ms": breakdown, "exchange_check": exchange_check,
            "e2e": {"value": world * T * e_steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": host_x.numel() * 2 + host_labels.numel() * 4,
                    "d2h_bytes_per_step": 8, "steps": e_steps, "ms_per_step": ms_e2e / e_steps},
            "gpu_launches": st.library_launches_per_step() * args.steps,
            "loss": float(st.loss_sum[0]) / max(float(st.loss_sum[1]), 1.0),
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="chain", choices=["chain", "stack"],
                    help="chain (default): the elementwise op chain the headline metric is quoted on; stack: the 4-layer token-sharded training step")
    ap.add_argument("--tokens", type=int, default=0, help="stack workload only: tokens per GPU (default 16384)")
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
