"""bench.py without a GPU: the CPU arm prints the contract's JSON line, the byte accounting of the chain adds up, and the host-memory
placement helper of the multi-rank arm leaves a machine without a GPU (or with one NUMA node) alone."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "tokens_per_s_op_chain" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"] == _bench_module().chain_config(1)                 # the same object the GPU arm prints


def test_chain_byte_accounting():
    b = _bench_module()
    d, f, e = b.D_MODEL, b.FFN, 2
    qk = (b.N_HEADS + b.N_KV) * b.HEAD_DIM
    per_token = {"rms_norm": 2 * d * e + 8, "rope": 2 * qk * e + 4, "swiglu": 3 * f * e, "swiglu_bwd_x": 5 * f * e, "rope_bwd_x": 2 * qk * e + 4,
                 "rms_norm_bwd_x": 4 * d * e + 8, "rms_norm_bwd_w": 2 * d * e + 4, "rms_norm_bwd_x_w": 4 * d * e + 8}
    assert b.BYTES_PER_TOKEN == per_token
    assert sum(b.BYTES_PER_TOKEN[n] for n in b.CHAIN_OPS) == 319512 and sum(b.BYTES_PER_TOKEN[n] for n in b.CHAIN_OPS_SEPARATE) == 335900
    assert b.CHAIN_OPS[:5] == b.CHAIN_OPS_SEPARATE[:5] and b.DOMINANT in b.CHAIN_OPS


def test_host_memory_placement_leaves_a_box_without_gpu_alone():
    b = _bench_module()
    before = os.sched_getaffinity(0)
    info = b.host_memory_near_gpu(0)
    assert isinstance(info, dict) and info["mempolicy"] == "unchanged" and info["cpu_affinity"] == "unchanged"
    assert os.sched_getaffinity(0) == before
