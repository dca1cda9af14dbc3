"""The entry point for callers that cannot allocate: dfb200_rms_norm_bwd_w_static keeps its partial sums in an array
built into the library instead of a caller workspace (think of a host program whose own arena already owns the whole
device, or a step loop that must not run into cudaMalloc's device-wide synchronisation). Called here through the
C-ABI, twice in a row with different shapes so that the second call sees the first call's leftovers in the shared
array, and compared with the regular entry point, which runs the same kernels on a caller-provided workspace.

This file is collected last on purpose: it must pass on its own in a fresh process and after every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from util import check_lowp, f32, to_dev, to_host

pytestmark = pytest.mark.gpu

BF = O.BF16


def _run_both(lib, n_rows, n_cols, seed):
    X, dY = O.fill_normal(BF, (n_rows, n_cols), seed), O.fill_normal(BF, (n_rows, n_cols), seed + 1)
    rms = (1.0 / np.sqrt((f32(X, BF).astype(np.float64) ** 2).mean(1) + 1e-5)).astype(np.float32)
    dW0 = O.fill_normal(BF, (n_cols,), seed + 2)
    Xd, dYd, rmsd = to_dev(X, BF), to_dev(dY, BF), torch.from_numpy(rms).cuda()
    stream = torch.cuda.current_stream().cuda_stream

    dW_static = to_dev(dW0, BF)
    rc = lib.dfb200_rms_norm_bwd_w_static(5, 5, n_rows, n_cols, 1e-5, rmsd.data_ptr(), Xd.data_ptr(), dYd.data_ptr(), dW_static.data_ptr(), stream)
    assert rc == 0, lib.dfb200_last_error().decode()

    need = lib.dfb200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    dW_regular = to_dev(dW0, BF)
    rc = lib.dfb200_rms_norm_bwd_w(5, 5, n_rows, n_cols, 1e-5, rmsd.data_ptr(), Xd.data_ptr(), dYd.data_ptr(), dW_regular.data_ptr(),
                                   ws.data_ptr(), need, stream)
    assert rc == 0, lib.dfb200_last_error().decode()
    torch.cuda.synchronize()
    oracle = O.rms_norm_bwd_w(BF, BF, rms, X, dY, dW0)
    return to_host(dW_static, BF), to_host(dW_regular, BF), oracle


def test_static_scratch_variant_matches_regular_entry_point():
    from dataflow_lib_b200 import _lib
    lib = _lib.lib
    # two calls in a row; the second is smaller, so most of the array still holds the first call's partial sums
    for n_rows, n_cols, seed in ((1000, 4096, 31), (300, 1024, 47)):
        got, regular, oracle = _run_both(lib, n_rows, n_cols, seed)
        assert np.array_equal(got, regular), f"{n_rows}x{n_cols}: built-in scratch and caller workspace must give the same bits"
        check_lowp(got, oracle, BF, f"rms_norm_bwd_w_static {n_rows}x{n_cols} vs oracle", rel=1e-2, scale=float(np.sqrt(n_rows)))
    # the same first shape again: stale contents of the larger run before it must not leak into the result
    got, regular, _ = _run_both(lib, 1000, 4096, 31)
    assert np.array_equal(got, regular)


def test_static_scratch_variant_rejects_shapes_beyond_its_array():
    from dataflow_lib_b200 import _lib
    lib = _lib.lib
    n_rows, n_cols = 64, 16384                       # 148 SMs x 16384 columns x 4 B = 9.7 MB > the 5 MiB array
    x = torch.zeros(n_rows, n_cols, dtype=torch.bfloat16, device="cuda")
    dW = torch.full((n_cols,), 3.0, dtype=torch.bfloat16, device="cuda")
    rms = torch.ones(n_rows, device="cuda")
    rc = lib.dfb200_rms_norm_bwd_w_static(5, 5, n_rows, n_cols, 1e-5, rms.data_ptr(), x.data_ptr(), x.data_ptr(), dW.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == -4, rc                              # DFB200_ERR_WORKSPACE
    msg = lib.dfb200_last_error().decode()
    assert "built-in array" in msg and "16384" in msg, msg
    torch.cuda.synchronize()
    assert torch.all(dW == 3.0), "a rejected call must not touch the output"
