"""The drop-in shown by a run: the reference's own handle, registry and submit_* wrappers (compiled unchanged into
oracle/_ref/libref_handle.so) with this library's plug-ins registered behind them. The caller side lives in ref_handle_driver.py and runs
in a process of its own (the reference's handle makes a private CUDA context and leaves it current on the thread)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
REF_HANDLE = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libref_handle.so")


def test_plugins_run_under_the_reference_handle():
    assert os.path.exists(REF_HANDLE), "oracle/_ref/libref_handle.so is missing: run `make -C oracle ref` where the reference tree is mounted"
    run = subprocess.run([sys.executable, os.path.join(HERE, "ref_handle_driver.py")], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:] + "\n" + run.stderr[-4000:]
    assert "reference handle ok" in run.stdout
