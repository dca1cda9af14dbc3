"""A plain C program (tests/c_caller/chain.c) written against include/dataflow_api.h the way the reference's own test mains
use its API, compiled with gcc and linked with libdataflow_b200.so only: proves the headers are usable from C, the library
exports what they declare, and (on a GPU) that the handle, transfers, dependencies and ops work without any Python."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_DIR = os.path.join(ROOT, "dataflow_lib_b200", "lib")


@pytest.fixture(scope="module")
def chain_binary(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("c_caller") / "chain")
    cmd = ["gcc", "-O1", "-std=gnu11", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "c_caller", "chain.c"),
           "-o", out, "-L" + LIB_DIR, "-ldataflow_b200", "-lm", "-Wl,-rpath," + LIB_DIR]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_c_caller_links(chain_binary):
    res = subprocess.run([chain_binary, "link"], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0 and "rms_norm_BF16 has 8 arguments" in res.stdout and "matmul has 19 arguments" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_c_caller_runs_the_ops(chain_binary):
    res = subprocess.run([chain_binary], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "all checks passed" in res.stdout, res.stdout + res.stderr
