"""Host-side invariants of the launch planners (tests/cpp/test_plans.cu): compiled with nvcc and run on the CPU -
no kernel is launched, so no GPU is needed."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_launch_planners():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    src = os.path.join(HERE, "cpp", "test_plans.cu")
    binary = os.path.join(HERE, "cpp", "test_plans")
    headers = [os.path.join(ROOT, "include", "raft_b200", "detail", f)
               for f in os.listdir(os.path.join(ROOT, "include", "raft_b200", "detail"))]
    newest = max(os.path.getmtime(p) for p in headers + [src])
    if not os.path.exists(binary) or os.path.getmtime(binary) < newest:
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "--expt-relaxed-constexpr",
                        "--expt-extended-lambda", "-I" + os.path.join(ROOT, "include"), src, "-o", binary],
                       check=True, timeout=600)
    r = subprocess.run([binary], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout[-4000:]
