"""Runs the C++ test program of the drop-in raft::linalg headers (tests/cpp/test_dropin.cu): the
stand-alone build, and - when it was built - the overlay build that puts this repository's
raft/linalg headers in front of the reference's own raft/core headers."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(binary):
    r = subprocess.run([binary], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout[-4000:]
    assert "FAIL" not in r.stdout


def test_dropin_standalone(cuda):
    binary = os.path.join(HERE, "cpp", "test_dropin")
    assert os.path.exists(binary), "build it with `make -C tests/cpp` (done by __graft_entry__.build())"
    _run(binary)


def test_dropin_overlay(cuda):
    binary = os.path.join(HERE, "cpp", "test_dropin_overlay")
    if not os.path.exists(binary):
        pytest.skip("overlay build needs the reference checkout at build time")
    _run(binary)


def test_reference_stats_on_overlay(cuda):
    """The reference's own raft::stats::{sum, mean, stddev, vars, weighted_mean} headers compiled
    on top of this repository's raft/linalg headers (tests/cpp/test_stats_overlay.cu)."""
    binary = os.path.join(HERE, "cpp", "test_stats_overlay")
    if not os.path.exists(binary):
        pytest.skip("overlay build needs the reference checkout at build time")
    _run(binary)


def test_multi_device_layer(cuda):
    """include/raft_b200_mg.h (one host process, NCCL) on every visible device: tests/cpp/test_mg.cu.
    One device exercises the whole call path with a one-rank communicator; two or more add the
    all-reduce across devices and unequal / empty shards."""
    binary = os.path.join(HERE, "cpp", "test_mg")
    assert os.path.exists(binary), "build it with `make -C tests/cpp` (done by __graft_entry__.build())"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([binary], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout[-4000:]


def _run_snmg(name):
    binary = os.path.join(HERE, "cpp", name)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([binary], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "SNMG ALL PASSED" in r.stdout, r.stdout[-4000:]
    assert "FAIL" not in r.stdout


def test_sharded_overloads_standalone(cuda):
    """raft::linalg::reduce / reduce_rows_by_key taking a raft::device_resources_snmg and one view per device
    (include/raft/linalg/sharded_reduce.cuh), stand-alone build, on every visible device: tests/cpp/test_snmg.cu."""
    assert os.path.exists(os.path.join(HERE, "cpp", "test_snmg")), "build it with `make -C tests/cpp`"
    _run_snmg("test_snmg")


def test_sharded_overloads_on_the_reference_core(cuda):
    """The same program compiled against the reference's own raft/core: resources.hpp, the MULTI_GPU and
    NCCL_COMM resources (core/resource/multi_gpu.hpp, nccl_comm.hpp)."""
    if not os.path.exists(os.path.join(HERE, "cpp", "test_snmg_overlay")):
        pytest.skip("overlay build needs the reference checkout at build time")
    _run_snmg("test_snmg_overlay")
