"""raft::linalg::mapThenSumReduce / map_reduce on the row kernels (a 1 x len matrix): the
reference's test cases (cpp/tests/linalg/map_then_reduce.cu: sum of 1024*1024 uniform(-1, 1) values
at tolerance 1e-3 / 1e-6; min = 1 and max = 5 of 1237 values in [2, 3) with a 1 planted at 42 and a
5 at 337), the lengths of its benchmark (bench/prims/linalg/map_then_reduce.cu:50-60), and the
reference's own kernels on the same device inputs."""
import numpy as np
import pytest
import torch

from raft_b200 import linalg
from util import device_synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref as r
    if not r.available():
        return None
    r.load()
    return r


@pytest.mark.parametrize("n", [1, 7, 1237, 1024 * 1024, 1024 * 1024 + 1, 1024 * 1024 + 2, 32 * 1024 * 1024 + 2])
@pytest.mark.parametrize("dt,out_dt,tol", [(np.float32, torch.float32, 1e-5), (np.float32, torch.float64, 1e-9),
                                           (np.float64, torch.float64, 1e-9)])
def test_sum(cuda, oracle, ref, n, dt, out_dt, tol):
    t, host = device_synth((n,), dt, 1234, "uniform", -1, 1, cuda)
    ours = linalg.map_reduce(t, out_dtype=out_dt)
    exp = oracle.reduce(host.reshape(1, -1))
    # the sum of n values in (-1, 1) is ~sqrt(n): compare on the scale of the terms, as the
    # reference's test does with its absolute 1e-3
    scale = max(1.0, float(np.sqrt(n)))
    assert abs(float(ours[0]) - float(exp[0])) <= tol * scale
    if ref is not None and out_dt == t.dtype and n >= 1237:
        theirs = torch.zeros(1, dtype=t.dtype, device=cuda)
        assert ref.map_then_sum_reduce(theirs, t) == 0
        assert abs(float(theirs[0]) - float(exp[0])) <= 1e-3 * scale      # the reference's own tolerance
        assert abs(float(theirs[0]) - float(ours[0])) <= 1e-3 * scale


@pytest.mark.parametrize("map_op", ["sq", "abs"])
def test_named_maps(cuda, oracle, map_op):
    t, host = device_synth((3_000_001,), np.float32, 7, "uniform", -1, 1, cuda)
    ours = linalg.map_reduce(t, map_op=map_op)
    exp = oracle.reduce(host.reshape(1, -1), main_op=map_op)
    oracle.assert_approx(exp, ours.cpu().numpy(), 1e-5, map_op)


def test_min_max_known_answers(cuda, oracle, ref):
    t, host = device_synth((1237,), np.float32, 137, "uniform", 2, 3, cuda)
    t[42] = 1.0
    t[337] = 5.0
    fmax, fmin = float(np.finfo(np.float32).max), float(np.finfo(np.float32).tiny)
    lo = linalg.map_reduce(t, reduce_op="min", neutral=fmax)
    hi = linalg.map_reduce(t, reduce_op="max", neutral=fmin)
    assert float(lo[0]) == 1.0 and float(hi[0]) == 5.0
    hi64 = linalg.map_reduce(t, reduce_op="max", neutral=fmin, out_dtype=torch.float64)
    assert float(hi64[0]) == 5.0
    if ref is not None:
        o = torch.zeros(1, dtype=torch.float32, device=cuda)
        assert ref.map_reduce_minmax(o, t, "min", fmax) == 0 and float(o[0]) == 1.0
        assert ref.map_reduce_minmax(o, t, "max", fmin) == 0 and float(o[0]) == 5.0


def test_sum_is_reproducible_and_exact_on_integers(cuda):
    """No atomics: the same bits on every run; integer-valued floats below 2^24 sum exactly."""
    t, host = device_synth((10_000_019,), np.float32, 3, "int", 0, 2, cuda)
    a = linalg.map_reduce(t)
    b = linalg.map_reduce(t)
    assert torch.equal(a, b)
    assert float(a[0]) == float(host.astype(np.float64).sum())
    u, _ = device_synth((10_000_019,), np.float32, 4, "uniform", -1, 1, cuda)
    assert torch.equal(linalg.map_reduce(u), linalg.map_reduce(u))
