"""Parity of b2r_row_normalize with the oracle and with the reference's own kernel over the
reference's test grid (cpp/tests/linalg/normalize.cu:117-140: rows {11, 101, 12345} x cols
{2, 3, 7, 12, 33, 125, 254} x {L1, L2, Linf}, uniform(-10, 10), tolerance 1e-5 fp32 / 1e-8 fp64),
wider rows for every kernel policy, and the rows the reference leaves untouched."""
import numpy as np
import pytest
import torch

from raft_b200 import linalg
from util import device_synth

pytestmark = pytest.mark.gpu

NORMS = ["L1", "L2", "Linf"]


@pytest.fixture(scope="module")
def ref():
    from oracle import ref as r
    if not r.available():
        return None
    r.load()
    return r


@pytest.mark.parametrize("rows", [11, 101, 12345])
@pytest.mark.parametrize("cols", [2, 3, 7, 12, 33, 125, 254])
@pytest.mark.parametrize("norm", NORMS)
@pytest.mark.parametrize("dt,tol", [(np.float32, 1e-5), (np.float64, 1e-8)])
def test_reference_grid(cuda, oracle, ref, rows, cols, norm, dt, tol):
    t, host = device_synth((rows, cols), dt, 1234, "uniform", -10, 10, cuda)
    ours = linalg.row_normalize(t, norm)
    exp = oracle.row_normalize(host, norm)
    oracle.assert_approx(exp, ours.cpu().numpy(), tol, "ours vs oracle")
    if ref is not None:
        theirs = torch.zeros_like(t)
        assert ref.row_normalize(theirs, t, norm) == 0
        oracle.assert_approx(exp, theirs.cpu().numpy(), tol, "reference vs oracle")  # pins the oracle
        oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), tol, "ours vs reference")


# every policy: sub-warp sizes 1..32 with 1/2/4/8 vectors per lane, unaligned scalar rows, CTA per row
@pytest.mark.parametrize("rows,cols", [(5000, 4), (5000, 8), (5000, 16), (5000, 32), (5000, 64), (3000, 128),
                                       (3000, 256), (2000, 512), (2000, 516), (1000, 1024), (1000, 1023), (700, 1028),
                                       (300, 2048), (100, 4100), (37, 16384), (5, 100001)])
@pytest.mark.parametrize("norm", NORMS)
@pytest.mark.parametrize("dt,tol", [(np.float32, 1e-5), (np.float64, 1e-8)])
def test_policies(cuda, oracle, ref, rows, cols, norm, dt, tol):
    t, host = device_synth((rows, cols), dt, 99, "uniform", -10, 10, cuda)
    ours = linalg.row_normalize(t, norm)
    exp = oracle.row_normalize(host, norm)
    oracle.assert_approx(exp, ours.cpu().numpy(), tol, "ours vs oracle")
    if ref is not None and dt == np.float32:
        theirs = torch.zeros_like(t)
        assert ref.row_normalize(theirs, t, norm) == 0
        oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), tol, "ours vs reference")


@pytest.mark.parametrize("cols", [8, 100, 128, 1024, 5000])
@pytest.mark.parametrize("norm", NORMS)
def test_rows_below_eps_are_not_written(cuda, oracle, cols, norm):
    rows = 257
    t, host = device_synth((rows, cols), np.float32, 5, "uniform", -1, 1, cuda)
    t[::3] = 0.0            # zero rows: norm 0 <= eps
    t[1::7] *= 1e-12        # tiny rows: norm below the default eps of 1e-8
    host = t.cpu().numpy()
    out = torch.full_like(t, 7.0)
    linalg.row_normalize(t, norm, out=out)
    exp = oracle.row_normalize(host, norm, prev=np.full_like(host, 7.0))
    oracle.assert_approx(exp, out.cpu().numpy(), 1e-5, "sentinel rows")
    assert torch.all(out[::3] == 7.0)
    # a larger eps skips more rows
    out2 = torch.full_like(t, -1.0)
    linalg.row_normalize(t, norm, out=out2, eps=1e3)
    exp2 = oracle.row_normalize(host, norm, eps=1e3, prev=np.full_like(host, -1.0))
    oracle.assert_approx(exp2, out2.cpu().numpy(), 1e-5, "eps 1e3")


@pytest.mark.parametrize("cols", [16, 128, 3000])
def test_in_place(cuda, oracle, cols):
    t, host = device_synth((999, cols), np.float32, 8, "uniform", -10, 10, cuda)
    linalg.row_normalize(t, "L2", out=t)
    oracle.assert_approx(oracle.row_normalize(host, "L2"), t.cpu().numpy(), 1e-5, "in place")


def test_unit_norm_property_full_size(cuda):
    """100 000 x 1024 (the largest register-resident row of the reference's bench grid): every row of
    the result has L2 norm 1 and the direction of the input."""
    t = torch.empty((100000, 1024), dtype=torch.float32, device=cuda)
    linalg.synth_fill(t, 3, "uniform", -10, 10)
    out = linalg.row_normalize(t, "L2")
    n = linalg.norm(out, "L2", fin_op="sqrt")
    assert torch.allclose(n, torch.ones_like(n), atol=2e-6)
    scale = linalg.norm(t, "L2", fin_op="sqrt")
    assert torch.allclose(out[::997] * scale[::997, None], t[::997], rtol=1e-5, atol=1e-5)


def test_argument_checks(cuda):
    t = torch.zeros((4, 8), dtype=torch.float32, device=cuda)
    with pytest.raises(ValueError):
        linalg.row_normalize(t, "L2", out=torch.zeros((5, 8), dtype=torch.float32, device=cuda))
    with pytest.raises(ValueError):
        linalg.row_normalize(t, "L2", out=torch.zeros((4, 9), dtype=torch.float32, device=cuda))
    with pytest.raises(ValueError):
        linalg.row_normalize(t, "L0")
    with pytest.raises(ValueError):
        linalg.row_normalize(t.t(), "L2")


@pytest.mark.parametrize("rows,cols,dt,tol", [(100003, 1, np.float32, 1e-5), (70001, 2, np.float32, 1e-5),
                                              (50002, 3, np.float32, 1e-5), (33333, 7, np.float32, 1e-5),
                                              (20001, 17, np.float32, 1e-5), (9999, 33, np.float32, 1e-5),
                                              (12346, 65, np.float32, 1e-5), (5003, 129, np.float32, 1e-5),
                                              (3001, 513, np.float32, 1e-5), (2002, 1001, np.float32, 1e-5),
                                              (20001, 7, np.float64, 1e-8), (5001, 131, np.float64, 1e-8),
                                              # rows on 16-byte boundaries
                                              (30001, 8, np.float32, 1e-5), (20001, 36, np.float32, 1e-5),
                                              (10001, 96, np.float32, 1e-5), (7001, 100, np.float32, 1e-5),
                                              (3001, 400, np.float32, 1e-5), (2001, 784, np.float32, 1e-5),
                                              (5001, 50, np.float64, 1e-8)])
@pytest.mark.parametrize("norm", NORMS)
@pytest.mark.parametrize("tile_kb", [None, "6"])
def test_staged(cuda, oracle, ref, knobs, rows, cols, dt, tol, norm, tile_kb):
    """The shared-memory staged kernel (block copies in both directions), forced onto small inputs: rows off
    and on 16-byte boundaries, 1..32 lanes per row, rows behind the last boundary, default and tiny tiles;
    rows at or below eps stay untouched (tiles with such rows are stored row by row), in place as well."""
    knobs(B2R_ROW_STAGED_MIN_KB="1", B2R_ROW_STAGED_WIDE_MIN_KB="1", B2R_ROW_STAGED_ALIGNED="2",
          B2R_ROW_STAGED_KB=tile_kb)
    t, host = device_synth((rows, cols), dt, 77, "uniform", -10, 10, cuda)
    ours = linalg.row_normalize(t, norm)
    exp = oracle.row_normalize(host, norm)
    oracle.assert_approx(exp, ours.cpu().numpy(), tol, "staged vs oracle")
    knobs(B2R_ROW_STAGED="2")
    direct = linalg.row_normalize(t, norm)
    oracle.assert_approx(direct.cpu().numpy(), ours.cpu().numpy(), tol * 0.1, "staged vs direct")
    knobs(B2R_ROW_STAGED=None)
    # rows that must not be written: scattered zero rows and one whole stretch of them
    t[::97] = 0.0
    t[rows // 2: rows // 2 + 700] = 0.0
    host = t.cpu().numpy()
    out = torch.full_like(t, 7.0)
    linalg.row_normalize(t, norm, out=out)
    exp = oracle.row_normalize(host, norm, prev=np.full_like(host, 7.0))
    oracle.assert_approx(exp, out.cpu().numpy(), tol, "sentinel rows")
    assert torch.all(out[::97] == 7.0)
    # in place
    keep = t.clone()
    linalg.row_normalize(t, norm, out=t)
    exp = oracle.row_normalize(host, norm, prev=host.copy())
    oracle.assert_approx(exp, t.cpu().numpy(), tol, "in place")
    assert torch.equal(t[::97], keep[::97])


def test_staged_full_size(cuda, oracle):
    """12 000 002 x 23 fp32 (1.1 GB, default policy, two rows behind the last boundary), L2: unit rows."""
    t, _ = device_synth((12000002, 23), np.float32, 78, "uniform", -10, 10, cuda)
    out = linalg.row_normalize(t, "L2")
    n = torch.linalg.vector_norm(out.double(), dim=1)
    assert float((n - 1.0).abs().max()) < 1e-5
    norms = torch.linalg.vector_norm(t.double(), dim=1)
    for c in (0, 11, 22):
        assert float((out[:, c].double() * norms - t[:, c].double()).abs().max()) < 1e-4
