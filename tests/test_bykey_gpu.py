"""Parity of b2r_reduce_rows_by_key / b2r_reduce_cols_by_key with the fp64 oracle over the
reference's test shapes (cpp/tests/linalg/reduce_rows_by_key.cu:164-263,
cpp/tests/linalg/reduce_cols_by_key.cu:107-126)."""
import numpy as np
import pytest
import torch

from raft_b200 import linalg
from util import device_synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nobs,cols,nkeys,dt,tol", [
    (128, 32, 6, np.float32, 1e-6),
    (128, 32, 3, np.float32, 1e-6),
    (512, 1024, 40, np.float64, 1e-9),
    (100000, 37, 32, np.float32, 1e-5),
    (100000, 37, 2048, np.float32, 1e-5),
    (20000, 128, 1024, np.float32, 1e-5),
    (5000, 4, 7, np.float32, 1e-5),
    (3000, 130, 300, np.float64, 1e-9),
    (300000, 64, 1024, np.float32, 1e-5),    # several groups of several windows, ragged last group
    (300000, 16, 16384, np.float32, 1e-5),   # one group of 19 windows, about 18 rows per key
    (70000, 32, 24576, np.float32, 1e-5),    # most keys the sorted path takes
    (70000, 32, 30000, np.float32, 1e-5),    # beyond it: shared-memory table slices
    (40000, 2048, 16, np.float32, 1e-5),     # few long rows: the columns of a work unit are split over warps
    (40000, 2052, 300, np.float32, 1e-5),    # ... with a ragged last part
    (33000, 1030, 7, np.float64, 1e-9),
])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("key_dt", [np.int32, np.int64])
def test_rows_by_key_grid(cuda, oracle, nobs, cols, nkeys, dt, tol, weighted, key_dt):
    A, hA = device_synth((nobs, cols), dt, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((nobs,), key_dt, 4321, "int", 0, nkeys, cuda)
    w, hw = device_synth((nobs,), dt, 77, "uniform", 0, 2, cuda) if weighted else (None, None)
    counts = torch.empty(nkeys, dtype=torch.int64, device=cuda)
    sums = linalg.reduce_rows_by_key(A, keys, nkeys, d_weights=w, counts=counts)
    esum, ecnt = oracle.rows_by_key(hA, hk, nkeys, weights=hw)
    oracle.assert_approx(esum, sums.cpu().numpy(), tol, "reset")
    assert np.array_equal(counts.cpu().numpy(), ecnt)  # counts are exact
    # accumulate a second time without reset (reset_sums=false of the reference)
    linalg.reduce_rows_by_key(A, keys, nkeys, d_sums=sums, d_weights=w, reset_sums=False, counts=counts)
    oracle.assert_approx(2 * esum, sums.cpu().numpy(), 2 * tol, "accumulate")
    assert np.array_equal(counts.cpu().numpy(), 2 * ecnt)


def test_rows_by_key_lda_and_workspace(cuda, oracle):
    nobs, cols, lda, nkeys = 70001, 48, 64, 200  # above the one-launch kernel's row limit: scratch is needed
    full, hfull = device_synth((nobs, lda), np.float32, 9, "normal", 0, 1, cuda)
    keys, hk = device_synth((nobs,), np.int32, 10, "int", 0, nkeys, cuda)
    A = full[:, :cols]  # row stride 64, 48 used columns
    sums = linalg.reduce_rows_by_key(A, keys, nkeys)
    esum, _ = oracle.rows_by_key(np.ascontiguousarray(hfull[:, :cols]), hk, nkeys)
    oracle.assert_approx(esum, sums.cpu().numpy(), 1e-5)
    need = linalg.reduce_rows_by_key_workspace_bytes(A, nkeys, lda=lda)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    sums2 = linalg.reduce_rows_by_key(A, keys, nkeys, workspace=ws)
    oracle.assert_approx(esum, sums2.cpu().numpy(), 1e-5)


def test_rows_by_key_skewed_and_missing_keys(cuda, oracle):
    nobs, cols, nkeys = 50000, 64, 500
    A, hA = device_synth((nobs, cols), np.float32, 21, "normal", 0, 1, cuda)
    hk = np.zeros(nobs, dtype=np.int32)
    hk[::7] = 499
    hk[1::1000] = 250  # most keys never occur, one key dominates
    keys = torch.from_numpy(hk).to(cuda)
    counts = torch.empty(nkeys, dtype=torch.int64, device=cuda)
    sums = linalg.reduce_rows_by_key(A, keys, nkeys, counts=counts)
    esum, ecnt = oracle.rows_by_key(hA, hk, nkeys)
    oracle.assert_approx(esum, sums.cpu().numpy(), 1e-5)
    assert np.array_equal(counts.cpu().numpy(), ecnt)


@pytest.mark.parametrize("nobs,cols,nkeys,dt,tol", [(128, 32, 6, np.float32, 1e-6), (512, 1024, 40, np.float64, 1e-9),
                                                    (20000, 128, 1024, np.float32, 1e-5), (5000, 4, 7, np.float32, 1e-5),
                                                    (3000, 130, 300, np.float64, 1e-9), (32768, 64, 3, np.float32, 1e-5)])
@pytest.mark.parametrize("weighted", [False, True])
def test_rows_by_key_sorted_pipeline_on_small_inputs(cuda, oracle, knobs, nobs, cols, nkeys, dt, tol, weighted):
    """Inputs of up to 32768 rows take the one-launch kernel by default; the five-kernel sorted pipeline must give
    the same answers on them."""
    knobs(B2R_KEY_ALGO="2")
    A, hA = device_synth((nobs, cols), dt, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((nobs,), np.int32, 4321, "int", 0, nkeys, cuda)
    w, hw = device_synth((nobs,), dt, 77, "uniform", 0, 2, cuda) if weighted else (None, None)
    counts = torch.empty(nkeys, dtype=torch.int64, device=cuda)
    sums = linalg.reduce_rows_by_key(A, keys, nkeys, d_weights=w, counts=counts)
    esum, ecnt = oracle.rows_by_key(hA, hk, nkeys, weights=hw)
    oracle.assert_approx(esum, sums.cpu().numpy(), tol, "sorted pipeline")
    assert np.array_equal(counts.cpu().numpy(), ecnt)


@pytest.mark.parametrize("nobs,cols,nkeys", [(10000, 128, 64), (10000, 128, 4096), (32768, 128, 1), (32768, 36, 70000),
                                             (1, 5, 3), (9999, 1000, 17), (200, 8, 200)])
def test_rows_by_key_one_launch_kernel(cuda, oracle, knobs, nobs, cols, nkeys):
    """Shapes aimed at the one-launch kernel (forced: by default it only takes inputs of about a megabyte per
    CTA): the reference's smallest bench shapes (bench/prims/linalg/reduce_rows_by_key.cu:55-72), one key for all
    rows, far more keys than rows, one row, rows of several column passes."""
    knobs(B2R_KEY_ALGO="3")
    A, hA = device_synth((nobs, cols), np.float32, 12, "uniform", -1, 1, cuda)
    keys, hk = device_synth((nobs,), np.int32, 13, "int", 0, nkeys, cuda)
    counts = torch.empty(nkeys, dtype=torch.int64, device=cuda)
    sums = linalg.reduce_rows_by_key(A, keys, nkeys, counts=counts)
    assert linalg.reduce_rows_by_key_workspace_bytes(A, nkeys) == 0
    esum, ecnt = oracle.rows_by_key(hA, hk, nkeys)
    oracle.assert_approx(esum, sums.cpu().numpy(), 1e-5, "one launch")
    assert np.array_equal(counts.cpu().numpy(), ecnt)
    linalg.reduce_rows_by_key(A, keys, nkeys, d_sums=sums, reset_sums=False, counts=counts)
    oracle.assert_approx(2 * esum, sums.cpu().numpy(), 2e-5, "accumulate")
    assert np.array_equal(counts.cpu().numpy(), 2 * ecnt)


@pytest.mark.parametrize("nobs,cols,nkeys", [(128, 32, 6), (100000, 37, 2048), (60000, 128, 1024), (512, 1024, 40)])
def test_rows_by_key_table_algorithm(cuda, oracle, knobs, nobs, cols, nkeys):
    # the shared-memory-table kernel is the fallback for more keys than the sort kernel's
    # histogram holds; B2R_KEY_ALGO=1 forces it for ordinary sizes
    knobs(B2R_KEY_ALGO="1")
    A, hA = device_synth((nobs, cols), np.float32, 31, "uniform", -1, 1, cuda)
    keys, hk = device_synth((nobs,), np.int32, 32, "int", 0, nkeys, cuda)
    w, hw = device_synth((nobs,), np.float32, 33, "uniform", 0, 2, cuda)
    counts = torch.empty(nkeys, dtype=torch.int64, device=cuda)
    sums = linalg.reduce_rows_by_key(A, keys, nkeys, d_weights=w, counts=counts)
    esum, ecnt = oracle.rows_by_key(hA, hk, nkeys, weights=hw)
    oracle.assert_approx(esum, sums.cpu().numpy(), 1e-5)
    assert np.array_equal(counts.cpu().numpy(), ecnt)


def test_rows_by_key_many_keys(cuda, oracle):
    # more keys than the sort kernel's shared-memory histogram holds -> table algorithm
    nobs, cols, nkeys = 200000, 16, 60000
    A, hA = device_synth((nobs, cols), np.float32, 41, "uniform", -1, 1, cuda)
    keys, hk = device_synth((nobs,), np.int32, 42, "int", 0, nkeys, cuda)
    sums = linalg.reduce_rows_by_key(A, keys, nkeys)
    esum, _ = oracle.rows_by_key(hA, hk, nkeys)
    oracle.assert_approx(esum, sums.cpu().numpy(), 1e-5)


def test_rows_by_key_empty(cuda):
    A = torch.empty((0, 16), dtype=torch.float32, device=cuda)
    keys = torch.empty((0,), dtype=torch.int32, device=cuda)
    sums = torch.full((5, 16), 3.0, device=cuda)
    linalg.reduce_rows_by_key(A, keys, 5, d_sums=sums, reset_sums=False)
    assert torch.all(sums == 3.0)
    linalg.reduce_rows_by_key(A, keys, 5, d_sums=sums, reset_sums=True)
    assert torch.all(sums == 0.0)


# cpp/tests/linalg/reduce_cols_by_key.cu:107-126 (a representative subset of the 60-case grid,
# every extreme included)
@pytest.mark.parametrize("rows,cols,nkeys", [(1, 1234, 7), (1, 101010, 2022), (9, 9999, 42), (63, 1234, 515),
                                             (63, 101010, 127), (1024, 1234, 7), (1024, 9999, 2022),
                                             (1024, 1234, 127), (9, 101010, 7), (3000, 300, 60000)])
@pytest.mark.parametrize("dt,tol", [(np.float32, 1e-3), (np.float64, 1e-6)])
def test_cols_by_key_grid(cuda, oracle, rows, cols, nkeys, dt, tol):
    data, hd = device_synth((rows, cols), dt, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((cols,), np.int32, 55, "int", 0, nkeys, cuda)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys)
    exp = oracle.cols_by_key(hd, hk, nkeys)
    oracle.assert_approx(exp, out.cpu().numpy(), tol, "reset")
    linalg.reduce_cols_by_key(data, keys, out=out, reset_sums=False)
    oracle.assert_approx(2 * exp, out.cpu().numpy(), 2 * tol, "accumulate")


# the sorted-column-tiles kernels on every shape of the grid above (forced: the small ones would
# take the single-kernel path), on shapes that exercise every tile geometry (RT 1..8, CH 256..4096,
# columns split over CTAs or not, ragged last chunk and last row tile, scalar and 16-byte staging),
# and the largest key count they take
@pytest.mark.parametrize("rows,cols,nkeys", [(1, 1234, 7), (1, 101010, 2022), (9, 9999, 42), (63, 1234, 515),
                                             (63, 101010, 127), (1024, 1234, 7), (1024, 9999, 2022),
                                             (1024, 1234, 127), (9, 101010, 7), (2, 300, 8192), (5, 70000, 8192),
                                             (4000, 4096, 64), (4001, 4100, 3), (300, 50001, 1), (20000, 256, 5),
                                             (7, 8, 4), (100, 100000, 4096), (1000, 10000, 512)])
@pytest.mark.parametrize("dt,tol", [(np.float32, 1e-5), (np.float64, 1e-9)])
@pytest.mark.parametrize("key_dt", [np.int32, np.int64])
@pytest.mark.parametrize("staging", ["tma", "registers"])
def test_cols_by_key_sorted_tiles(cuda, oracle, knobs, rows, cols, nkeys, dt, tol, key_dt, staging):
    knobs(B2R_COLKEY_ALGO="2")
    knobs(B2R_COLKEY_TMA="1" if staging == "tma" else "2")
    data, hd = device_synth((rows, cols), dt, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((cols,), key_dt, 55, "int", 0, nkeys, cuda)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys)
    exp = oracle.cols_by_key(hd, hk, nkeys)
    oracle.assert_approx(exp, out.cpu().numpy(), tol, "reset")
    linalg.reduce_cols_by_key(data, keys, out=out, reset_sums=False)
    oracle.assert_approx(2 * exp, out.cpu().numpy(), 2 * tol, "accumulate")
    # no floating-point atomics: a repeat gives the same bits (fp64 segment sums of fp32 data)
    if dt == np.float32:
        again = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys)
        assert torch.equal(again, linalg.reduce_cols_by_key(data, keys, nkeys=nkeys))


# the walk form of the sorted tiles (a warp walks the sorted columns of its keys; up to 256 keys), forced, on every
# tile shape it has (8 / 16 / 32 rows), with ragged last chunks and row tiles, columns split over CTAs or not,
# fewer keys than warps (slices), a caller's workspace, and a key that owns no column
@pytest.mark.parametrize("rows,cols,nkeys", [(1, 1236, 7), (9, 10000, 42), (63, 101012, 127), (1024, 1236, 7),
                                             (1024, 9996, 256), (4001, 4100, 3), (300, 50004, 1), (20000, 256, 5),
                                             (7, 8, 4), (2000, 30000, 16), (2000, 30000, 64), (33, 70000, 200)])
@pytest.mark.parametrize("dt,tol", [(np.float32, 1e-5), (np.float64, 1e-9)])
@pytest.mark.parametrize("rt", [8, 16, 32])
def test_cols_by_key_walk_form(cuda, oracle, knobs, rows, cols, nkeys, dt, tol, rt):
    knobs(B2R_COLKEY_ALGO="3", B2R_COLKEY32_RT=str(rt))
    data, hd = device_synth((rows, cols), dt, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((cols,), np.int32, 55, "int", 0, max(1, nkeys - 1), cuda)  # the last key stays empty
    ws = torch.empty(max(1, linalg.reduce_cols_by_key_workspace_bytes(data, nkeys)), dtype=torch.uint8, device=cuda)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys, workspace=ws)
    exp = oracle.cols_by_key(hd, hk, nkeys)
    oracle.assert_approx(exp, out.cpu().numpy(), tol, "reset")
    linalg.reduce_cols_by_key(data, keys, out=out, reset_sums=False)
    oracle.assert_approx(2 * exp, out.cpu().numpy(), 2 * tol, "accumulate")
    # no floating-point atomics: a repeat gives the same bits (fp64 partial sums of fp32 data)
    if dt == np.float32:
        again = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys)
        assert torch.equal(again, linalg.reduce_cols_by_key(data, keys, nkeys=nkeys))
    assert linalg.last_kernel_status(cuda) == 0


# the table form (no sort: a shared-memory cell per key, row and warp; fp32, up to 255 keys), forced, with ragged last
# boxes and row tiles, columns split over CTAs or not, 8 and 4 consumer warps, a caller's workspace, a key that owns
# no column, int64 keys, and accumulation into existing sums
@pytest.mark.parametrize("rows,cols,nkeys", [(1, 1236, 7), (9, 10000, 42), (63, 101012, 127), (1024, 1236, 70),
                                             (1024, 9996, 255), (4001, 4100, 129), (300, 5004, 1), (20000, 256, 128),
                                             (7, 228, 4), (2000, 30000, 128), (33, 700000, 200), (257, 228 * 40, 65)])
@pytest.mark.parametrize("key_dt", [np.int32, np.int64])
def test_cols_by_key_table_form(cuda, oracle, knobs, rows, cols, nkeys, key_dt):
    knobs(B2R_COLKEY_ALGO="4")
    data, hd = device_synth((rows, cols), np.float32, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((cols,), key_dt, 55, "int", 0, max(1, nkeys - 1), cuda)  # the last key stays empty
    ws = torch.empty(max(1, linalg.reduce_cols_by_key_workspace_bytes(data, nkeys)), dtype=torch.uint8, device=cuda)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys, workspace=ws)
    exp = oracle.cols_by_key(hd, hk, nkeys)
    # the cells are fp32: with a handful of keys (forced here; by itself the library takes this form from 65 keys
    # on) one output is the sum of tens of thousands of fp32 additions and gets the looser bound
    tol = 1e-5 if nkeys >= 16 else 3e-5
    oracle.assert_approx(exp, out.cpu().numpy(), tol, "reset")
    linalg.reduce_cols_by_key(data, keys, out=out, reset_sums=False)
    oracle.assert_approx(2 * exp, out.cpu().numpy(), 2 * tol, "accumulate")
    again = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys)
    assert torch.equal(again, linalg.reduce_cols_by_key(data, keys, nkeys=nkeys))  # fixed order of all additions
    assert linalg.last_kernel_status(cuda) == 0


def test_cols_by_key_table_form_by_itself_and_against_the_other_forms(cuda, oracle, knobs):
    data, hd = device_synth((1000, 60000), np.float32, 8, "normal", 0, 1, cuda)
    keys, hk = device_synth((60000,), np.int32, 9, "int", 0, 100, cuda)
    exp = oracle.cols_by_key(hd, hk, 100)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=100)  # 100 keys, 240 MB: the table form by the library's choice
    oracle.assert_approx(exp, out.cpu().numpy(), 1e-5, "auto")
    knobs(B2R_COLKEY_ALGO="2")
    seg = linalg.reduce_cols_by_key(data, keys, nkeys=100)
    oracle.assert_approx(seg.cpu().numpy().astype(np.float64), out.cpu().numpy(), 1e-5, "against a lane per segment")


def test_cols_by_key_single_kernel_path(cuda, oracle, knobs):
    knobs(B2R_COLKEY_ALGO="1")
    data, hd = device_synth((2000, 3000), np.float32, 3, "uniform", -1, 1, cuda)
    keys, hk = device_synth((3000,), np.int32, 4, "int", 0, 77, cuda)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=77)
    oracle.assert_approx(oracle.cols_by_key(hd, hk, 77), out.cpu().numpy(), 1e-3, "shared-memory atomics")


def test_cols_by_key_unaligned_view(cuda, oracle):
    """A matrix whose base pointer is only 4-byte aligned takes the scalar staging path."""
    buf, _ = device_synth((1500 * 1000 + 1,), np.float32, 9, "uniform", -1, 1, cuda)
    data = buf[1:].view(1500, 1000)
    keys, hk = device_synth((1000,), np.int32, 4, "int", 0, 33, cuda)
    out = linalg.reduce_cols_by_key(data, keys, nkeys=33)
    oracle.assert_approx(oracle.cols_by_key(data.cpu().numpy(), hk, 33), out.cpu().numpy(), 1e-5, "unaligned")


def test_cols_by_key_shape_errors(cuda):
    data = torch.ones((4, 6), device=cuda)
    keys = torch.zeros(6, dtype=torch.int32, device=cuda)
    with pytest.raises(ValueError):
        linalg.reduce_cols_by_key(data, keys, out=torch.zeros((3, 2), device=cuda))
    with pytest.raises(ValueError):
        linalg.reduce_cols_by_key(data, keys[:5], nkeys=2)
    with pytest.raises(ValueError):
        linalg.reduce_cols_by_key(data, keys, out=torch.zeros((4, 2), device=cuda), nkeys=3)
