"""The product and the CPU oracle against the REFERENCE's own kernels (oracle/_ref, built from
the reference headers for sm_100a) on identical device inputs. Skipped when that library was
not built (no reference checkout at build time)."""
import numpy as np
import pytest
import torch

from raft_b200 import _lib as L
from raft_b200 import linalg
from util import as_layout, device_synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref as r
    if not r.available():
        pytest.skip("oracle/_ref/libraft_ref.so not built")
    r.load()
    return r


CASES = [("identity", "add", "identity"), ("sq", "add", "identity"), ("sq", "add", "sqrt"), ("abs", "add", "identity"),
         ("abs", "max", "identity"), ("identity", "max", "identity")]
ENUM = {"identity": 0, "sq": 1, "abs": 2, "add": 0, "max": 2, "sqrt": 1}


@pytest.mark.parametrize("main,red,fin", CASES)
@pytest.mark.parametrize("rows,cols", [(11, 7), (1234, 33), (1234, 128), (1000, 500), (4096, 1024), (9, 33333)])
@pytest.mark.parametrize("layout", [0, 1])
def test_contiguous_against_reference(cuda, oracle, ref, main, red, fin, rows, cols, layout):
    t, host = device_synth((rows, cols), np.float32, 1234, "uniform", -1, 1, cuda)
    d = as_layout(t, layout)
    apply = L.ALONG_ROWS if layout == 0 else L.ALONG_COLUMNS
    n_out = rows if apply == L.ALONG_ROWS else cols
    theirs = torch.empty(n_out, dtype=torch.float32, device=cuda)
    st = ref.reduce(d, apply, theirs, layout=layout, main_op=ENUM[main], reduce_op=ENUM[red], final_op=ENUM[fin])
    assert st == 0
    ours = linalg.reduce(d, apply, main_op=main, reduce_op=red, final_op=fin)
    exp = oracle.reduce(host, apply=apply, layout=layout, main_op=main, reduce_op=red, final_op=fin)
    oracle.assert_approx(exp, theirs.cpu().numpy(), 1e-5, "reference vs oracle")  # pins the oracle
    oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), 1e-5, "ours vs reference")
    if red == "max":
        assert torch.equal(ours, theirs)


@pytest.mark.parametrize("main,red,fin,scalar", [("identity", "add", "identity", 1.0), ("identity", "add", "mul_const", 0.125),
                                                 ("identity", "add", "div_const", 1024.0), ("sq", "add", "sqrt", 1.0),
                                                 ("abs", "max", "identity", 1.0)])
@pytest.mark.parametrize("rows,cols", [(1024, 32), (1024, 64), (1024, 256), (12345, 77), (200000, 64)])
@pytest.mark.parametrize("layout", [0, 1])
def test_strided_against_reference(cuda, oracle, ref, main, red, fin, scalar, rows, cols, layout):
    t, host = device_synth((rows, cols), np.float32, 1234, "uniform", -1, 1, cuda)
    d = as_layout(t, layout)
    apply = L.ALONG_COLUMNS if layout == 0 else L.ALONG_ROWS
    n_out = rows if apply == L.ALONG_ROWS else cols
    fin_e = {"identity": 0, "sqrt": 1, "mul_const": 2, "div_const": 3}[fin]
    theirs = torch.empty(n_out, dtype=torch.float32, device=cuda)
    st = ref.reduce(d, apply, theirs, layout=layout, main_op=ENUM[main], reduce_op=ENUM[red], final_op=fin_e,
                    final_scalar=scalar)
    assert st == 0
    ours = linalg.reduce(d, apply, main_op=main, reduce_op=red, final_op=fin, final_scalar=scalar)
    exp = oracle.reduce(host, apply=apply, layout=layout, main_op=main, reduce_op=red, final_op=fin, final_scalar=scalar)
    # the reference's strided sum adds per-block results with fp32 atomics in scheduling order
    # (linalg/detail/strided_reduction.cuh:54-76): its error varies from run to run and grows with the
    # rows - with 200000 of them it is only good to ~5e-5, and 12345 have missed 1e-5 once
    ref_tol = 1e-5 if rows <= 2000 else (5e-5 if rows <= 20000 else 2e-4)
    oracle.assert_approx(exp, theirs.cpu().numpy(), ref_tol, "reference vs oracle")
    oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), ref_tol, "ours vs reference")
    oracle.assert_approx(exp, ours.cpu().numpy(), 1e-5, "ours vs oracle")


@pytest.mark.parametrize("op", ["argmin", "argmax"])
@pytest.mark.parametrize("rows,cols", [(11, 7), (1234, 33), (1234, 128), (1234, 500), (100000, 64)])
@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_kvp_against_reference(cuda, oracle, ref, op, rows, cols, dt):
    t, host = device_synth((rows, cols), dt, 3, "int", 0, 16, cuda)  # frequent ties
    init = float("inf") if op == "argmin" else -float("inf")
    theirs = linalg.KeyValueVector(rows, t.dtype, cuda)
    st = ref.reduce(t, L.ALONG_ROWS, theirs, main_op=L.MAIN_TO_KVP, reduce_op=L.REDUCE_ARGMIN if op == "argmin"
                    else L.REDUCE_ARGMAX, init=init, init_key=0)
    assert st == 0
    ours = linalg.reduce(t, L.ALONG_ROWS, main_op="to_kvp", reduce_op=op, init=init)
    assert torch.equal(ours.keys, theirs.keys)      # bit exact, ties -> lowest index
    assert torch.equal(ours.values, theirs.values)
    ek, ev = oracle.reduce(host, main_op="to_kvp", reduce_op=op, init=init)
    assert np.array_equal(theirs.keys.cpu().numpy().astype(np.int64), ek)


@pytest.mark.parametrize("nobs,cols,nkeys", [(128, 32, 6), (128, 32, 3), (100000, 37, 32), (100000, 37, 2048),
                                             (50000, 128, 1024)])
@pytest.mark.parametrize("weighted", [False, True])
def test_rows_by_key_against_reference(cuda, oracle, ref, nobs, cols, nkeys, weighted):
    A, hA = device_synth((nobs, cols), np.float32, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((nobs,), np.int32, 4321, "int", 0, nkeys, cuda)
    w, hw = device_synth((nobs,), np.float32, 77, "uniform", 0, 2, cuda) if weighted else (None, None)
    theirs = torch.empty((nkeys, cols), dtype=torch.float32, device=cuda)
    assert ref.rows_by_key(theirs, A, keys, nkeys, weights=w) == 0
    ours = linalg.reduce_rows_by_key(A, keys, nkeys, d_weights=w)
    exp, _ = oracle.rows_by_key(hA, hk, nkeys, weights=hw)
    # the reference adds in fp32 with one global atomic per element, in scheduling order
    # (linalg/detail/reduce_rows_by_key.cuh:299): thousands of rows per key leave it good to a
    # few 1e-4 only, and the figure changes from run to run
    oracle.assert_approx(exp, theirs.cpu().numpy(), 1e-3, "reference vs oracle")
    oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), 1e-3, "ours vs reference")
    oracle.assert_approx(exp, ours.cpu().numpy(), 1e-5, "ours vs oracle")


@pytest.mark.parametrize("rows,cols,nkeys", [(1, 1234, 7), (9, 9999, 42), (63, 1234, 515), (1024, 1234, 127)])
def test_cols_by_key_against_reference(cuda, oracle, ref, rows, cols, nkeys):
    data, hd = device_synth((rows, cols), np.float32, 1234, "uniform", -1, 1, cuda)
    keys, hk = device_synth((cols,), np.int32, 55, "int", 0, nkeys, cuda)
    theirs = torch.empty((rows, nkeys), dtype=torch.float32, device=cuda)
    assert ref.cols_by_key(theirs, data, keys, nkeys) == 0
    ours = linalg.reduce_cols_by_key(data, keys, nkeys=nkeys)
    exp = oracle.cols_by_key(hd, hk, nkeys)
    oracle.assert_approx(exp, theirs.cpu().numpy(), 1e-3, "reference vs oracle")
    oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), 1e-3, "ours vs reference")


@pytest.mark.parametrize("main,red,fin", [("identity", "add", "identity"), ("sq", "add", "sqrt"), ("abs", "max", "identity")])
@pytest.mark.parametrize("rows,cols", [(1234, 33), (1000, 500), (9, 33333)])
@pytest.mark.parametrize("apply", [0, 1])
def test_double_precision_against_reference(cuda, oracle, ref, main, red, fin, rows, cols, apply):
    t, host = device_synth((rows, cols), np.float64, 4321, "uniform", -1, 1, cuda)
    n_out = rows if apply == L.ALONG_ROWS else cols
    theirs = torch.empty(n_out, dtype=torch.float64, device=cuda)
    assert ref.reduce(t, apply, theirs, main_op=ENUM[main], reduce_op=ENUM[red], final_op=ENUM[fin]) == 0
    ours = linalg.reduce(t, apply, main_op=main, reduce_op=red, final_op=fin)
    exp = oracle.reduce(host, apply=apply, main_op=main, reduce_op=red, final_op=fin)
    oracle.assert_approx(exp, theirs.cpu().numpy(), 1e-9, "reference vs oracle")
    oracle.assert_approx(theirs.cpu().numpy(), ours.cpu().numpy(), 1e-9, "ours vs reference")
    if red == "max":
        assert torch.equal(ours, theirs)
