"""ctypes wrapper of the CPU oracle (oracle/oracle.c) - TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg import this module.
Inputs and outputs are numpy arrays on the host.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")

DT = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.float16): 2, np.dtype(np.int32): 3,
      np.dtype(np.int64): 4, np.dtype(np.int16): 5, np.dtype(np.uint32): 6}
MAIN = {"identity": 0, "sq": 1, "abs": 2, "nz": 3, "to_kvp": 4}
REDUCE = {"add": 0, "min": 1, "max": 2, "argmin": 3, "argmax": 4}
FINAL = {"identity": 0, "sqrt": 1, "mul_const": 2, "div_const": 3, "abs": 4}
KIND = {"uniform": 0, "normal": 1, "int": 2}

_lib = None


def build():
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        lib = ctypes.CDLL(LIB_PATH)
        vp, i32, i64, dbl, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_double, ctypes.c_uint64
        lib.synth_fill.argtypes = [vp, i32, i64, i64, u64, i32, dbl, dbl]
        lib.oracle_reduce.argtypes = [vp, i32, i32, i32, i64, i64, i32, i32, i32, dbl, dbl, i64, i32, vp, vp]
        lib.oracle_rows_by_key.argtypes = [vp, i32, i64, vp, i32, vp, i64, i64, i64, i32, vp, vp]
        lib.oracle_cols_by_key.argtypes = [vp, i32, vp, i32, i64, i64, i64, i32, vp]
        lib.oracle_row_normalize.argtypes = [vp, vp, i32, i64, i64, i32, dbl]
        lib.oracle_compare_approx.argtypes = [vp, vp, i64, dbl, vp, vp, vp]
        lib.oracle_compare_approx.restype = i64
        lib.omp_threads.restype = i32
        lib.omp_row_sum_f32.argtypes = [vp, i64, i64, i32, i32, vp]
        lib.omp_row_sum_f32.restype = None
        lib.omp_col_sum_f32.argtypes = [vp, i64, i64, dbl, vp]
        lib.omp_row_argmin_f32.argtypes = [vp, i64, i64, vp, vp]
        lib.omp_row_argmin_f32.restype = None
        lib.omp_rows_by_key_f32.argtypes = [vp, vp, i64, i64, i64, vp, vp]
        _lib = lib
    return _lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def synth(shape, dtype, seed, kind, lo=0.0, hi=1.0, first_index=0):
    """Host copy of b2r_synth_fill: same bits as the device generator."""
    out = np.empty(shape, dtype=dtype)
    load().synth_fill(_ptr(out), DT[out.dtype], out.size, first_index, seed, KIND[kind], float(lo), float(hi))
    return out


def reduce(data, apply=0, layout=0, main_op="identity", reduce_op="add", final_op="identity", final_scalar=1.0,
           init=0.0, init_key=0, inplace=False, prev_val=None, prev_key=None):
    """fp64 oracle of raft::linalg::reduce. `data` is a 2-D array whose MEMORY is in `layout`
    (0 row-major, 1 column-major) for the logical shape data.shape. Returns out (float64), or
    (keys int64, values float64) for argmin / argmax."""
    n_rows, n_cols = data.shape
    mem = np.ascontiguousarray(data if layout == 0 else data.T)
    n_out = n_rows if apply == 0 else n_cols
    kvp = reduce_op in ("argmin", "argmax")
    out_val = np.zeros(n_out, dtype=np.float64) if prev_val is None else np.array(prev_val, dtype=np.float64)
    out_key = np.zeros(n_out, dtype=np.int64) if prev_key is None else np.array(prev_key, dtype=np.int64)
    rc = load().oracle_reduce(_ptr(mem), DT[mem.dtype], layout, apply, n_rows, n_cols, MAIN[main_op],
                              REDUCE[reduce_op], FINAL[final_op], float(final_scalar), float(init), int(init_key),
                              1 if inplace else 0, _ptr(out_val), _ptr(out_key) if kvp else None)
    assert rc == 0, rc
    return (out_key, out_val) if kvp else out_val


def rows_by_key(A, keys, nkeys, weights=None, prev_sums=None, prev_counts=None, lda=None):
    nrows = keys.shape[0]
    ncols = A.shape[1]
    A = np.ascontiguousarray(A)
    keys = np.ascontiguousarray(keys)
    reset = prev_sums is None
    sums = np.zeros((nkeys, ncols), dtype=np.float64) if reset else np.array(prev_sums, dtype=np.float64)
    counts = np.zeros(nkeys, dtype=np.int64) if prev_counts is None else np.array(prev_counts, dtype=np.int64)
    w = np.ascontiguousarray(weights) if weights is not None else None
    rc = load().oracle_rows_by_key(_ptr(A), DT[A.dtype], lda or A.shape[1], _ptr(keys), DT[keys.dtype], _ptr(w),
                                   nrows, ncols, nkeys, 1 if reset else 0, _ptr(sums), _ptr(counts))
    assert rc == 0, rc
    return sums, counts


def cols_by_key(data, keys, nkeys, prev=None):
    data = np.ascontiguousarray(data)
    keys = np.ascontiguousarray(keys)
    nrows, ncols = data.shape
    reset = prev is None
    out = np.zeros((nrows, nkeys), dtype=np.float64) if reset else np.array(prev, dtype=np.float64)
    rc = load().oracle_cols_by_key(_ptr(data), DT[data.dtype], _ptr(keys), DT[keys.dtype], nrows, ncols, nkeys,
                                   1 if reset else 0, _ptr(out))
    assert rc == 0, rc
    return out


def row_normalize(data, norm_type="L2", eps=1e-8, prev=None):
    """Oracle of raft::linalg::row_normalize (linalg/normalize.cuh:88-107): fp64 norm rounded once
    to the element type, division in the element type; rows with norm <= eps keep `prev` (zeros
    when not given)."""
    data = np.ascontiguousarray(data)
    out = np.zeros_like(data) if prev is None else np.array(prev, dtype=data.dtype)
    n_rows, n_cols = data.shape
    rc = load().oracle_row_normalize(_ptr(data), _ptr(out), DT[data.dtype], n_rows, n_cols,
                                     {"L1": 1, "L2": 2, "Linf": 3}[norm_type], float(eps))
    assert rc == 0, rc
    return out


def compare_approx(expect, actual, eps):
    """The reference's hybrid tolerance (cpp/tests/test_utils.h:31-45): |a-b| <= eps, or
    |a-b|/max(|a|,|b|) <= eps. Returns (n_mismatch, worst_abs, worst_rel, worst_index)."""
    e = np.ascontiguousarray(np.asarray(expect, dtype=np.float64).ravel())
    a = np.ascontiguousarray(np.asarray(actual, dtype=np.float64).ravel())
    assert e.shape == a.shape, (e.shape, a.shape)
    wa, wr, wi = ctypes.c_double(), ctypes.c_double(), ctypes.c_int64()
    bad = load().oracle_compare_approx(_ptr(e), _ptr(a), e.size, float(eps), ctypes.byref(wa), ctypes.byref(wr),
                                       ctypes.byref(wi))
    return bad, wa.value, wr.value, wi.value


def assert_approx(expect, actual, eps, what=""):
    bad, wa, wr, wi = compare_approx(expect, actual, eps)
    assert bad == 0, f"{what}: {bad} mismatches at eps={eps}; worst abs={wa:.3e} rel={wr:.3e} at index {wi}"


# ---- host baseline (OpenMP) -----------------------------------------------------------------
def omp_threads():
    return load().omp_threads()


def omp_row_sum(data, square=False, root=False):
    out = np.empty(data.shape[0], dtype=np.float32)
    load().omp_row_sum_f32(_ptr(data), data.shape[0], data.shape[1], int(square), int(root), _ptr(out))
    return out


def omp_col_sum(data, scale=1.0):
    out = np.empty(data.shape[1], dtype=np.float32)
    rc = load().omp_col_sum_f32(_ptr(data), data.shape[0], data.shape[1], float(scale), _ptr(out))
    assert rc == 0
    return out


def omp_row_argmin(data):
    k = np.empty(data.shape[0], dtype=np.int32)
    v = np.empty(data.shape[0], dtype=np.float32)
    load().omp_row_argmin_f32(_ptr(data), data.shape[0], data.shape[1], _ptr(k), _ptr(v))
    return k, v


def omp_rows_by_key(A, keys, nkeys):
    sums = np.empty((nkeys, A.shape[1]), dtype=np.float32)
    counts = np.empty(nkeys, dtype=np.int64)
    rc = load().omp_rows_by_key_f32(_ptr(A), _ptr(keys), A.shape[0], A.shape[1], nkeys, _ptr(sums), _ptr(counts))
    assert rc == 0
    return sums, counts
