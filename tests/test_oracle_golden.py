"""Pins the CPU oracle to the known-answer vectors of the reference's own tests (read from
the reference's test sources as text) and to its comparison rule. Runs without a GPU."""
import numpy as np
import pytest


def test_simple_max_reduce_3x4(oracle):
    # cpp/tests/linalg/reduce.cu:106-178: 3x4 matrix 1..12, identity / max / identity, init 0
    flat = np.arange(1, 13, dtype=np.float32)
    row_major = flat.reshape(3, 4)
    assert oracle.reduce(row_major, apply=0, layout=0, reduce_op="max").tolist() == [4, 8, 12]
    assert oracle.reduce(row_major, apply=1, layout=0, reduce_op="max").tolist() == [9, 10, 11, 12]
    col_major = flat.reshape(4, 3).T  # same memory read as a column-major 3x4 matrix
    assert oracle.reduce(col_major, apply=0, layout=1, reduce_op="max").tolist() == [10, 11, 12]
    assert oracle.reduce(col_major, apply=1, layout=1, reduce_op="max").tolist() == [3, 6, 9, 12]
    for dt in (np.float64,):
        assert oracle.reduce(row_major.astype(dt), apply=0, reduce_op="max").tolist() == [4, 8, 12]


def _pair_reduce(oracle, op, a, b):
    """reduce_op(a, b) for key/value pairs, evaluated through the oracle: a is the initial
    value, b the single element of a 1 x (b.key+1) row padded so that b sits at index b.key."""
    (ka, va), (kb, vb) = a, b
    pad = -np.inf if op == "argmax" else np.inf
    row = np.full((1, kb + 1), pad, dtype=np.float32)
    row[0, kb] = vb
    k, v = oracle.reduce(row, apply=0, reduce_op=op, main_op="to_kvp", init=va, init_key=ka)
    return int(k[0]), float(np.float32(v[0]))


def test_argmin_argmax_operator_cases(oracle):
    # cpp/tests/core/operators_device.cu:178-216 (same cases in operators_host.cpp:134-172)
    a, b, c = (0, np.float32(1.2)), (0, np.float32(3.4)), (1, np.float32(1.2))
    f = lambda p: (p[0], float(p[1]))
    amin = lambda x, y: _pair_reduce(oracle, "argmin", x, y)
    amax = lambda x, y: _pair_reduce(oracle, "argmax", x, y)
    assert amin(a, b) == f(a) and amin(b, a) == f(a)
    assert amin(a, c) == f(a) and amin(c, a) == f(a)
    assert amin(b, c) == f(c) and amin(c, b) == f(c)
    assert amax(a, b) == f(b) and amax(b, a) == f(b)
    assert amax(a, c) == f(a) and amax(c, a) == f(a)
    assert amax(b, c) == f(b) and amax(c, b) == f(b)


def test_argmin_argmax_matrix(oracle):
    # cpp/tests/matrix/argmin.cu:71-75 -> {0, 3, 3}; cpp/tests/matrix/argmax.cu, same matrix -> {3, 0, 2}
    m = np.array([0.1, 0.2, 0.3, 0.4, 0.4, 0.3, 0.2, 0.1, 0.2, 0.3, 0.5, 0.0], dtype=np.float32).reshape(3, 4)
    k, v = oracle.reduce(m, reduce_op="argmin", main_op="to_kvp", init=np.inf)
    assert k.tolist() == [0, 3, 3]
    assert np.allclose(v, [0.1, 0.1, 0.0])
    k, _ = oracle.reduce(m, reduce_op="argmax", main_op="to_kvp", init=-np.inf)
    assert k.tolist() == [3, 0, 2]
    k, _ = oracle.reduce(m.astype(np.float64), reduce_op="argmin", main_op="to_kvp", init=np.inf)
    assert k.tolist() == [0, 3, 3]


@pytest.mark.parametrize("rows,cols,value,tol", [(4, 5, 1.0, 1e-4), (1024, 32, 1.0, 1e-4), (1024, 256, 1.0, 1e-4),
                                                 (1, 30, 0.001, 1e-4), (17, 5, 0.001, 1e-4), (7, 23, 0.001, 1e-4),
                                                 (3, 97, 0.001, 1e-4)])
@pytest.mark.parametrize("row_major", [True, False])
def test_constant_matrix_sums(oracle, rows, cols, value, tol, row_major):
    # cpp/tests/stats/sum.cu:50-129: column sums of a constant matrix equal rows * value
    m = np.full((rows, cols), value, dtype=np.float32)
    got = oracle.reduce(m, apply=1, layout=0 if row_major else 1)
    oracle.assert_approx(np.full(cols, rows * value), got, tol)


def test_error_compensation_case(oracle):
    # cpp/tests/stats/sum.cu:58-75: per column, triples (3v, -v*1e7, +v*1e7) must still sum to rows*v
    rows, cols, v = 1023, 32, 1.0
    m = np.full((rows, cols), v, dtype=np.float32)
    m[2::3] = v * 1e7
    m[1::3] = -v * 1e7
    m[0::3] = 3 * v
    got = oracle.reduce(m, apply=1)
    assert np.allclose(got, rows * v, rtol=1e-12)


def test_norm_functor_choice(oracle):
    # linalg/detail/norm.cuh:26-37: L1 = abs/add, L2 = sq/add (no root), Linf = abs/max
    m = np.array([[3, -4], [-1, 2]], dtype=np.float32)
    assert oracle.reduce(m, main_op="abs").tolist() == [7, 3]
    assert oracle.reduce(m, main_op="sq").tolist() == [25, 5]
    assert oracle.reduce(m, main_op="sq", final_op="sqrt").tolist() == [5, np.sqrt(5)]
    assert oracle.reduce(m, main_op="abs", reduce_op="max").tolist() == [4, 2]
    assert oracle.reduce(m, apply=1, main_op="abs").tolist() == [4, 6]


def test_inplace_rule(oracle):
    # cpp/tests/linalg/reduce.cuh:40-44: inplace -> final(reduce(old, acc))
    m = np.arange(6, dtype=np.float32).reshape(2, 3)
    prev = np.array([10.0, 20.0])
    got = oracle.reduce(m, main_op="sq", final_op="sqrt", inplace=True, prev_val=prev)
    assert np.allclose(got, np.sqrt(prev + (m.astype(np.float64) ** 2).sum(1)))


def test_rows_and_cols_by_key_small(oracle):
    # cpp/tests/linalg/reduce_rows_by_key.cu:21-44 and reduce_cols_by_key.cu:20-42
    A = np.arange(12, dtype=np.float32).reshape(4, 3)
    keys = np.array([1, 0, 1, 2], dtype=np.int32)
    sums, counts = oracle.rows_by_key(A, keys, 3)
    assert sums.tolist() == [[3, 4, 5], [6, 8, 10], [9, 10, 11]]
    assert counts.tolist() == [1, 2, 1]
    w = np.array([1, 2, 3, 4], dtype=np.float32)
    sums, _ = oracle.rows_by_key(A, keys, 3, weights=w)
    assert sums.tolist() == [[6, 8, 10], [18, 22, 26], [36, 40, 44]]
    ckeys = np.array([0, 1, 0], dtype=np.int32)
    assert oracle.cols_by_key(A, ckeys, 2).tolist() == [[2, 1], [8, 4], [14, 7], [20, 10]]


def test_compare_approx_rule(oracle):
    # cpp/tests/test_utils.h:31-45: absolute OR relative
    assert oracle.compare_approx([1e-7], [5e-6], 1e-5)[0] == 0  # abs
    assert oracle.compare_approx([1000.0], [1000.005], 1e-5)[0] == 0  # rel
    assert oracle.compare_approx([1.0], [1.001], 1e-5)[0] == 1


def test_synth_is_a_pure_function_of_index(oracle):
    a = oracle.synth((1000,), np.float32, 7, "uniform", -1, 1)
    b = oracle.synth((600,), np.float32, 7, "uniform", -1, 1, first_index=400)
    assert np.array_equal(a[400:], b)
    assert a.min() >= -1 and a.max() < 1
    k = oracle.synth((5000,), np.int32, 5, "int", 0, 1024)
    assert k.min() >= 0 and k.max() < 1024
    n = oracle.synth((200000,), np.float32, 1, "normal")
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1) < 0.01


def test_synth_golden(oracle):
    # committed fixture: first values of the generator, so the host and device generators
    # cannot drift apart unnoticed (the GPU test compares the device output to the same file)
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "synth_v1.npz")
    g = np.load(path)
    assert np.array_equal(g["uniform_f32"], oracle.synth((64,), np.float32, 0, "uniform", -1, 1))
    assert np.array_equal(g["normal_f32"], oracle.synth((64,), np.float32, 1, "normal"))
    assert np.array_equal(g["int_f32"], oracle.synth((64,), np.float32, 3, "int", 0, 16))
    assert np.array_equal(g["keys_i32"], oracle.synth((64,), np.int32, 5, "int", 0, 1024))
    assert np.array_equal(g["uniform_f64"], oracle.synth((64,), np.float64, 2, "uniform", 0, 1))


def test_map_reduce_known_answers(oracle):
    # cpp/tests/linalg/map_then_reduce.cu:133-171: 1237 values in [2, 3), a 1 planted at index 42 and a
    # 5 at 337; min with neutral numeric_limits::max gives 1, max with neutral numeric_limits::min gives 5
    v = oracle.synth((1237,), np.float32, 137, "uniform", 2, 3)
    v[42], v[337] = 1.0, 5.0
    lo = oracle.reduce(v.reshape(1, -1), reduce_op="min", init=float(np.finfo(np.float32).max))
    hi = oracle.reduce(v.reshape(1, -1), reduce_op="max", init=float(np.finfo(np.float32).tiny))
    assert lo[0] == 1.0 and hi[0] == 5.0


def test_row_normalize_known_answers(oracle):
    # hand-checkable rows: (3, 4) has L1 7, L2 5, Linf 4; a zero row keeps the previous content
    x = np.array([[3, 4], [0, 0], [-6, 8]], dtype=np.float32)
    prev = np.full_like(x, 9)
    assert np.array_equal(oracle.row_normalize(x, "L2", prev=prev),
                          np.array([[0.6, 0.8], [9, 9], [-0.6, 0.8]], dtype=np.float32))
    assert np.array_equal(oracle.row_normalize(x, "Linf", prev=prev),
                          np.array([[0.75, 1], [9, 9], [-0.75, 1]], dtype=np.float32))
    assert np.allclose(oracle.row_normalize(x.astype(np.float64), "L1", prev=prev.astype(np.float64)),
                       np.array([[3 / 7, 4 / 7], [9, 9], [-6 / 14, 8 / 14]]), rtol=0, atol=1e-15)
