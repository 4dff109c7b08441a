"""Parity of b2r_reduce / b2r_norm (through the C ABI) with the fp64 oracle, over the shape and
type grids of the reference's own tests. Tolerances are the reference's (CompareApprox rule)."""
import numpy as np
import pytest
import torch

from raft_b200 import _lib as L
from raft_b200 import linalg
from util import as_layout, device_synth

pytestmark = pytest.mark.gpu


def test_device_generator_matches_host(cuda, oracle):
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "synth_v1.npz"))
    for name, dt, seed, kind, lo, hi in [("uniform_f32", np.float32, 0, "uniform", -1, 1),
                                         ("normal_f32", np.float32, 1, "normal", 0, 1),
                                         ("int_f32", np.float32, 3, "int", 0, 16),
                                         ("keys_i32", np.int32, 5, "int", 0, 1024),
                                         ("uniform_f64", np.float64, 2, "uniform", 0, 1)]:
        _, host = device_synth((64,), dt, seed, kind, lo, hi, cuda)
        assert np.array_equal(host, g[name]), name
    for dt in (np.float32, np.float64, np.float16):
        _, host = device_synth((100003,), dt, 11, "normal", 0, 1, cuda)
        assert np.array_equal(host, oracle.synth((100003,), dt, 11, "normal"))
        _, host = device_synth((100003,), dt, 12, "uniform", -3, 5, cuda)
        assert np.array_equal(host, oracle.synth((100003,), dt, 12, "uniform", -3, 5))


def test_simple_max_reduce_3x4(cuda):
    # cpp/tests/linalg/reduce.cu:106-178
    for dt in (torch.float32, torch.float64):
        flat = torch.arange(1, 13, dtype=dt, device=cuda)
        rm = flat.reshape(3, 4)
        assert linalg.reduce(rm, linalg.ALONG_ROWS, reduce_op="max").tolist() == [4, 8, 12]
        assert linalg.reduce(rm, linalg.ALONG_COLUMNS, reduce_op="max").tolist() == [9, 10, 11, 12]
        cm = flat.reshape(4, 3).t()
        assert linalg.reduce(cm, linalg.ALONG_ROWS, reduce_op="max").tolist() == [10, 11, 12]
        assert linalg.reduce(cm, linalg.ALONG_COLUMNS, reduce_op="max").tolist() == [3, 6, 9, 12]


# cpp/tests/linalg/reduce.cu:292-317: (in, out) types x rows x cols x layout x axis, sq/add/sqrt
@pytest.mark.parametrize("in_dt,out_dt,tol", [(np.float32, torch.float32, 2e-6), (np.float64, torch.float64, 1e-9),
                                              (np.float32, torch.float64, 1e-9)])
@pytest.mark.parametrize("rows", [11, 1234])
@pytest.mark.parametrize("cols", [7, 33, 128, 500])
@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("apply", [0, 1])
def test_reduce_grid(cuda, oracle, in_dt, out_dt, tol, rows, cols, layout, apply):
    t, host = device_synth((rows, cols), in_dt, 1234, "uniform", -1, 1, cuda)
    d = as_layout(t, layout)
    n_out = rows if apply == 0 else cols
    dots = torch.empty(n_out, dtype=out_dt, device=cuda)
    linalg.reduce(d, apply, dots, init=0.0, main_op="sq", final_op="sqrt")
    exp = oracle.reduce(host, apply=apply, layout=layout, main_op="sq", final_op="sqrt")
    oracle.assert_approx(exp, dots.cpu().numpy(), tol, "not inplace")
    # second pass in place, as cpp/tests/linalg/reduce.cu:191-241 does
    exp2 = oracle.reduce(host, apply=apply, layout=layout, main_op="sq", final_op="sqrt", inplace=True,
                         prev_val=dots.cpu().numpy().astype(np.float64))
    linalg.reduce(d, apply, dots, init=0.0, inplace=True, main_op="sq", final_op="sqrt")
    oracle.assert_approx(exp2, dots.cpu().numpy(), tol, "inplace")


# cpp/tests/linalg/reduce.cu:321-341 "thick": few rows, very long
@pytest.mark.parametrize("rows", [3, 9])
@pytest.mark.parametrize("cols", [17771, 33333, 100000])
@pytest.mark.parametrize("in_dt,tol", [(np.float32, 1e-4), (np.float64, 1e-6)])
def test_reduce_thick(cuda, oracle, rows, cols, in_dt, tol):
    t, host = device_synth((rows, cols), in_dt, 1234, "uniform", -1, 1, cuda)
    got = linalg.reduce(t, linalg.ALONG_ROWS, main_op="sq", final_op="sqrt")
    oracle.assert_approx(oracle.reduce(host, main_op="sq", final_op="sqrt"), got.cpu().numpy(), tol)
    got = linalg.reduce(t, linalg.ALONG_ROWS)
    oracle.assert_approx(oracle.reduce(host), got.cpu().numpy(), 1e-5 if in_dt == np.float32 else 1e-9)


# one very long row and a few long rows: the split-row path with scratch memory
@pytest.mark.parametrize("rows,cols", [(1, 5_000_000), (2, 1_000_003), (5, 262144), (40, 65536)])
def test_reduce_split_rows(cuda, oracle, rows, cols):
    t, host = device_synth((rows, cols), np.float32, 99, "uniform", -1, 1, cuda)
    assert linalg.reduce_workspace_bytes(t) > 0
    got = linalg.reduce(t, linalg.ALONG_ROWS)
    oracle.assert_approx(oracle.reduce(host), got.cpu().numpy(), 1e-5)
    ws = torch.empty(linalg.reduce_workspace_bytes(t), dtype=torch.uint8, device=cuda)
    got2 = linalg.reduce(t, linalg.ALONG_ROWS, workspace=ws)
    assert torch.equal(got, got2)  # caller workspace and internal scratch give the same bits
    got = linalg.reduce(t, linalg.ALONG_ROWS, main_op="abs", reduce_op="max")
    assert np.array_equal(got.cpu().numpy(), np.abs(host).max(axis=1))
    kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
    assert np.array_equal(kv.keys.cpu().numpy(), host.argmin(axis=1))


# a handful of very long rows: the ring form of the split (segments of a row come through 32 KB bulk copies);
# the threshold is lowered so that ragged lengths, tails shorter than a vector and a last segment of a few
# vectors are all seen at sizes the oracle finishes quickly, then one case at the default threshold
@pytest.mark.parametrize("rows,cols", [(1, 5_000_000), (2, 1_000_003), (3, 262144 + 4), (7, 300_001), (16, 2048 * 148)])
@pytest.mark.parametrize("in_dt", [np.float32, np.float64, np.float16])
def test_reduce_split_rows_ring(cuda, oracle, knobs, rows, cols, in_dt):
    knobs(B2R_ROW_SPLIT_RING_MB="1")
    t, host = device_synth((rows, cols), in_dt, 77, "uniform", -1, 1, cuda)
    tol = {np.float32: 1e-5, np.float64: 1e-10, np.float16: 1e-5}[in_dt]
    got = linalg.reduce(t, linalg.ALONG_ROWS, out_dtype=torch.float32 if in_dt == np.float16 else None)
    oracle.assert_approx(oracle.reduce(host), got.cpu().numpy(), tol)
    knobs(B2R_ROW_SPLIT_RING="2")
    plain = linalg.reduce(t, linalg.ALONG_ROWS, out_dtype=torch.float32 if in_dt == np.float16 else None)
    oracle.assert_approx(plain.cpu().numpy().astype(np.float64), got.cpu().numpy(), tol)
    knobs(B2R_ROW_SPLIT_RING=None)
    if in_dt == np.float16:
        return
    prev = got.cpu().numpy().astype(np.float64)
    linalg.reduce(t, linalg.ALONG_ROWS, got, inplace=True, main_op="sq", final_op="sqrt")
    oracle.assert_approx(oracle.reduce(host, main_op="sq", final_op="sqrt", inplace=True, prev_val=prev),
                         got.cpu().numpy(), 10 * tol)
    got = linalg.reduce(t, linalg.ALONG_ROWS, main_op="abs", reduce_op="max")
    assert np.array_equal(got.cpu().numpy(), np.abs(host).max(axis=1))
    if in_dt == np.float32:
        kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
        assert np.array_equal(kv.keys.cpu().numpy(), host.argmin(axis=1))
        assert np.array_equal(kv.values.cpu().numpy(), host.min(axis=1))


def test_reduce_split_rows_ring_default_threshold(cuda, oracle):
    t, host = device_synth((2, (1 << 24) + 5), np.float32, 5, "uniform", -1, 1, cuda)  # 64 MiB + 20 B per row
    got = linalg.reduce(t, linalg.ALONG_ROWS, main_op="sq", final_op="sqrt")
    oracle.assert_approx(oracle.reduce(host, main_op="sq", final_op="sqrt"), got.cpu().numpy(), 1e-5)
    ones = torch.ones((1, 1 << 26), dtype=torch.float32, device=cuda)
    assert linalg.reduce(ones, linalg.ALONG_ROWS).item() == float(1 << 26)


# cpp/tests/linalg/coalesced_reduction.cu:109-139
@pytest.mark.parametrize("rows,cols,tol32,tol64", [(r, c, 2e-6, 1e-9) for r in (50, 10000)
                                                   for c in (2, 3, 7, 9, 20, 55, 100, 270)] + [(10, 25000, 1e-4, 1e-7)])
@pytest.mark.parametrize("in_dt", [np.float32, np.float64])
def test_coalesced_grid(cuda, oracle, rows, cols, tol32, tol64, in_dt):
    tol = tol32 if in_dt == np.float32 else tol64
    t, host = device_synth((rows, cols), in_dt, 1234, "uniform", -1, 1, cuda)
    dots = linalg.coalesced_reduction(t, main_op="sq", final_op="sqrt")
    exp = oracle.reduce(host, main_op="sq", final_op="sqrt")
    oracle.assert_approx(exp, dots.cpu().numpy(), tol)
    linalg.coalesced_reduction(t, dots, inplace=True, main_op="sq", final_op="sqrt")
    exp2 = oracle.reduce(host, main_op="sq", final_op="sqrt", inplace=True, prev_val=exp)
    oracle.assert_approx(exp2, dots.cpu().numpy(), 10 * tol)


# cpp/tests/linalg/strided_reduction.cu:94-102
@pytest.mark.parametrize("cols", [32, 64, 128, 256])
@pytest.mark.parametrize("in_dt,tol", [(np.float32, 1e-5), (np.float64, 1e-9)])
def test_strided_grid(cuda, oracle, cols, in_dt, tol):
    t, host = device_synth((1024, cols), in_dt, 1234, "uniform", -1, 1, cuda)
    dots = linalg.strided_reduction(t, main_op="sq")
    oracle.assert_approx(oracle.reduce(host, apply=1, main_op="sq"), dots.cpu().numpy(), tol)


# cpp/tests/linalg/norm.cu:236-306: L1 / L2 x root / no root x row / column x float, double, half
@pytest.mark.parametrize("norm_type,main", [("L1", "abs"), ("L2", "sq")])
@pytest.mark.parametrize("fin", ["identity", "sqrt"])
@pytest.mark.parametrize("rows,cols", [(11, 7), (11, 500), (1234, 33), (1234, 128)])
@pytest.mark.parametrize("in_dt,tol", [(np.float32, 1e-5), (np.float64, 1e-8), (np.float16, 1e-3)])
@pytest.mark.parametrize("apply", [0, 1])
@pytest.mark.parametrize("layout", [0, 1])
def test_norm_grid(cuda, oracle, norm_type, main, fin, rows, cols, in_dt, tol, apply, layout):
    t, host = device_synth((rows, cols), in_dt, 1234, "uniform", -1, 1, cuda)
    d = as_layout(t, layout)
    got = linalg.norm(d, norm_type, apply, fin_op=fin)
    assert got.dtype == (torch.float32 if in_dt == np.float16 else t.dtype)
    exp = oracle.reduce(host, apply=apply, layout=layout, main_op=main, final_op=fin)
    oracle.assert_approx(exp, got.cpu().numpy(), tol)


def test_norm_linf_and_l0(cuda, oracle):
    t, host = device_synth((321, 77), np.float32, 5, "normal", 0, 1, cuda)
    for apply in (0, 1):
        got = linalg.norm(t, "Linf", apply)
        assert np.array_equal(got.cpu().numpy(), np.abs(host).max(axis=1 - apply))  # max is exact
    with pytest.raises(L.B2RError):  # the reference throws for L0 (linalg/detail/norm.cuh:36)
        linalg.norm(t, "L0")


# cpp/tests/linalg/reduce.cu:346-411: key/value reductions for short / float / double
@pytest.mark.parametrize("in_dt", [np.int16, np.float32, np.float64, np.int32])
@pytest.mark.parametrize("rows", [11, 1234])
@pytest.mark.parametrize("cols", [7, 33, 128, 500])
@pytest.mark.parametrize("op", ["argmax", "argmin"])
def test_kvp_grid(cuda, oracle, in_dt, rows, cols, op):
    if np.issubdtype(in_dt, np.integer):
        t, host = device_synth((rows, cols), in_dt, 1234, "int", -50, 50, cuda)  # many ties
    else:
        t, host = device_synth((rows, cols), in_dt, 1234, "uniform", -1, 1, cuda)
    floating = not np.issubdtype(in_dt, np.integer)
    init = (float("inf") if op == "argmin" else -float("inf")) if floating else (32767 if op == "argmin" else -32768)
    kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op=op, init=init, init_key=0)
    ek, ev = oracle.reduce(host, main_op="to_kvp", reduce_op=op, init=init, init_key=0)
    assert np.array_equal(kv.keys.cpu().numpy().astype(np.int64), ek)  # bit exact
    assert np.array_equal(kv.values.cpu().numpy().astype(np.float64), ev)
    # the reference's test initial value {0, 0} (reduce.cu:360-386): a row whose extreme does not
    # beat 0 keeps the initial pair
    kv0 = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op=op, init=0, init_key=0)
    ek, ev = oracle.reduce(host, main_op="to_kvp", reduce_op=op, init=0, init_key=0)
    assert np.array_equal(kv0.keys.cpu().numpy().astype(np.int64), ek)
    assert np.array_equal(kv0.values.cpu().numpy().astype(np.float64), ev)
    # in place: combine with the previous pairs
    linalg.reduce(t, linalg.ALONG_ROWS, kv0, main_op="to_kvp", reduce_op=op, init=init, inplace=True)
    ek2, ev2 = oracle.reduce(host, main_op="to_kvp", reduce_op=op, init=init, inplace=True, prev_val=ev, prev_key=ek)
    assert np.array_equal(kv0.keys.cpu().numpy().astype(np.int64), ek2)
    assert np.array_equal(kv0.values.cpu().numpy().astype(np.float64), ev2)


@pytest.mark.parametrize("cols", [4, 16, 64, 128, 100, 1024, 3000])
@pytest.mark.parametrize("op", ["argmin", "argmax"])
@pytest.mark.parametrize("ring", [False, True])
def test_kvp_ties_with_the_start_value(cuda, oracle, knobs, cols, op, ring):
    """argmin_op / argmax_op are exact folds over {init, elements} (core/operators.hpp:187-203): an element EQUAL
    to init.value wins only with a lower key than init.key, NaN elements never win, and a row that holds nothing
    better keeps the start pair. The one-pass kernels walk a lane's elements with a strict compare and settle
    these cases afterwards; every one of them is checked against the oracle here, for start keys below, inside
    and above the columns, on the direct kernels and on the ring kernel."""
    if ring:
        knobs(B2R_ROW_TMA="1")
    rows = 6000
    best = 0.0 if op == "argmin" else 9.0
    t, host = device_synth((rows, cols), np.float32, 77, "int", 0, 10, cuda)
    host = host.copy()
    host[0::7] = 5.0                 # whole rows equal to the start value used below
    host[1::7] = np.inf if op == "argmin" else -np.inf   # nothing can beat an infinite start value
    host[2::7, : cols // 2] = np.nan   # NaN never wins
    host[3::7] = np.nan              # a row of NaN keeps the start pair
    host[4::7, cols - 1] = best      # the best value in the last column only
    t.copy_(torch.from_numpy(host))
    for init, init_key in ((5.0, 0), (5.0, cols // 2), (5.0, 10 * cols), (np.inf if op == "argmin" else -np.inf, 3),
                           (np.inf if op == "argmin" else -np.inf, 2 ** 31 - 1), (best, 1)):
        kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op=op, init=init, init_key=init_key)
        ek, ev = oracle.reduce(host, main_op="to_kvp", reduce_op=op, init=init, init_key=init_key)
        assert np.array_equal(kv.keys.cpu().numpy().astype(np.int64), ek), (init, init_key)
        assert np.array_equal(kv.values.cpu().numpy().astype(np.float64), ev, equal_nan=True), (init, init_key)


def test_kvp_column_major_and_strided_refusal(cuda, oracle):
    t, host = device_synth((300, 40), np.float32, 8, "int", 0, 4, cuda)
    cm = as_layout(t, 1)
    kv = linalg.reduce(cm, linalg.ALONG_COLUMNS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
    ek, ev = oracle.reduce(host, apply=1, layout=1, main_op="to_kvp", reduce_op="argmin", init=np.inf)
    assert np.array_equal(kv.keys.cpu().numpy().astype(np.int64), ek)
    with pytest.raises(L.B2RError):  # key/value outputs along the strided axis: refused as in the reference
        linalg.reduce(t, linalg.ALONG_COLUMNS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))


@pytest.mark.parametrize("main,red", [("identity", "add"), ("abs", "add"), ("nz", "add"), ("identity", "min"),
                                      ("identity", "max"), ("abs", "min"), ("abs", "max"), ("sq", "add")])
@pytest.mark.parametrize("apply", [0, 1])
def test_operator_combinations(cuda, oracle, main, red, apply):
    t, host = device_synth((257, 131), np.float32, 3, "int", -3, 4, cuda)  # zeros and repeats
    init = {"add": 0.0, "min": float("inf"), "max": -float("inf")}[red]
    got = linalg.reduce(t, apply, init=init, main_op=main, reduce_op=red, final_op="mul_const", final_scalar=0.5)
    exp = oracle.reduce(host, apply=apply, main_op=main, reduce_op=red, init=init, final_op="mul_const",
                        final_scalar=0.5)
    assert np.array_equal(got.cpu().numpy().astype(np.float64), exp)  # small integers: exact in fp32
    ti, hi = device_synth((100, 77), np.int32, 4, "int", -1000, 1000, cuda)
    iinit = {"add": 0, "min": 2**31 - 1, "max": -2**31}[red]
    goti = linalg.reduce(ti, apply, init=iinit, main_op=main, reduce_op=red)
    expi = oracle.reduce(hi, apply=apply, main_op=main, reduce_op=red, init=iinit)
    assert np.array_equal(goti.cpu().numpy().astype(np.float64), expi)


def test_final_ops(cuda, oracle):
    t, host = device_synth((64, 96), np.float32, 6, "uniform", -2, 2, cuda)
    for fin, sc in [("identity", 1), ("sqrt", 1), ("mul_const", 0.25), ("div_const", 64.0), ("abs", 1)]:
        main = "sq" if fin == "sqrt" else "identity"
        for apply in (0, 1):
            got = linalg.reduce(t, apply, main_op=main, final_op=fin, final_scalar=sc)
            exp = oracle.reduce(host, apply=apply, main_op=main, final_op=fin, final_scalar=sc)
            oracle.assert_approx(exp, got.cpu().numpy(), 1e-5, fin)


def test_error_compensation(cuda, oracle):
    # cpp/tests/stats/sum.cu:58-75 pattern along both axes: (3v, -v*1e7, +v*1e7) triples
    rows, cols, v = 3 * 341, 96, 1.0
    m = np.full((rows, cols), v, dtype=np.float32)
    m[2::3] = v * 1e7
    m[1::3] = -v * 1e7
    m[0::3] = 3 * v
    t = torch.from_numpy(m).to(cuda)
    got = linalg.reduce(t, linalg.ALONG_COLUMNS)
    oracle.assert_approx(np.full(cols, rows * v), got.cpu().numpy(), 1e-5)
    got = linalg.reduce(t.t().contiguous(), linalg.ALONG_ROWS)
    oracle.assert_approx(np.full(cols, rows * v), got.cpu().numpy(), 1e-5)


@pytest.mark.parametrize("rows,cols", [(100000, 64), (65537, 128), (300001, 4), (20000, 1024), (9000, 36), (70000, 256)])
@pytest.mark.parametrize("main,red,fin", [("identity", "add", "identity"), ("sq", "add", "sqrt"), ("abs", "max", "identity")])
def test_strided_tma_staged(cuda, oracle, knobs, rows, cols, main, red, fin):
    # the TMA-staged column kernel (narrow contiguous matrices), forced on; same results as the
    # register-staged kernel and within tolerance of the oracle
    t, host = device_synth((rows, cols), np.float32, 17, "uniform", -1, 1, cuda)
    plain = linalg.reduce(t, linalg.ALONG_COLUMNS, main_op=main, reduce_op=red, final_op=fin)
    knobs(B2R_COL_TMA="1")
    staged = linalg.reduce(t, linalg.ALONG_COLUMNS, main_op=main, reduce_op=red, final_op=fin)
    ws = torch.empty(linalg.reduce_workspace_bytes(t, linalg.ALONG_COLUMNS, reduce_op=red), dtype=torch.uint8, device=cuda)
    staged_ws = linalg.reduce(t, linalg.ALONG_COLUMNS, main_op=main, reduce_op=red, final_op=fin, workspace=ws)
    exp = oracle.reduce(host, apply=1, main_op=main, reduce_op=red, final_op=fin)
    assert not torch.isnan(staged).any()
    oracle.assert_approx(exp, staged.cpu().numpy(), 1e-5, "tma vs oracle")
    oracle.assert_approx(plain.cpu().numpy(), staged.cpu().numpy(), 1e-6, "tma vs register-staged")
    assert torch.equal(staged, staged_ws)
    td, hd = device_synth((rows, min(cols, 512)), np.float64, 18, "uniform", -1, 1, cuda)
    got = linalg.reduce(td, linalg.ALONG_COLUMNS, main_op=main, reduce_op=red, final_op=fin)
    oracle.assert_approx(oracle.reduce(hd, apply=1, main_op=main, reduce_op=red, final_op=fin), got.cpu().numpy(), 1e-9)


@pytest.mark.parametrize("rows,cols,dt", [(5000, 300, np.float32), (4100, 132, np.float32), (20000, 1024, np.float32),
                                          (9000, 2052, np.float32), (70000, 256, np.float32), (6000, 130, np.float64),
                                          (12345, 1000, np.float64), (8192, 520, np.float16), (5000, 260, np.int32)])
@pytest.mark.parametrize("main,red,fin", [("identity", "add", "identity"), ("sq", "add", "sqrt"), ("abs", "max", "identity")])
def test_strided_tiled_tma(cuda, oracle, knobs, rows, cols, dt, main, red, fin):
    """The tiled-TMA kernel of wide matrices (cp.async.bulk.tensor.2d), forced onto small shapes: ragged last
    column block, ragged last box of a row range, 16 / 8 / 4 / 2-byte elements, every state type."""
    if dt == np.int32 and fin == "sqrt":
        pytest.skip("no root of an integer sum")
    knobs(B2R_COL_TMA2D_MB="1")
    kind, lo, hi = ("int", -3, 4) if dt == np.int32 else ("uniform", -1, 1)
    t, host = device_synth((rows, cols), dt, 23, kind, lo, hi, cuda)
    if rows * cols * t.element_size() < (1 << 20):
        pytest.skip("below the smallest size the knob can force")
    out_dt = torch.float32 if dt == np.float16 else None
    got = linalg.reduce(t, linalg.ALONG_COLUMNS, main_op=main, reduce_op=red, final_op=fin, out_dtype=out_dt)
    exp = oracle.reduce(host, apply=1, main_op=main, reduce_op=red, final_op=fin)
    oracle.assert_approx(exp, got.cpu().numpy(), 1e-9 if dt == np.float64 else 1e-5, "tiled TMA")
    knobs(B2R_COL_TMA="2")  # register-staged kernel: same partial layout, same answers
    ldg = linalg.reduce(t, linalg.ALONG_COLUMNS, main_op=main, reduce_op=red, final_op=fin, out_dtype=out_dt)
    oracle.assert_approx(ldg.cpu().numpy(), got.cpu().numpy(), 1e-12 if dt == np.float64 else 1e-6, "vs register-staged")
    if red == "max" or dt == np.int32:
        assert torch.equal(got, ldg)


def test_strided_tiled_tma_full_size(cuda):
    """300 000 x 1024 fp32 (1.2 GB, default policy): integer-valued data, so every column sum is exact."""
    t, host = device_synth((300000, 1024), np.float32, 31, "int", 0, 16, cuda)
    got = linalg.reduce(t, linalg.ALONG_COLUMNS)
    assert np.array_equal(got.cpu().numpy().astype(np.int64), host.sum(axis=0, dtype=np.int64))
    mean = linalg.reduce(t, linalg.ALONG_COLUMNS, final_op="div_const", final_scalar=300000.0)
    assert np.allclose(mean.cpu().numpy(), host.mean(axis=0, dtype=np.float64), rtol=1e-6, atol=0)


@pytest.mark.parametrize("rows,cols", [(100000, 128), (65537, 64), (300001, 4), (20001, 500), (16384, 36), (70000, 256),
                                       (50000, 96)])
def test_rows_tma_staged(cuda, oracle, knobs, rows, cols):
    # the TMA-staged row kernel (short contiguous rows), forced on: sums, norms and argmin
    t, host = device_synth((rows, cols), np.float32, 19, "int", -4, 5, cuda)
    knobs(B2R_ROW_TMA="1")
    got = linalg.reduce(t, linalg.ALONG_ROWS)
    assert np.array_equal(got.cpu().numpy().astype(np.float64), host.astype(np.float64).sum(1))
    got = linalg.norm(t, "L2", linalg.ALONG_ROWS, fin_op="sqrt")
    oracle.assert_approx(oracle.reduce(host, main_op="sq", final_op="sqrt"), got.cpu().numpy(), 1e-6)
    kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
    ek, ev = oracle.reduce(host, main_op="to_kvp", reduce_op="argmin", init=np.inf)
    assert np.array_equal(kv.keys.cpu().numpy().astype(np.int64), ek)
    assert np.array_equal(kv.values.cpu().numpy().astype(np.float64), ev)
    prev = got.clone()
    linalg.reduce(t, linalg.ALONG_ROWS, got, inplace=True, main_op="abs", reduce_op="max")
    assert np.array_equal(got.cpu().numpy(), np.maximum(prev.cpu().numpy(), np.abs(host).max(1)))
    tu, hu = device_synth((rows, cols), np.float32, 20, "uniform", -1, 1, cuda)
    got = linalg.reduce(tu, linalg.ALONG_ROWS)
    knobs(B2R_ROW_TMA=None)
    oracle.assert_approx(oracle.reduce(hu), got.cpu().numpy(), 1e-5)
    oracle.assert_approx(linalg.reduce(tu, linalg.ALONG_ROWS).cpu().numpy(), got.cpu().numpy(), 1e-6)


@pytest.mark.parametrize("rows,cols,dt", [(100003, 1, np.float32), (70001, 2, np.float32), (50002, 3, np.float32),
                                          (33333, 7, np.float32), (40001, 8 + 1, np.float32), (20001, 17, np.float32),
                                          (9999, 33, np.float32), (12346, 65, np.float32), (5003, 129, np.float32),
                                          (3001, 513, np.float32), (2002, 1001, np.float32), (1003, 1023, np.float32),
                                          (20001, 7, np.float64), (5001, 131, np.float64), (30003, 13, np.float16),
                                          (25001, 9, np.int32),
                                          # rows on 16-byte boundaries (staged when their length fits the lane groups badly)
                                          (30001, 8, np.float32), (20001, 36, np.float32), (10001, 96, np.float32),
                                          (7001, 100, np.float32), (3001, 400, np.float32), (2001, 784, np.float32),
                                          (1501, 1024, np.float32), (5001, 50, np.float64), (9001, 24, np.float16),
                                          (9001, 100, np.int32)])
@pytest.mark.parametrize("tile_kb", [None, "6"])
def test_rows_staged_odd_widths(cuda, oracle, knobs, rows, cols, dt, tile_kb):
    """Contiguous rows through the shared-memory staged kernel, forced onto small inputs: rows off 16-byte
    boundaries (element loads) and on them (16-byte loads, rotated starts); lane-per-row, four rows per lane,
    2..32 lanes per row; row counts that leave rows behind the last 16-byte boundary; default and tiny tiles
    (many tiles per CTA, every ring depth)."""
    if tile_kb is not None and cols * np.dtype(dt).itemsize * 8 > 6 * 1024:
        pytest.skip("eight rows do not fit the tiny tile")
    knobs(B2R_ROW_STAGED_MIN_KB="1", B2R_ROW_STAGED_WIDE_MIN_KB="1", B2R_ROW_STAGED_ALIGNED="2", B2R_ROW_STAGED_KB=tile_kb)
    t, host = device_synth((rows, cols), dt, 29, "uniform" if dt == np.float16 else "int", -4, 5, cuda)
    out_dt = torch.float32 if dt == np.float16 else None
    got = linalg.reduce(t, linalg.ALONG_ROWS, out_dtype=out_dt)
    if dt == np.float16:
        oracle.assert_approx(oracle.reduce(host), got.cpu().numpy(), 1e-5)
        return
    assert np.array_equal(got.cpu().numpy().astype(np.float64), host.astype(np.float64).sum(1))
    if dt == np.int32:
        return
    got = linalg.norm(t, "L2", linalg.ALONG_ROWS, fin_op="sqrt")
    oracle.assert_approx(oracle.reduce(host, main_op="sq", final_op="sqrt"), got.cpu().numpy(), 1e-6)
    kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
    ek, ev = oracle.reduce(host, main_op="to_kvp", reduce_op="argmin", init=np.inf)
    assert np.array_equal(kv.keys.cpu().numpy().astype(np.int64), ek)
    assert np.array_equal(kv.values.cpu().numpy().astype(np.float64), ev)
    if dt == np.float32:
        idx = torch.empty(rows, dtype=torch.int32, device=cuda)
        linalg.argmin(t, idx)
        assert np.array_equal(idx.cpu().numpy().astype(np.int64), ek)
    prev = got.clone()
    linalg.reduce(t, linalg.ALONG_ROWS, got, inplace=True, main_op="abs", reduce_op="max")
    assert np.array_equal(got.cpu().numpy(), np.maximum(prev.cpu().numpy(), np.abs(host).max(1)))
    # same bits as the direct kernels for a sum of uniform data (both carry fp32 sums in fp64)
    tu, hu = device_synth((rows, cols), dt, 30, "uniform", -1, 1, cuda)
    staged = linalg.reduce(tu, linalg.ALONG_ROWS, init=0.5)
    knobs(B2R_ROW_STAGED="2")
    direct = linalg.reduce(tu, linalg.ALONG_ROWS, init=0.5)
    oracle.assert_approx(oracle.reduce(hu, init=0.5), staged.cpu().numpy(), 1e-5 if dt == np.float32 else 1e-12)
    oracle.assert_approx(direct.cpu().numpy(), staged.cpu().numpy(), 1e-6 if dt == np.float32 else 1e-13)


def test_rows_staged_full_size(cuda):
    """40 000 003 x 7 fp32 (1.1 GB, default policy, three rows behind the last boundary): exact integer sums."""
    t, host = device_synth((40000003, 7), np.float32, 33, "int", 0, 16, cuda)
    got = linalg.reduce(t, linalg.ALONG_ROWS)
    assert np.array_equal(got.cpu().numpy().astype(np.int64), host.sum(axis=1, dtype=np.int64))


@pytest.mark.parametrize("rows,cols", [(0, 5), (5, 0), (1, 1), (1, 300), (300, 1), (2, 2)])
def test_degenerate_shapes(cuda, oracle, rows, cols):
    t = torch.full((rows, cols), 2.0, dtype=torch.float32, device=cuda)
    for apply in (0, 1):
        n_out = rows if apply == 0 else cols
        n_red = cols if apply == 0 else rows
        got = linalg.reduce(t, apply, init=0.0)
        assert got.shape == (n_out,)
        assert got.cpu().tolist() == [2.0 * n_red] * n_out


def test_exhaustive_small_widths(cuda, oracle):
    # every row length 1..300 against the oracle: exercises every lane-group size, the vector
    # and scalar paths and every tail
    for n_rows in (1, 2, 31, 33, 1000):
        for d in list(range(1, 70)) + [96, 127, 128, 129, 255, 256, 257, 300]:
            t, host = device_synth((n_rows, d), np.float32, 100 + d, "int", -8, 9, cuda)
            got = linalg.reduce(t, linalg.ALONG_ROWS)
            assert np.array_equal(got.cpu().numpy().astype(np.float64), host.astype(np.float64).sum(1)), (n_rows, d)
            got = linalg.reduce(t, linalg.ALONG_COLUMNS)
            assert np.array_equal(got.cpu().numpy().astype(np.float64), host.astype(np.float64).sum(0)), (n_rows, d)


def test_canary_outputs_not_overrun(cuda):
    # outputs sit inside a larger buffer filled with a canary; nothing outside may change
    for rows, cols, apply in [(1001, 67, 0), (1001, 67, 1), (9, 70001, 0), (70001, 9, 1)]:
        t = torch.ones((rows, cols), dtype=torch.float32, device=cuda)
        n_out = rows if apply == 0 else cols
        buf = torch.full((n_out + 64,), -777.0, dtype=torch.float32, device=cuda)
        linalg.reduce(t, apply, buf[32:32 + n_out])
        assert torch.all(buf[:32] == -777.0) and torch.all(buf[32 + n_out:] == -777.0)
        assert torch.all(buf[32:32 + n_out] == (cols if apply == 0 else rows))


def test_bad_arguments(cuda):
    t = torch.ones((4, 5), dtype=torch.float32, device=cuda)
    with pytest.raises(ValueError):  # RAFT_EXPECTS: output size (linalg/reduce.cuh:162-168)
        linalg.reduce(t, linalg.ALONG_ROWS, torch.empty(5, device=cuda))
    with pytest.raises(ValueError):  # RAFT_EXPECTS: contiguous input (linalg/reduce.cuh:157)
        linalg.reduce(torch.ones((8, 10), device=cuda)[::2, ::2], linalg.ALONG_ROWS)
    with pytest.raises(L.B2RError):
        linalg.reduce(t.to(torch.int64), linalg.ALONG_ROWS)
    lib = L.load()
    assert lib.b2r_reduce(None, None, None, None, 0, None) == L.ERR_BAD_ARG
    d = L.ReduceDesc(n_rows=-1, n_cols=3)
    assert lib.b2r_reduce(d, t.data_ptr(), t.data_ptr(), None, 0, None) == L.ERR_BAD_ARG
    d = L.ReduceDesc(n_rows=4, n_cols=5)
    assert lib.b2r_reduce(d, None, t.data_ptr(), None, 0, None) == L.ERR_BAD_ARG
    torch.cuda.synchronize()


def test_dependent_launches_change_no_result(cuda, knobs):
    """The hot kernels are launched with programmatic stream serialization (a kernel may be scheduled while its
    predecessor drains and waits for it before touching global memory). Back-to-back calls that feed one another,
    with the feature on and off (B2R_DEP_LAUNCH=2), must give the same bits."""
    a, _ = device_synth((200000, 64), np.float32, 3, "uniform", -1, 1, cuda)
    keys, _ = device_synth((200000,), np.int32, 4, "int", 0, 100, cuda)

    def chain():
        col = linalg.reduce(a, linalg.ALONG_COLUMNS)                       # two launches
        row = linalg.reduce(a, linalg.ALONG_ROWS, main_op="sq", final_op="sqrt")
        nrm = linalg.row_normalize(a, "L2")
        col2 = linalg.reduce(nrm, linalg.ALONG_COLUMNS)                    # reads what the previous call wrote
        byk = linalg.reduce_rows_by_key(nrm, keys, 100)                    # five launches
        tot = linalg.reduce(byk.reshape(1, -1), linalg.ALONG_ROWS)
        return [col, row, nrm, col2, byk, tot]

    on = [t.clone() for t in chain()]
    for _ in range(3):  # again, back to back, into fresh outputs
        again = chain()
    torch.cuda.synchronize(cuda)
    knobs(B2R_DEP_LAUNCH="2")
    off = chain()
    for x, y, z in zip(on, again, off):
        assert torch.equal(x, y)
        assert torch.equal(x, z)
