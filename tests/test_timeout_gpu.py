"""The give-up path of every kernel that waits on shared-memory barriers, without a fault: a test hook
(B2R_TEST_SKIP_TILE) makes the producer of the first CTA never request one tile, so the consumers' wait
for it runs out with NO copy of that tile in flight; the wait limit is set to 30 ms for the test. Expected,
for every kernel: the call returns normally, b2r_last_kernel_status reports B2R_ERR_TIMEOUT, the
floating-point outputs the CTA did not finish are NaN, and the next call (hook off) is correct again."""
import numpy as np
import pytest
import torch

from raft_b200 import _lib as L
from raft_b200 import linalg

pytestmark = pytest.mark.gpu


def _fresh(cuda):
    assert linalg.last_kernel_status(cuda) in (L.OK, L.ERR_TIMEOUT)  # clears whatever an earlier test left
    assert linalg.last_kernel_status(cuda) == L.OK


def _expect_timeout_then_ok(cuda, knobs, forced, run, check_nan, check_ok):
    _fresh(cuda)
    knobs(B2R_TEST_SKIP_TILE="3", B2R_WAIT_LIMIT_MS="30", **forced)  # tile index 2 of CTA 0 never arrives
    out = run()
    assert linalg.last_kernel_status(cuda, clear=False) == L.ERR_TIMEOUT
    assert linalg.last_kernel_status(cuda) == L.ERR_TIMEOUT  # still set; this read clears it
    assert linalg.last_kernel_status(cuda) == L.OK
    check_nan(out)
    knobs(B2R_TEST_SKIP_TILE=None, B2R_WAIT_LIMIT_MS=None)
    out = run()
    assert linalg.last_kernel_status(cuda) == L.OK
    check_ok(out)


def test_column_reduction_ring(cuda, knobs):
    t = torch.ones((100000, 64), dtype=torch.float32, device=cuda)
    _expect_timeout_then_ok(cuda, knobs, {}, lambda: linalg.reduce(t, linalg.ALONG_COLUMNS),
                            lambda o: torch.isnan(o).all().item() or pytest.fail("column sums not NaN"),
                            lambda o: torch.all(o == 100000.0).item() or pytest.fail("column sums wrong"))


def test_wide_column_reduction_tiled_tma(cuda, knobs):
    t = torch.ones((20000, 2048), dtype=torch.float32, device=cuda)
    _expect_timeout_then_ok(cuda, knobs, {"B2R_COL_TMA2D_MB": "64"}, lambda: linalg.reduce(t, linalg.ALONG_COLUMNS),
                            lambda o: torch.isnan(o[:128]).all().item() or pytest.fail("column sums not NaN"),
                            lambda o: torch.all(o == 20000.0).item() or pytest.fail("column sums wrong"))


def test_row_ring(cuda, knobs):
    t = torch.ones((100000, 64), dtype=torch.float32, device=cuda)
    _expect_timeout_then_ok(cuda, knobs, {"B2R_ROW_TMA": "1"}, lambda: linalg.reduce(t, linalg.ALONG_ROWS),
                            lambda o: (torch.isnan(o).any().item() and not torch.isnan(o[-1000:]).any().item())
                            or pytest.fail("unfinished rows not NaN"),
                            lambda o: torch.all(o == 64.0).item() or pytest.fail("row sums wrong"))


def test_row_ring_key_value_output_reports_through_the_status(cuda, knobs):
    t = torch.ones((100000, 64), dtype=torch.float32, device=cuda)
    run = lambda: linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
    _expect_timeout_then_ok(cuda, knobs, {"B2R_ROW_TMA": "1"}, run, lambda o: None,
                            lambda o: (torch.all(o.keys == 0).item() and torch.all(o.values == 1.0).item())
                            or pytest.fail("argmin wrong"))


def test_split_row_ring(cuda, knobs):
    t = torch.ones((2, 1 << 22), dtype=torch.float32, device=cuda)
    _expect_timeout_then_ok(cuda, knobs, {"B2R_ROW_SPLIT_RING_MB": "1"}, lambda: linalg.reduce(t, linalg.ALONG_ROWS),
                            lambda o: (torch.isnan(o[0]).item() and not torch.isnan(o[1]).item())
                            or pytest.fail("unfinished row not NaN"),
                            lambda o: torch.all(o == float(1 << 22)).item() or pytest.fail("row sums wrong"))


def test_staged_rows_off_16_byte_boundaries(cuda, knobs):
    t = torch.ones((400000, 31), dtype=torch.float32, device=cuda)
    _expect_timeout_then_ok(cuda, knobs, {"B2R_ROW_STAGED_MIN_KB": "1024"}, lambda: linalg.reduce(t, linalg.ALONG_ROWS),
                            lambda o: torch.isnan(o).any().item() or pytest.fail("unfinished rows not NaN"),
                            lambda o: torch.all(o == 31.0).item() or pytest.fail("row sums wrong"))


def test_staged_row_normalize(cuda, knobs):
    t = torch.ones((400000, 31), dtype=torch.float32, device=cuda)
    want = 1.0 / np.sqrt(31.0)
    _expect_timeout_then_ok(cuda, knobs, {"B2R_ROW_STAGED_MIN_KB": "1024"}, lambda: linalg.row_normalize(t, "L2"),
                            lambda o: torch.isnan(o).any().item() or pytest.fail("unfinished rows not NaN"),
                            lambda o: torch.allclose(o, torch.full_like(o, want), rtol=1e-6)
                            or pytest.fail("normalised rows wrong"))


def test_keyed_column_sums_ring(cuda, knobs):
    t = torch.ones((512, 32768), dtype=torch.float32, device=cuda)
    keys = (torch.arange(32768, device=cuda, dtype=torch.int32) % 16).contiguous()
    _expect_timeout_then_ok(cuda, knobs, {"B2R_COLKEY_ALGO": "2"}, lambda: linalg.reduce_cols_by_key(t, keys, nkeys=16),
                            lambda o: torch.isnan(o).any().item() or pytest.fail("unfinished sums not NaN"),
                            lambda o: torch.all(o == 2048.0).item() or pytest.fail("keyed column sums wrong"))


def test_keyed_column_sums_walk_ring(cuda, knobs):
    t = torch.ones((512, 32768), dtype=torch.float32, device=cuda)
    keys = (torch.arange(32768, device=cuda, dtype=torch.int32) % 16).contiguous()
    _expect_timeout_then_ok(cuda, knobs, {"B2R_COLKEY_ALGO": "3"}, lambda: linalg.reduce_cols_by_key(t, keys, nkeys=16),
                            lambda o: torch.isnan(o).any().item() or pytest.fail("unfinished sums not NaN"),
                            lambda o: torch.all(o == 2048.0).item() or pytest.fail("keyed column sums wrong"))


def test_keyed_column_sums_table_ring(cuda, knobs):
    t = torch.ones((512, 32768), dtype=torch.float32, device=cuda)
    keys = (torch.arange(32768, device=cuda, dtype=torch.int32) % 100).contiguous()
    want = torch.bincount(keys.long(), minlength=100).to(torch.float32)
    _expect_timeout_then_ok(cuda, knobs, {"B2R_COLKEY_ALGO": "4"}, lambda: linalg.reduce_cols_by_key(t, keys, nkeys=100),
                            lambda o: torch.isnan(o).any().item() or pytest.fail("unfinished sums not NaN"),
                            lambda o: torch.all(o == want[None, :]).item() or pytest.fail("keyed column sums wrong"))


def test_wait_limit_setter_and_status_string(cuda):
    lib = L.load()
    assert lib.b2r_set_wait_limit_ms(250) == L.OK
    assert lib.b2r_set_wait_limit_ms(0) == L.OK
    assert lib.b2r_last_kernel_status(None, 0) == L.ERR_BAD_ARG
    assert lib.b2r_status_string(L.ERR_TIMEOUT).decode().startswith("a bounded wait")
