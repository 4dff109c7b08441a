"""b2r_column_sum_f32_noalloc - the entry point for callers that may not allocate - against
the regular b2r_reduce column path, through the C ABI. Collected last on purpose (file name),
so that a run stopping at the first failure has already run everything else; it also passes
when run alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

from raft_b200 import _lib as L
from raft_b200 import linalg

pytestmark = pytest.mark.gpu


def _noalloc(data, out, final_op=L.FINAL_IDENTITY, scalar=1.0):
    n_rows, n_cols = data.shape
    with torch.cuda.device(data.device):
        return L.load().b2r_column_sum_f32_noalloc(out.data_ptr(), data.data_ptr(), n_rows, n_cols, final_op, scalar,
                                                   torch.cuda.current_stream(data.device).cuda_stream)


@pytest.mark.parametrize("rows,cols", [(100000, 64), (4097, 130), (1, 7), (300000, 33), (50, 4096)])
def test_matches_regular_entry_point_twice_in_a_row(cuda, rows, cols):
    a = torch.empty((rows, cols), dtype=torch.float32, device=cuda)
    b = torch.empty((rows, cols), dtype=torch.float32, device=cuda)
    linalg.synth_fill(a, 71, "uniform", -1, 1)
    linalg.synth_fill(b, 72, "normal")
    for data in (a, b):  # two calls in a row share the library's scratch array
        expect = linalg.reduce(data, linalg.ALONG_COLUMNS)
        got = torch.full((cols,), float("nan"), dtype=torch.float32, device=cuda)
        assert _noalloc(data, got) == L.OK
        torch.cuda.synchronize()
        # same kernels, same launch shape, fixed summation order: identical bits; the parity
        # tolerance of the suite (1e-5, absolute or relative) is the stated bound
        e, g = expect.cpu().numpy().astype(np.float64), got.cpu().numpy().astype(np.float64)
        diff = np.abs(e - g)
        assert np.all((diff <= 1e-5) | (diff <= 1e-5 * np.maximum(np.abs(e), np.abs(g))))
        assert torch.equal(expect, got)
    mean = torch.empty(cols, dtype=torch.float32, device=cuda)
    assert _noalloc(a, mean, L.FINAL_DIV_CONST, float(rows)) == L.OK
    assert torch.equal(mean, linalg.reduce(a, linalg.ALONG_COLUMNS, final_op="div_const", final_scalar=float(rows)))


def _free_bytes():
    free, _ = torch.cuda.mem_get_info()
    return free


@pytest.mark.parametrize("rows,cols", [(100000, 1024), (20000, 1000), (300, 70000), (8192, 70000), (9000, 900)])
def test_shapes_whose_preferred_plan_exceeds_the_array(cuda, rows, cols):
    """b2r_reduce would use more than 1 MiB of scratch for these (a partial row per CTA of 148 x cols x 8
    bytes, or two row ranges of 70000 columns); the entry point plans a launch that fits its array, runs
    it twice in a row, takes no device memory, and agrees with b2r_reduce within the suite's tolerance."""
    data = torch.empty((rows, cols), dtype=torch.float32, device=cuda)
    linalg.synth_fill(data, 73, "uniform", -1, 1)
    expect = linalg.reduce(data, linalg.ALONG_COLUMNS).cpu().numpy().astype(np.float64)
    got = torch.full((cols,), float("nan"), dtype=torch.float32, device=cuda)
    assert _noalloc(data, got) == L.OK  # first call on the device may resolve the array's address
    torch.cuda.synchronize()
    before = _free_bytes()
    for _ in range(2):
        got.fill_(float("nan"))
        assert _noalloc(data, got) == L.OK
        torch.cuda.synchronize()
        g = got.cpu().numpy().astype(np.float64)
        diff = np.abs(expect - g)
        assert np.all((diff <= 1e-5) | (diff <= 1e-5 * np.maximum(np.abs(expect), np.abs(g))))
    assert _free_bytes() == before  # nothing was allocated on the device


def test_limit_and_bad_arguments(cuda, knobs):
    lib = L.load()
    assert lib.b2r_column_sum_f32_noalloc_max_scratch() == 1 << 20
    # a launch shape four times wider than the default would need 2368 row ranges x 128 columns of fp64
    # partials = 2.4 MB from b2r_reduce; the entry point fits its plan under the 1 MiB array instead
    tall = torch.ones((200000, 128), dtype=torch.float32, device=cuda)
    out = torch.full((128,), 5.0, dtype=torch.float32, device=cuda)
    knobs(B2R_COL_CPS="16", B2R_COL_TMA="2")
    assert linalg.reduce_workspace_bytes(tall, linalg.ALONG_COLUMNS) > (1 << 20)
    assert _noalloc(tall, out) == L.OK
    torch.cuda.synchronize()
    assert torch.all(out == 200000.0)
    knobs(B2R_COL_CPS=None, B2R_COL_TMA=None)
    out.fill_(5.0)
    assert _noalloc(tall, out) == L.OK
    assert torch.all(out == 200000.0)
    small = torch.ones((8, 8), dtype=torch.float32, device=cuda)
    assert lib.b2r_column_sum_f32_noalloc(None, small.data_ptr(), 8, 8, 0, 1.0, None) == L.ERR_BAD_ARG
    assert lib.b2r_column_sum_f32_noalloc(out.data_ptr(), small.data_ptr(), -1, 8, 0, 1.0, None) == L.ERR_BAD_ARG
    assert lib.b2r_column_sum_f32_noalloc(out.data_ptr(), small.data_ptr(), 8, 8, 99, 1.0, None) == L.ERR_BAD_ARG
    assert lib.b2r_column_sum_f32_noalloc(out.data_ptr(), small.data_ptr(), 8, 0, 0, 1.0, None) == L.OK
    torch.cuda.synchronize()
