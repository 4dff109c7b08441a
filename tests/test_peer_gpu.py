"""The one-kernel all-reduce over peer memory (b2r_peer_allreduce_sum) on ONE GPU, through the C ABI:
a single-rank exchange, a two-rank exchange emulated by running the two ranks' kernels one after the
other (kernels that wait on one another must not share a GPU, so the first one is given a short limit
and is EXPECTED to report a timeout: its partner has not run yet - a wait that runs out because
nothing sets the flag, no fault), and the argument checks. The real multi-GPU run is tests/mg_check.py."""
import ctypes

import pytest
import torch

from raft_b200 import _lib as L

pytestmark = pytest.mark.gpu


def _area(lib, world, rank, payload):
    a = ctypes.c_void_p()
    assert lib.b2r_peer_area_create(world, rank, payload, ctypes.byref(a)) == L.OK
    return a


def _call(lib, area, sums, counts, scale=1.0):
    return lib.b2r_peer_allreduce_sum(area, sums.data_ptr() if sums is not None else None,
                                      sums.numel() if sums is not None else 0,
                                      counts.data_ptr() if counts is not None else None,
                                      counts.numel() if counts is not None else 0, scale,
                                      torch.cuda.current_stream().cuda_stream)


def _status(lib, area, clear=1):
    torch.cuda.synchronize()
    out = ctypes.c_int32(-1)
    assert lib.b2r_peer_area_status(area, ctypes.byref(out), clear) == L.OK
    return out.value


@pytest.mark.parametrize("n_f32,n_i64", [(64, 0), (131072, 1024), (7, 3), (0, 5), (1001, 0)])
def test_single_rank_exchange_is_the_identity_times_scale(cuda, n_f32, n_i64):
    lib = L.load()
    a = _area(lib, 1, 0, n_f32 * 4 + n_i64 * 8 + 32)
    sums = torch.randn(n_f32, device=cuda) if n_f32 else None
    counts = torch.randint(0, 1 << 40, (n_i64,), dtype=torch.int64, device=cuda) if n_i64 else None
    e_s = sums.clone() * 0.5 if n_f32 else None
    e_c = counts.clone() if n_i64 else None
    for _ in range(3):  # both data sets and the flag sequence
        if n_f32:
            sums.copy_(e_s * 2)
        assert _call(lib, a, sums, counts, 0.5) == L.OK
        assert _status(lib, a) == L.OK
        if n_f32:
            assert torch.equal(sums, e_s)
        if n_i64:
            assert torch.equal(counts, e_c)
    assert lib.b2r_peer_area_destroy(a) == L.OK


@pytest.mark.parametrize("n_f32,n_i64", [(5000, 33), (64, 0), (100, 7)])  # flagged chunks; tagged words
def test_two_ranks_one_after_the_other_and_the_wait_that_runs_out(cuda, n_f32, n_i64):
    lib = L.load()
    a0, a1 = _area(lib, 2, 0, n_f32 * 4 + n_i64 * 8 + 32), _area(lib, 2, 1, n_f32 * 4 + n_i64 * 8 + 32)
    assert lib.b2r_peer_area_link(a0, 1, a1) == L.OK and lib.b2r_peer_area_link(a1, 0, a0) == L.OK
    assert lib.b2r_peer_area_set_wait_limit_ms(a0, 20) == L.OK
    s0, s1 = torch.randn(n_f32, device=cuda), torch.randn(n_f32, device=cuda)
    c0 = torch.arange(n_i64, dtype=torch.int64, device=cuda)
    c1 = torch.full((n_i64,), 1 << 33, dtype=torch.int64, device=cuda)
    want_s, want_c = s0 + s1, c0 + c1
    keep0 = s0.clone()
    # rank 0 delivers its partial everywhere, then waits for rank 1's flag, which nothing sets: after 20 ms it
    # gives up, leaves its outputs as they were and records the timeout
    assert _call(lib, a0, s0, c0) == L.OK
    assert _status(lib, a0) == L.ERR_TIMEOUT
    assert torch.equal(s0, keep0)
    assert _status(lib, a0) == L.OK  # cleared
    # rank 1 runs afterwards: rank 0's partial and flag are already in its area, so it finishes at once
    assert _call(lib, a1, s1, c1) == L.OK
    assert _status(lib, a1) == L.OK
    assert torch.equal(s1, want_s) and torch.equal(c1, want_c)
    assert lib.b2r_peer_area_destroy(a0) == L.OK and lib.b2r_peer_area_destroy(a1) == L.OK


def test_argument_checks(cuda):
    lib = L.load()
    bad = ctypes.c_void_p()
    assert lib.b2r_peer_area_create(0, 0, 64, ctypes.byref(bad)) == L.ERR_BAD_ARG
    assert lib.b2r_peer_area_create(2, 2, 64, ctypes.byref(bad)) == L.ERR_BAD_ARG
    assert lib.b2r_peer_area_create(17, 0, 64, ctypes.byref(bad)) == L.ERR_BAD_ARG
    a = _area(lib, 2, 0, 256)
    x = torch.zeros(1024, device=cuda)
    assert _call(lib, a, x, None) == L.ERR_TOO_LARGE      # 4 KB payload, 256-byte slots
    assert _call(lib, a, x[:8], None) == L.ERR_BAD_ARG    # rank 1 was never opened or linked
    assert lib.b2r_peer_area_set_wait_limit_ms(a, 0) == L.ERR_BAD_ARG
    assert lib.b2r_peer_area_destroy(a) == L.OK
    assert lib.b2r_status_string(L.ERR_TIMEOUT).decode().startswith("a bounded wait")
