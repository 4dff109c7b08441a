"""The five benchmark configurations at FULL size on the device: a seeded sample of the
outputs is checked against the fp64 oracle, and size-independent properties cover the rest
(sum of sums, linearity, idempotence of argmin, counts adding up)."""
import numpy as np
import pytest
import torch

from raft_b200 import linalg

pytestmark = pytest.mark.gpu

TOL = 1e-5  # fp32 sums and norms against the fp64 oracle, the reference's abs-or-rel rule


def _rows_on_host(t, idx):
    return t[torch.as_tensor(idx, device=t.device)].cpu().numpy()


def test_c1_row_sum_4096x1024(cuda, oracle):
    t = torch.empty((4096, 1024), dtype=torch.float32, device=cuda)
    linalg.synth_fill(t, 0, "uniform", -1, 1)
    got = linalg.coalesced_reduction(t).cpu().numpy()
    host = t.cpu().numpy()
    assert np.array_equal(host, oracle.synth((4096, 1024), np.float32, 0, "uniform", -1, 1))
    oracle.assert_approx(oracle.reduce(host), got, TOL)


def test_c2_row_l2_norms_1Mx128(cuda, oracle):
    n, d = 1_000_000, 128
    t = torch.empty((n, d), dtype=torch.float32, device=cuda)
    linalg.synth_fill(t, 1, "normal")
    sq = linalg.norm(t, "L2", linalg.ALONG_ROWS)
    rt = linalg.norm(t, "L2", linalg.ALONG_ROWS, fin_op="sqrt")
    idx = np.random.default_rng(0).choice(n, 20000, replace=False)
    idx = np.concatenate([idx, [0, 1, n - 2, n - 1]])
    sample = _rows_on_host(t, idx)
    oracle.assert_approx(oracle.reduce(sample, main_op="sq"), sq.cpu().numpy()[idx], TOL)
    oracle.assert_approx(oracle.reduce(sample, main_op="sq", final_op="sqrt"), rt.cpu().numpy()[idx], TOL)
    # properties over ALL rows: root of the squared norm; total energy equals the column-wise total
    assert torch.allclose(rt, sq.sqrt(), rtol=1e-6, atol=0)
    col = linalg.norm(t, "L2", linalg.ALONG_COLUMNS, out_dtype=torch.float32)
    assert abs(sq.double().sum().item() - col.double().sum().item()) <= 1e-6 * sq.double().sum().item()


def test_c3_col_sum_and_mean_16Mx64(cuda, oracle):
    n, d = 16_777_216, 64
    t = torch.empty((n, d), dtype=torch.float32, device=cuda)
    linalg.synth_fill(t, 2, "uniform", 0, 1)
    s = linalg.strided_reduction(t)
    m = linalg.strided_reduction(t, final_op="div_const", final_scalar=float(n))
    # oracle on the whole matrix, streamed through the host in slabs (fp64 partial sums add exactly enough)
    exp = np.zeros(d, dtype=np.float64)
    slab = 1 << 20
    for r0 in range(0, n, slab):
        exp += oracle.reduce(t[r0:r0 + slab].cpu().numpy(), apply=1)
    oracle.assert_approx(exp, s.cpu().numpy(), TOL)
    oracle.assert_approx(exp / n, m.cpu().numpy(), TOL)
    # repeated call gives the same bits (no atomics anywhere in the column path)
    assert torch.equal(s, linalg.strided_reduction(t))


def test_c4_row_argmin_8Mx64(cuda, oracle):
    n, d = 8_388_608, 64
    t = torch.empty((n, d), dtype=torch.float32, device=cuda)
    linalg.synth_fill(t, 3, "int", 0, 16)
    kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op="argmin", init=float("inf"))
    keys, vals = kv.keys, kv.values
    # every row, on the device, against an independent formulation: value = row minimum, key = first position of it
    rmin = t.min(dim=1).values
    assert torch.equal(vals, rmin)
    first = (t == rmin[:, None]).to(torch.int8).argmax(dim=1).to(torch.int32)
    assert torch.equal(keys, first)
    idx = np.random.default_rng(1).choice(n, 50000, replace=False)
    ek, ev = oracle.reduce(_rows_on_host(t, idx), main_op="to_kvp", reduce_op="argmin", init=np.inf)
    assert np.array_equal(keys.cpu().numpy()[idx].astype(np.int64), ek)
    assert np.array_equal(vals.cpu().numpy()[idx].astype(np.float64), ev)


def test_c5_keyed_row_sum_10Mx128(cuda, oracle):
    n, d, nkeys = 10_000_000, 128, 1024
    t = torch.empty((n, d), dtype=torch.float32, device=cuda)
    keys = torch.empty((n,), dtype=torch.int32, device=cuda)
    linalg.synth_fill(t, 4, "normal")
    linalg.synth_fill(keys, 5, "int", 0, nkeys)
    counts = torch.empty(nkeys, dtype=torch.int64, device=cuda)
    sums = linalg.reduce_rows_by_key(t, keys, nkeys, counts=counts)
    assert counts.sum().item() == n
    assert torch.equal(counts, torch.bincount(keys.long(), minlength=nkeys))
    # the oracle over ALL rows for a subset of keys (rows gathered on the device first)
    hk = keys.cpu().numpy()
    pick = np.array([0, 1, 511, 1023, 77, 300])
    for k in pick:
        rows = np.nonzero(hk == k)[0]
        sample = _rows_on_host(t, rows)
        exp = oracle.reduce(sample, apply=1)
        oracle.assert_approx(exp, sums[k].cpu().numpy(), TOL, f"key {k}")
    # property over all keys: the key sums add up to the column sums of the whole matrix
    col = linalg.strided_reduction(t).double()
    tot = sums.double().sum(dim=0)
    assert torch.allclose(tot, col, rtol=0, atol=2e-3)
