"""b2r_matrix_argmin / b2r_matrix_argmax (raft::matrix::argmin / argmax) through the C ABI: the
reference's known-answer matrices and seeded grids against the oracle, bit exact."""
import numpy as np
import pytest
import torch

from raft_b200 import _lib as L
from raft_b200 import linalg
from util import device_synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", [torch.float32, torch.float64])
def test_known_answer_matrices(cuda, dt):
    # cpp/tests/matrix/argmin.cu:71-75 -> {0, 3, 3}; cpp/tests/matrix/argmax.cu:71-72 -> {3, 0, 2}
    m = torch.tensor([0.1, 0.2, 0.3, 0.4, 0.4, 0.3, 0.2, 0.1, 0.2, 0.3, 0.5, 0.0], dtype=dt, device=cuda).reshape(3, 4)
    assert linalg.argmin(m).tolist() == [0, 3, 3]
    assert linalg.argmax(m).tolist() == [3, 0, 2]
    assert linalg.argmin(m, index_dtype=torch.int64).tolist() == [0, 3, 3]


# shapes of cpp/bench/prims/matrix/argmin.cu:55-60 (scaled down) plus ragged ones
@pytest.mark.parametrize("rows,cols", [(1000, 64), (1000, 128), (1000, 256), (1000, 512), (1000, 1024), (100000, 64),
                                       (11, 7), (1234, 33), (3, 100000), (1, 1)])
@pytest.mark.parametrize("in_dt", [np.float32, np.float64])
def test_grid_against_oracle(cuda, oracle, rows, cols, in_dt):
    t, host = device_synth((rows, cols), in_dt, 3, "int", 0, 16, cuda)  # frequent ties
    for name, fn, init in (("argmin", linalg.argmin, np.inf), ("argmax", linalg.argmax, -np.inf)):
        got = fn(t)
        ek, _ = oracle.reduce(host, main_op="to_kvp", reduce_op=name, init=init)
        assert np.array_equal(got.cpu().numpy().astype(np.int64), ek), name
        kv = linalg.reduce(t, linalg.ALONG_ROWS, main_op="to_kvp", reduce_op=name, init=init)
        assert torch.equal(kv.keys, got)  # same kernels, key part only


def test_errors(cuda):
    t = torch.ones((4, 5), device=cuda)
    with pytest.raises(ValueError):
        linalg.argmin(t, out=torch.empty(5, dtype=torch.int32, device=cuda))
    with pytest.raises(ValueError):
        linalg.argmin(t.t())
    with pytest.raises(L.B2RError):
        linalg.argmin(t.to(torch.float16))
