"""ctypes wrapper of oracle/_ref/libraft_ref.so - the reference's own raft::linalg kernels built
for sm_100a by oracle/build_ref.sh. TEST INFRASTRUCTURE: used by tests/ (to validate the CPU
oracle and the product against the real reference on identical device inputs) and by
bench.py's reference arm. Works on torch CUDA tensors."""
import ctypes
import os

import torch

from raft_b200 import _lib as L

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libraft_ref.so")
_lib = None


def available():
    return os.path.exists(LIB_PATH)


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        for name in ("ref_reduce_contiguous", "ref_reduce_strided", "ref_reduce_kvp"):
            getattr(lib, name).argtypes = [ctypes.POINTER(L.ReduceDesc), vp, vp, vp]
        lib.ref_rows_by_key.argtypes = [vp, vp, i64, vp, vp, i32, i64, i64, i64, i32, vp]
        lib.ref_cols_by_key.argtypes = [vp, vp, vp, i32, i64, i64, i64, i32, vp]
        lib.ref_map_then_sum_reduce.argtypes = [vp, vp, i32, i64, vp]
        lib.ref_map_reduce_minmax.argtypes = [vp, vp, i64, i32, ctypes.c_float, vp]
        lib.ref_row_normalize.argtypes = [vp, vp, i32, i64, i64, i32, vp]
        _lib = lib
    return _lib


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def reduce(data, apply, dots, layout=L.ROW_MAJOR, main_op=L.MAIN_IDENTITY, reduce_op=L.REDUCE_ADD,
           final_op=L.FINAL_IDENTITY, final_scalar=1.0, init=0.0, init_key=0, inplace=False, out_dtype=None):
    """Runs the reference's raft::linalg::reduce. `data` is the logical [n_rows, n_cols] tensor
    (row- or column-major memory per `layout`); `dots` a tensor or a linalg.KeyValueVector.
    Returns the library status (0 ok, 2 combination not built into the wrapper)."""
    from raft_b200.linalg import _DTYPES, _KVP_OF, KeyValueVector
    n_rows, n_cols = data.shape
    in_dt = _DTYPES[data.dtype]
    kvp = isinstance(dots, KeyValueVector)
    out_dt = _KVP_OF[in_dt] if kvp else _DTYPES[dots.dtype]
    desc = L.ReduceDesc(in_dtype=in_dt, out_dtype=out_dt, layout=layout, apply=apply, n_rows=n_rows, n_cols=n_cols,
                        main_op=main_op, reduce_op=reduce_op, final_op=final_op, inplace=1 if inplace else 0,
                        init=float(init), init_i=0, init_key=int(init_key), final_scalar=float(final_scalar))
    lib = load()
    contiguous = (layout == L.ROW_MAJOR) == (apply == L.ALONG_ROWS)
    fn = lib.ref_reduce_kvp if kvp else (lib.ref_reduce_contiguous if contiguous else lib.ref_reduce_strided)
    with torch.cuda.device(data.device):
        return fn(desc, dots.data_ptr(), data.data_ptr(), _stream(data.device))


def rows_by_key(sums, A, keys, nkeys, weights=None, reset=True):
    from raft_b200.linalg import _DTYPES
    nrows, ncols = A.shape
    with torch.cuda.device(A.device):
        return load().ref_rows_by_key(sums.data_ptr(), A.data_ptr(), A.stride(0), keys.data_ptr(),
                                      weights.data_ptr() if weights is not None else None, _DTYPES[A.dtype], nrows,
                                      ncols, nkeys, 1 if reset else 0, _stream(A.device))


def cols_by_key(out, data, keys, nkeys, reset=True):
    from raft_b200.linalg import _DTYPES
    nrows, ncols = data.shape
    with torch.cuda.device(data.device):
        return load().ref_cols_by_key(out.data_ptr(), data.data_ptr(), keys.data_ptr(), _DTYPES[data.dtype], nrows,
                                      ncols, nkeys, 1 if reset else 0, _stream(data.device))


def row_normalize(out, data, norm_type):
    """The reference's raft::linalg::row_normalize<norm_type> (default eps). norm_type: "L1", "L2", "Linf"."""
    from raft_b200.linalg import _DTYPES, _NORM
    n_rows, n_cols = data.shape
    with torch.cuda.device(data.device):
        return load().ref_row_normalize(out.data_ptr(), data.data_ptr(), _DTYPES[data.dtype], n_rows, n_cols,
                                        _NORM[norm_type], _stream(data.device))


def map_then_sum_reduce(out, data):
    """The reference's mapThenSumReduce(out, len, identity_op, stream, data)."""
    from raft_b200.linalg import _DTYPES
    with torch.cuda.device(data.device):
        return load().ref_map_then_sum_reduce(out.data_ptr(), data.data_ptr(), _DTYPES[data.dtype], data.numel(),
                                              _stream(data.device))


def map_reduce_minmax(out, data, reduce_op, neutral):
    """The reference's map_reduce with identity_op and cuda::minimum ("min") / cuda::maximum ("max"), float."""
    with torch.cuda.device(data.device):
        return load().ref_map_reduce_minmax(out.data_ptr(), data.data_ptr(), data.numel(),
                                            L.REDUCE_MIN if reduce_op == "min" else L.REDUCE_MAX, float(neutral),
                                            _stream(data.device))
