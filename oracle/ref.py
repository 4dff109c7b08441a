"""ctypes wrapper of oracle/_ref/libraft_ref.so - the reference's own raft::linalg kernels built
for sm_100a by oracle/build_ref.sh. TEST INFRASTRUCTURE: used by tests/ (to validate the CPU
oracle and the product against the real reference on identical device inputs) and by
bench.py's reference arm. Works on torch CUDA tensors."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libraft_ref.so")
_lib = None


class _Abi:
    """The enums and the descriptor the wrapper shares with the product's C ABI (include/raft_b200.h),
    restated here so that this module - and the benchmark's reference arm - never imports the product."""
    F32, F64, F16, I32, I64, I16, U32 = 0, 1, 2, 3, 4, 5, 6
    KVP_I32_F32, KVP_I32_F64, KVP_I32_I16, KVP_I32_I32 = 16, 17, 18, 19
    ROW_MAJOR, COL_MAJOR = 0, 1
    ALONG_ROWS, ALONG_COLUMNS = 0, 1
    MAIN_IDENTITY, MAIN_SQ, MAIN_ABS, MAIN_NZ, MAIN_TO_KVP = 0, 1, 2, 3, 4
    REDUCE_ADD, REDUCE_MIN, REDUCE_MAX, REDUCE_ARGMIN, REDUCE_ARGMAX = 0, 1, 2, 3, 4
    FINAL_IDENTITY, FINAL_SQRT, FINAL_MUL_CONST, FINAL_DIV_CONST, FINAL_ABS = 0, 1, 2, 3, 4

    class ReduceDesc(ctypes.Structure):
        _fields_ = [("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32), ("layout", ctypes.c_int32),
                    ("apply", ctypes.c_int32), ("n_rows", ctypes.c_int64), ("n_cols", ctypes.c_int64),
                    ("main_op", ctypes.c_int32), ("reduce_op", ctypes.c_int32), ("final_op", ctypes.c_int32),
                    ("inplace", ctypes.c_int32), ("init", ctypes.c_double), ("init_i", ctypes.c_int64),
                    ("init_key", ctypes.c_int64), ("final_scalar", ctypes.c_double)]


L = _Abi
_DTYPES = {torch.float32: L.F32, torch.float64: L.F64, torch.float16: L.F16, torch.int32: L.I32,
           torch.int64: L.I64, torch.int16: L.I16}
_KVP_OF = {L.F32: L.KVP_I32_F32, L.F64: L.KVP_I32_F64, L.I16: L.KVP_I32_I16, L.I32: L.KVP_I32_I32}
_NORM = {"L1": 1, "L2": 2, "Linf": 3}


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
           final_op=L.FINAL_IDENTITY, final_scalar=1.0, init=0.0, init_key=0, inplace=False, out_dtype=None,
           kvp=None):
    """Runs the reference's raft::linalg::reduce. `data` is the logical [n_rows, n_cols] tensor
    (row- or column-major memory per `layout`); `dots` a tensor, or for key/value output anything
    with a data_ptr() over an array of {int32 key, value} pairs (a linalg.KeyValueVector; with
    kvp=True a plain tensor of that many bytes). Returns the library status (0 ok, 2 combination
    not built into the wrapper)."""
    n_rows, n_cols = data.shape
    in_dt = _DTYPES[data.dtype]
    if kvp is None:
        kvp = not isinstance(dots, torch.Tensor)
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
    nrows, ncols = A.shape
    with torch.cuda.device(A.device):
        return load().ref_rows_by_key(sums.data_ptr(), A.data_ptr(), A.stride(0), keys.data_ptr(),
                                      weights.data_ptr() if weights is not None else None, _DTYPES[A.dtype], nrows,
                                      ncols, nkeys, 1 if reset else 0, _stream(A.device))


def cols_by_key(out, data, keys, nkeys, reset=True):
    nrows, ncols = data.shape
    with torch.cuda.device(data.device):
        return load().ref_cols_by_key(out.data_ptr(), data.data_ptr(), keys.data_ptr(), _DTYPES[data.dtype], nrows,
                                      ncols, nkeys, 1 if reset else 0, _stream(data.device))


def row_normalize(out, data, norm_type):
    """The reference's raft::linalg::row_normalize<norm_type> (default eps). norm_type: "L1", "L2", "Linf"."""
    n_rows, n_cols = data.shape
    with torch.cuda.device(data.device):
        return load().ref_row_normalize(out.data_ptr(), data.data_ptr(), _DTYPES[data.dtype], n_rows, n_cols,
                                        _NORM[norm_type], _stream(data.device))


def map_then_sum_reduce(out, data):
    """The reference's mapThenSumReduce(out, len, identity_op, stream, data)."""
    with torch.cuda.device(data.device):
        return load().ref_map_then_sum_reduce(out.data_ptr(), data.data_ptr(), _DTYPES[data.dtype], data.numel(),
                                              _stream(data.device))


def map_reduce_minmax(out, data, reduce_op, neutral):
    """The reference's map_reduce with identity_op and cuda::minimum ("min") / cuda::maximum ("max"), float."""
    with torch.cuda.device(data.device):
        return load().ref_map_reduce_minmax(out.data_ptr(), data.data_ptr(), data.numel(),
                                            L.REDUCE_MIN if reduce_op == "min" else L.REDUCE_MAX, float(neutral),
                                            _stream(data.device))
