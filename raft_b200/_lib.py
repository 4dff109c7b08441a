"""ctypes binding of the C ABI declared in include/raft_b200.h.

The shared library is built in-tree (``make -C raft_b200/csrc`` or ``__graft_entry__.build()``).
There is no fallback: if it is missing, loading raises with the build command.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libraft_b200.so")

# b2r_status
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TOO_LARGE, ERR_TIMEOUT = 0, 1, 2, 3, 4, 5
# b2r_dtype
F32, F64, F16, I32, I64, I16, U32 = 0, 1, 2, 3, 4, 5, 6
KVP_I32_F32, KVP_I32_F64, KVP_I32_I16, KVP_I32_I32 = 16, 17, 18, 19
# b2r_layout / b2r_apply
ROW_MAJOR, COL_MAJOR = 0, 1
ALONG_ROWS, ALONG_COLUMNS = 0, 1
# b2r_main_op / b2r_reduce_op / b2r_final_op / b2r_norm_type
MAIN_IDENTITY, MAIN_SQ, MAIN_ABS, MAIN_NZ, MAIN_TO_KVP = 0, 1, 2, 3, 4
REDUCE_ADD, REDUCE_MIN, REDUCE_MAX, REDUCE_ARGMIN, REDUCE_ARGMAX = 0, 1, 2, 3, 4
FINAL_IDENTITY, FINAL_SQRT, FINAL_MUL_CONST, FINAL_DIV_CONST, FINAL_ABS = 0, 1, 2, 3, 4
NORM_L0, NORM_L1, NORM_L2, NORM_LINF = 0, 1, 2, 3


class ReduceDesc(ctypes.Structure):
    """b2r_reduce_desc"""
    _fields_ = [
        ("in_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("layout", ctypes.c_int32),
        ("apply", ctypes.c_int32),
        ("n_rows", ctypes.c_int64),
        ("n_cols", ctypes.c_int64),
        ("main_op", ctypes.c_int32),
        ("reduce_op", ctypes.c_int32),
        ("final_op", ctypes.c_int32),
        ("inplace", ctypes.c_int32),
        ("init", ctypes.c_double),
        ("init_i", ctypes.c_int64),
        ("init_key", ctypes.c_int64),
        ("final_scalar", ctypes.c_double),
    ]


# every symbol include/raft_b200.h declares: name -> (restype, argtypes)
_vp, _i32, _i64, _sz, _dbl, _u64 = (ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t,
                                    ctypes.c_double, ctypes.c_uint64)
SIGNATURES = {
    "b2r_reduce": (ctypes.c_int, [ctypes.POINTER(ReduceDesc), _vp, _vp, _vp, _sz, _vp]),
    "b2r_reduce_workspace_bytes": (_sz, [ctypes.POINTER(ReduceDesc), _vp]),
    "b2r_norm": (ctypes.c_int, [_i32, _i32, _i32, _i32, _i32, _i64, _i64, _i32, _dbl, _vp, _vp, _vp, _sz, _vp]),
    "b2r_reduce_rows_by_key": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp, _vp, _i32, _i32, _i64, _i64, _i64, _i32,
                                              _vp, _sz, _vp]),
    "b2r_reduce_rows_by_key_workspace_bytes": (_sz, [_vp, _i64, _i32, _i64, _i64, _i64]),
    "b2r_reduce_cols_by_key": (ctypes.c_int, [_vp, _vp, _vp, _i32, _i32, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "b2r_reduce_cols_by_key_workspace_bytes": (_sz, [_vp, _i32, _i64, _i64, _i64]),
    "b2r_last_kernel_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int32), _i32]),
    "b2r_set_wait_limit_ms": (ctypes.c_int, [ctypes.c_uint32]),
    "b2r_row_normalize": (ctypes.c_int, [_vp, _vp, _i32, _i64, _i64, _i32, _dbl, _vp]),
    "b2r_matrix_argmin": (ctypes.c_int, [_vp, _i32, _vp, _i32, _i64, _i64, _vp]),
    "b2r_matrix_argmax": (ctypes.c_int, [_vp, _i32, _vp, _i32, _i64, _i64, _vp]),
    "b2r_column_sum_f32_noalloc": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i32, _dbl, _vp]),
    "b2r_column_sum_f32_noalloc_max_scratch": (_sz, []),
    "b2r_apply_final": (ctypes.c_int, [_vp, _i32, _i64, _i32, _dbl, _vp]),
    "b2r_synth_fill": (ctypes.c_int, [_vp, _i32, _i64, _i64, _u64, _i32, _dbl, _dbl, _vp]),
    "b2r_peer_area_create": (ctypes.c_int, [_i32, _i32, _sz, ctypes.POINTER(ctypes.c_void_p)]),
    "b2r_peer_area_ipc_handle": (ctypes.c_int, [_vp, _vp]),
    "b2r_peer_area_open": (ctypes.c_int, [_vp, _i32, _vp]),
    "b2r_peer_area_link": (ctypes.c_int, [_vp, _i32, _vp]),
    "b2r_peer_area_set_wait_limit_ms": (ctypes.c_int, [_vp, ctypes.c_uint32]),
    "b2r_peer_allreduce_sum": (ctypes.c_int, [_vp, _vp, _i64, _vp, _i64, _dbl, _vp]),
    "b2r_peer_area_status": (ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_int32), _i32]),
    "b2r_peer_area_destroy": (ctypes.c_int, [_vp]),
    "b2r_probe_empty_launch": (ctypes.c_int, [_vp]),
    "b2r_probe_stream_read": (ctypes.c_int, [_vp, _sz, _vp, _vp]),
    "b2r_trim_scratch_pool": (ctypes.c_int, []),
    "b2r_reload_tuning": (ctypes.c_int, []),
    "b2r_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "b2r_last_cuda_error": (ctypes.c_int, []),
    "b2r_version": (ctypes.c_char_p, []),
}

_lib = None


def load():
    """Loads libraft_b200.so and types every entry point. Raises if the library is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is not built. Build it with `make -C raft_b200/csrc -j8` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class B2RError(RuntimeError):
    """A non-zero b2r_status. Bad arguments map to the reference's raft::logic_error,
    unsupported combinations to raft::exception, CUDA failures to raft::cuda_error."""

    def __init__(self, status, where):
        lib = load()
        msg = lib.b2r_status_string(status).decode()
        if status == ERR_CUDA:
            msg += f" [cudaError {lib.b2r_last_cuda_error()}]"
        super().__init__(f"{where}: {msg}")
        self.status = status


def check(status, where):
    if status != OK:
        raise B2RError(status, where)
