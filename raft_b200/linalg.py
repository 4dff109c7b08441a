"""Host-side mirror of the raft::linalg reduction entry points, on torch CUDA tensors.

Every function forwards to the C ABI (include/raft_b200.h) on the current torch CUDA stream
and is asynchronous, like the reference. Names, argument meaning and error behaviour follow
the reference:

  reduce               linalg/reduce.cuh:140-180  (mdspan form: matrix view, vector view, init,
                       inplace, main_op, reduce_op, final_op)
  coalesced_reduction  linalg/coalesced_reduction.cuh:104-149
  strided_reduction    linalg/strided_reduction.cuh:115-160
  norm                 linalg/norm.cuh:112-148
  reduce_rows_by_key   linalg/reduce_rows_by_key.cuh:140-181
  reduce_cols_by_key   linalg/reduce_cols_by_key.cuh:76-102

Shape errors raise ValueError where the reference's RAFT_EXPECTS raises raft::logic_error;
unsupported type / operator combinations raise B2RError (raft::exception in the reference).
Functors are named by strings because a C ABI cannot carry a device lambda; the C++ headers
under include/raft/ accept arbitrary functors.
"""
import contextlib

import torch

from . import _lib as L

_DTYPES = {
    torch.float32: L.F32,
    torch.float64: L.F64,
    torch.float16: L.F16,
    torch.int32: L.I32,
    torch.int64: L.I64,
    torch.int16: L.I16,
}
_MAIN = {"identity": L.MAIN_IDENTITY, "sq": L.MAIN_SQ, "abs": L.MAIN_ABS, "nz": L.MAIN_NZ, "to_kvp": L.MAIN_TO_KVP}
_REDUCE = {"add": L.REDUCE_ADD, "min": L.REDUCE_MIN, "max": L.REDUCE_MAX, "argmin": L.REDUCE_ARGMIN,
           "argmax": L.REDUCE_ARGMAX}
_FINAL = {"identity": L.FINAL_IDENTITY, "sqrt": L.FINAL_SQRT, "mul_const": L.FINAL_MUL_CONST,
          "div_const": L.FINAL_DIV_CONST, "abs": L.FINAL_ABS}
_NORM = {"L1": L.NORM_L1, "L2": L.NORM_L2, "Linf": L.NORM_LINF, "L0": L.NORM_L0}
_KVP_OF = {L.F32: L.KVP_I32_F32, L.F64: L.KVP_I32_F64, L.I16: L.KVP_I32_I16, L.I32: L.KVP_I32_I32}

ALONG_ROWS = L.ALONG_ROWS
ALONG_COLUMNS = L.ALONG_COLUMNS


def _as_int(v):
    try:
        return int(v)
    except (OverflowError, ValueError):  # inf / nan initial values of floating outputs
        return 0


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_NO_SWITCH = contextlib.nullcontext()


def _stream_ptr(device):
    """cudaStream_t of torch's current stream on `device`."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def _on(device):
    """Context that makes `device` current - a no-op object when it already is (the usual case; switching
    costs microseconds that small reductions notice)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _layout_of(data):
    """Row- or column-major contiguous 2-D tensor -> (layout, n_rows, n_cols); else ValueError,
    like RAFT_EXPECTS(is_row_or_column_major(data)) in linalg/reduce.cuh:157."""
    if data.dim() != 2:
        raise ValueError("Input must be a matrix")
    n_rows, n_cols = data.shape
    if data.is_contiguous():
        return L.ROW_MAJOR, n_rows, n_cols
    if data.t().is_contiguous():
        return L.COL_MAJOR, n_rows, n_cols
    raise ValueError("Input must be contiguous")


def _require_cuda(t, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")


class KeyValueVector:
    """Device array of {int32 key, value} pairs with the memory layout of
    raft::KeyValuePair<int, V> (core/kvp.hpp:20-27)."""

    def __init__(self, n, value_dtype, device):
        self.value_dtype = value_dtype
        self.n = n
        wide = value_dtype == torch.float64
        self.raw = torch.empty((n, 2), dtype=torch.int64 if wide else torch.int32, device=device)

    def data_ptr(self):
        return self.raw.data_ptr()

    @property
    def keys(self):
        if self.value_dtype == torch.float64:
            return self.raw.view(torch.int32)[:, 0]
        return self.raw[:, 0]

    @property
    def values(self):
        if self.value_dtype == torch.float64:
            return self.raw[:, 1].view(torch.float64)
        if self.value_dtype == torch.float32:
            return self.raw[:, 1].view(torch.float32)
        if self.value_dtype == torch.int16:
            return self.raw.view(torch.int16)[:, 2]
        return self.raw[:, 1]

    def fill(self, key, value):
        self.keys.fill_(key)
        self.values.fill_(value)


def reduce(data, apply=ALONG_ROWS, dots=None, init=0.0, inplace=False, main_op="identity", reduce_op="add",
           final_op="identity", final_scalar=1.0, out_dtype=None, init_key=0, workspace=None):
    """dots[k] = final_op(reduce_op over the reduced axis of main_op(data[..], index)).

    `apply` = ALONG_ROWS gives one output per row, ALONG_COLUMNS one per column. With
    reduce_op "argmin"/"argmax" (and main_op "to_kvp") `dots` is a KeyValueVector.
    Returns `dots`.
    """
    _require_cuda(data, "data")
    layout, n_rows, n_cols = _layout_of(data)
    n_out = n_rows if apply == ALONG_ROWS else n_cols
    in_dt = _DTYPES.get(data.dtype)
    if in_dt is None:
        raise L.B2RError(L.ERR_UNSUPPORTED, "reduce")
    kvp = reduce_op in ("argmin", "argmax")
    if kvp:
        if dots is None:
            dots = KeyValueVector(n_out, data.dtype, data.device)
        if not isinstance(dots, KeyValueVector) or dots.value_dtype != data.dtype:
            raise ValueError("argmin/argmax need a KeyValueVector of the input's value type")
        out_dt = _KVP_OF.get(in_dt)
        if out_dt is None:
            raise L.B2RError(L.ERR_UNSUPPORTED, "reduce")
        n_dots = dots.n
    else:
        if dots is None:
            dots = torch.empty(n_out, dtype=out_dtype or (torch.float32 if data.dtype == torch.float16
                                                          else data.dtype), device=data.device)
        _require_cuda(dots, "dots")
        out_dt = _DTYPES.get(dots.dtype)
        n_dots = dots.numel()
        if not dots.is_contiguous():
            raise ValueError("Output must be contiguous")
    if n_dots != n_out:
        raise ValueError("Output should be equal to number of %s in Input" %
                         ("rows" if apply == ALONG_ROWS else "columns"))
    desc = L.ReduceDesc(in_dtype=in_dt, out_dtype=out_dt, layout=layout, apply=apply, n_rows=n_rows, n_cols=n_cols,
                        main_op=_MAIN[main_op], reduce_op=_REDUCE[reduce_op], final_op=_FINAL[final_op],
                        inplace=1 if inplace else 0, init=float(init), init_i=_as_int(init), init_key=int(init_key),
                        final_scalar=float(final_scalar))
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None \
        else (None, 0)
    lib = L.load()
    with _on(data.device):
        st = lib.b2r_reduce(desc, dots.data_ptr(), data.data_ptr(), ws_ptr, ws_bytes, _stream_ptr(data.device))
    L.check(st, "b2r_reduce")
    return dots


def reduce_workspace_bytes(data, apply=ALONG_ROWS, reduce_op="add", out_dtype=None):
    layout, n_rows, n_cols = _layout_of(data)
    in_dt = _DTYPES[data.dtype]
    out_dt = _KVP_OF[in_dt] if reduce_op in ("argmin", "argmax") else _DTYPES[out_dtype or data.dtype]
    desc = L.ReduceDesc(in_dtype=in_dt, out_dtype=out_dt, layout=layout, apply=apply, n_rows=n_rows, n_cols=n_cols,
                        reduce_op=_REDUCE[reduce_op])
    with _on(data.device):
        return L.load().b2r_reduce_workspace_bytes(desc, data.data_ptr())


def coalesced_reduction(data, dots=None, init=0.0, inplace=False, main_op="identity", reduce_op="add",
                        final_op="identity", final_scalar=1.0, **kw):
    """Reduction along the contiguous dimension: rows of a row-major matrix, columns of a
    column-major one (linalg/coalesced_reduction.cuh:104-149)."""
    layout, _, _ = _layout_of(data)
    apply = ALONG_ROWS if layout == L.ROW_MAJOR else ALONG_COLUMNS
    return reduce(data, apply, dots, init, inplace, main_op, reduce_op, final_op, final_scalar, **kw)


def strided_reduction(data, dots=None, init=0.0, inplace=False, main_op="identity", reduce_op="add",
                      final_op="identity", final_scalar=1.0, **kw):
    """Reduction along the strided dimension: columns of a row-major matrix, rows of a
    column-major one (linalg/strided_reduction.cuh:115-160)."""
    layout, _, _ = _layout_of(data)
    apply = ALONG_COLUMNS if layout == L.ROW_MAJOR else ALONG_ROWS
    return reduce(data, apply, dots, init, inplace, main_op, reduce_op, final_op, final_scalar, **kw)


def norm(data, norm_type="L2", apply=ALONG_ROWS, out=None, fin_op="identity", final_scalar=1.0, out_dtype=None,
         workspace=None):
    """L1 / L2 / Linf norm of every row or column (linalg/norm.cuh:112-148). As in the
    reference L2 is the SQUARED norm unless fin_op is "sqrt"; "L0" is refused."""
    _require_cuda(data, "data")
    layout, n_rows, n_cols = _layout_of(data)
    n_out = n_rows if apply == ALONG_ROWS else n_cols
    if out is None:
        out = torch.empty(n_out, dtype=out_dtype or (torch.float32 if data.dtype == torch.float16 else data.dtype),
                          device=data.device)
    if out.numel() != n_out:
        raise ValueError("Output should be equal to number of %s in Input" %
                         ("rows" if apply == ALONG_ROWS else "columns"))
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None \
        else (None, 0)
    with _on(data.device):
        st = L.load().b2r_norm(_NORM[norm_type], apply, layout, _DTYPES[data.dtype], _DTYPES[out.dtype], n_rows,
                               n_cols, _FINAL[fin_op], float(final_scalar), out.data_ptr(), data.data_ptr(), ws_ptr,
                               ws_bytes, _stream_ptr(data.device))
    L.check(st, "b2r_norm")
    return out


_KEY_DTYPES = {torch.int32: L.I32, torch.int64: L.I64, torch.uint32: L.U32} if hasattr(torch, "uint32") else \
    {torch.int32: L.I32, torch.int64: L.I64}


def reduce_rows_by_key(d_A, d_keys, n_unique_keys, d_sums=None, d_weights=None, reset_sums=True, counts=None,
                       lda=None, workspace=None):
    """d_sums[d_keys[i], :] += d_weights[i] * d_A[i, :] (linalg/reduce_rows_by_key.cuh:140-181).

    d_A is [nrows x ncols] row-major (row stride `lda`, default ncols); d_sums is
    [n_unique_keys x ncols]. `counts` (int64 [n_unique_keys], optional) receives the rows per
    key - an extension the reference does not have. Returns d_sums.
    """
    _require_cuda(d_A, "d_A")
    _require_cuda(d_keys, "d_keys")
    if d_A.dim() != 2:
        raise ValueError("d_A must be a matrix")
    nrows, ncols = d_A.shape
    if lda is None:
        if d_A.stride(1) != 1 and ncols > 1:
            raise ValueError("d_A must be row-major")
        lda = d_A.stride(0) if nrows > 1 else ncols
    if d_keys.numel() != nrows:
        raise ValueError("Keys is not of size nrows")
    if d_weights is not None and d_weights.numel() != nrows:
        raise ValueError("Weights is not of size nrows")
    if d_sums is None:
        d_sums = torch.zeros((n_unique_keys, ncols), dtype=d_A.dtype, device=d_A.device)
    if tuple(d_sums.shape) != (n_unique_keys, ncols) or not d_sums.is_contiguous():
        raise ValueError("Output is not of size ncols * n_unique_keys")
    if d_sums.dtype != d_A.dtype or (d_weights is not None and d_weights.dtype != d_A.dtype):
        raise L.B2RError(L.ERR_UNSUPPORTED, "reduce_rows_by_key")
    if counts is not None and (counts.dtype != torch.int64 or counts.numel() != n_unique_keys):
        raise ValueError("counts must be int64 of size n_unique_keys")
    key_dt = _KEY_DTYPES.get(d_keys.dtype)
    if key_dt is None or d_A.dtype not in (torch.float32, torch.float64):
        raise L.B2RError(L.ERR_UNSUPPORTED, "reduce_rows_by_key")
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None \
        else (None, 0)
    with _on(d_A.device):
        st = L.load().b2r_reduce_rows_by_key(
            d_sums.data_ptr(), counts.data_ptr() if counts is not None else None, d_A.data_ptr(), lda,
            d_keys.data_ptr(), d_weights.data_ptr() if d_weights is not None else None, _DTYPES[d_A.dtype], key_dt,
            nrows, ncols, n_unique_keys, 1 if reset_sums else 0, ws_ptr, ws_bytes, _stream_ptr(d_A.device))
    L.check(st, "b2r_reduce_rows_by_key")
    return d_sums


def reduce_rows_by_key_workspace_bytes(d_A, n_unique_keys, lda=None):
    nrows, ncols = d_A.shape
    with _on(d_A.device):
        return L.load().b2r_reduce_rows_by_key_workspace_bytes(d_A.data_ptr(), lda or ncols, _DTYPES[d_A.dtype],
                                                               nrows, ncols, n_unique_keys)


def reduce_cols_by_key(data, keys, out=None, nkeys=0, reset_sums=True, workspace=None):
    """out[r, keys[c]] += data[r, c] (linalg/reduce_cols_by_key.cuh:76-102). nkeys = 0 infers
    the number of keys from out.shape[1], as the reference does. `workspace` (uint8, see
    reduce_cols_by_key_workspace_bytes) keeps the call allocation-free."""
    _require_cuda(data, "data")
    _require_cuda(keys, "keys")
    if data.dim() != 2 or not data.is_contiguous():
        raise ValueError("data must be a row-major matrix")
    nrows, ncols = data.shape
    if out is None:
        if nkeys <= 0:
            raise ValueError("nkeys or out is required")
        out = torch.zeros((nrows, nkeys), dtype=data.dtype, device=data.device)
    if nkeys > 0:
        if out.shape[1] != nkeys:
            raise ValueError("Output doesn't have nkeys columns")
    else:
        nkeys = out.shape[1]
    if out.shape[0] != nrows:
        raise ValueError("Output doesn't have the same number of rows as input")
    if keys.numel() != ncols:
        raise ValueError("Keys is not of size ncols")
    key_dt = _KEY_DTYPES.get(keys.dtype)
    if key_dt is None or data.dtype not in (torch.float32, torch.float64) or out.dtype != data.dtype:
        raise L.B2RError(L.ERR_UNSUPPORTED, "reduce_cols_by_key")
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None \
        else (None, 0)
    with _on(data.device):
        st = L.load().b2r_reduce_cols_by_key(out.data_ptr(), data.data_ptr(), keys.data_ptr(), _DTYPES[data.dtype],
                                             key_dt, nrows, ncols, nkeys, 1 if reset_sums else 0, ws_ptr, ws_bytes,
                                             _stream_ptr(data.device))
    L.check(st, "b2r_reduce_cols_by_key")
    return out


def reduce_cols_by_key_workspace_bytes(data, nkeys):
    nrows, ncols = data.shape
    with _on(data.device):
        return L.load().b2r_reduce_cols_by_key_workspace_bytes(data.data_ptr(), _DTYPES[data.dtype], nrows, ncols,
                                                               nkeys)


def last_kernel_status(device, clear=True):
    """Synchronises `device` and returns L.OK, or L.ERR_TIMEOUT if a bounded wait inside a kernel of any
    earlier call on that device ran out (that call's unfinished floating-point outputs are NaN)."""
    import ctypes
    torch.cuda.synchronize(device)
    out = ctypes.c_int32(0)
    with _on(device):
        L.check(L.load().b2r_last_kernel_status(ctypes.byref(out), 1 if clear else 0), "b2r_last_kernel_status")
    return out.value


def set_wait_limit_ms(ms):
    """Bound of every wait inside the kernels that stage tiles through shared memory; 0 = the default."""
    L.check(L.load().b2r_set_wait_limit_ms(int(ms)), "b2r_set_wait_limit_ms")


def _matrix_arg(fn_name, data, out, index_dtype):
    _require_cuda(data, "in")
    if data.dim() != 2 or not data.is_contiguous():
        raise ValueError("in must be a row-major matrix")
    n_rows, n_cols = data.shape
    if out is None:
        out = torch.empty(n_rows, dtype=index_dtype, device=data.device)
    if out.numel() != n_rows:
        raise ValueError("Size of output vector must equal number of rows in input matrix.")
    if data.dtype not in (torch.float32, torch.float64) or out.dtype not in (torch.int32, torch.int64):
        raise L.B2RError(L.ERR_UNSUPPORTED, fn_name)
    with _on(data.device):
        st = getattr(L.load(), fn_name)(out.data_ptr(), _DTYPES[out.dtype], data.data_ptr(), _DTYPES[data.dtype],
                                        n_rows, n_cols, _stream_ptr(data.device))
    L.check(st, fn_name)
    return out


def argmin(data, out=None, index_dtype=torch.int32):
    """raft::matrix::argmin (matrix/argmin.cuh:27-39): index of the smallest element of every row
    of a row-major matrix, lowest index on ties."""
    return _matrix_arg("b2r_matrix_argmin", data, out, index_dtype)


def argmax(data, out=None, index_dtype=torch.int32):
    """raft::matrix::argmax (matrix/argmax.cuh:27-39): index of the largest element of every row,
    lowest index on ties."""
    return _matrix_arg("b2r_matrix_argmax", data, out, index_dtype)


def map_reduce(data, map_op="identity", reduce_op="add", neutral=0.0, out=None, out_dtype=None, workspace=None):
    """raft::linalg::mapReduce / mapThenSumReduce for the named map functors
    (linalg/map_reduce.cuh:43-103, linalg/map_then_reduce.cuh:37-53):
    out[0] = reduce_op over i of map_op(data[i]); `neutral` is the identity of reduce_op.
    `data` is any contiguous tensor, read as a flat array. Returns a one-element tensor."""
    _require_cuda(data, "data")
    if not data.is_contiguous():
        raise ValueError("Input must be contiguous")
    flat = data.reshape(1, -1)
    if out is None:
        out = torch.empty(1, dtype=out_dtype or data.dtype, device=data.device)
    return reduce(flat, ALONG_ROWS, out, init=neutral, main_op=map_op, reduce_op=reduce_op, workspace=workspace)


def row_normalize(data, norm_type="L2", out=None, eps=1e-8):
    """raft::linalg::row_normalize<norm_type> (linalg/normalize.cuh:88-107): every row of a
    row-major matrix divided by its L1 / L2 / Linf norm. A row whose norm is <= eps is not
    written: `out` keeps what it held there (the reference's behaviour), so pass an initialised
    `out` if such rows can occur. `out` may be `data`."""
    _require_cuda(data, "data")
    if data.dim() != 2 or not data.is_contiguous():
        raise ValueError("Input must be contiguous")
    if out is None:
        out = torch.zeros_like(data)
    _require_cuda(out, "out")
    if not out.is_contiguous():
        raise ValueError("Output must be contiguous")
    if out.shape[0] != data.shape[0]:
        raise ValueError("The number of rows of the input and output should be equal")
    if out.shape[1] != data.shape[1]:
        raise ValueError("The number of columns of the input and output should be equal")
    if out.dtype != data.dtype:
        raise ValueError("input and output must have the same element type")
    if norm_type not in ("L1", "L2", "Linf"):
        raise ValueError("Unsupported norm type: %s" % norm_type)
    n_rows, n_cols = data.shape
    with _on(data.device):
        st = L.load().b2r_row_normalize(out.data_ptr(), data.data_ptr(), _DTYPES[data.dtype], n_rows, n_cols,
                                        _NORM[norm_type], float(eps), _stream_ptr(data.device))
    L.check(st, "b2r_row_normalize")
    return out


def probe_empty_launch(device):
    """One empty kernel on the device's current stream (the cost floor of an event pair around a launch)."""
    with _on(device):
        L.check(L.load().b2r_probe_empty_launch(_stream_ptr(device)), "b2r_probe_empty_launch")


def probe_stream_read(data):
    """Reads `data` once with plain streaming loads and does nothing else (the read floor of its size)."""
    _require_cuda(data, "data")
    with _on(data.device):
        L.check(L.load().b2r_probe_stream_read(data.data_ptr(), data.numel() * data.element_size(), None,
                                               _stream_ptr(data.device)), "b2r_probe_stream_read")


def reload_tuning():
    """Makes the library read its B2R_* environment knobs again (they are otherwise read once, at the
    first call). For tests and sweeps that change them within one process."""
    L.check(L.load().b2r_reload_tuning(), "b2r_reload_tuning")


def apply_final(v, final_op, final_scalar=1.0):
    """v[i] = final_op(v[i]) in place (the deferred final step of a sharded reduction)."""
    _require_cuda(v, "v")
    with _on(v.device):
        st = L.load().b2r_apply_final(v.data_ptr(), _DTYPES[v.dtype], v.numel(), _FINAL[final_op],
                                      float(final_scalar), _stream_ptr(v.device))
    L.check(st, "b2r_apply_final")
    return v


def synth_fill(dst, seed, kind, lo=0.0, hi=1.0, first_index=0):
    """Fills `dst` (any shape, contiguous) with the counter-based synthetic data of
    b2r_synth_fill: kind "uniform", "normal" or "int"."""
    _require_cuda(dst, "dst")
    if not dst.is_contiguous():
        raise ValueError("dst must be contiguous")
    k = {"uniform": 0, "normal": 1, "int": 2}[kind]
    with _on(dst.device):
        st = L.load().b2r_synth_fill(dst.data_ptr(), _DTYPES[dst.dtype], dst.numel(), first_index, seed, k,
                                     float(lo), float(hi), _stream_ptr(dst.device))
    L.check(st, "b2r_synth_fill")
    return dst
