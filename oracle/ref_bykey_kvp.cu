// oracle/_ref: the reference's key/value row reduction, reduce_rows_by_key and reduce_cols_by_key.
#include "ref_common.cuh"

#include <raft/linalg/reduce_cols_by_key.cuh>
#include <raft/linalg/reduce_rows_by_key.cuh>

using namespace refwrap;

template <typename T>
static int kvp(const b2r_reduce_desc& d, void* out, const void* in, cudaStream_t s)
{
  using KV = raft::KeyValuePair<int, T>;
  const KV init{int(d.init_key), T(d.init)};
  if (d.reduce_op == B2R_REDUCE_ARGMIN)
    return run<true, true, T, KV>(d, out, in, init, ValueToKVP<T, int>{}, raft::argmin_op{}, raft::identity_op{}, s);
  if (d.reduce_op == B2R_REDUCE_ARGMAX)
    return run<true, true, T, KV>(d, out, in, init, ValueToKVP<T, int>{}, raft::argmax_op{}, raft::identity_op{}, s);
  return B2R_ERR_UNSUPPORTED;
}

// row-major, along rows, KeyValuePair<int, T> outputs
REF_EXPORT int ref_reduce_kvp(const b2r_reduce_desc* d, void* out, const void* in, cudaStream_t s)
{
  if (d->layout != B2R_ROW_MAJOR || d->apply != B2R_ALONG_ROWS) return B2R_ERR_UNSUPPORTED;
  if (d->in_dtype == B2R_F32 && d->out_dtype == B2R_KVP_I32_F32) return kvp<float>(*d, out, in, s);
  if (d->in_dtype == B2R_F64 && d->out_dtype == B2R_KVP_I32_F64) return kvp<double>(*d, out, in, s);
  return B2R_ERR_UNSUPPORTED;
}

template <typename T>
static int rows_by_key(void* sums, const void* A, int64_t lda, const void* keys, const void* w, int64_t nrows,
                       int64_t ncols, int64_t nkeys, int reset, cudaStream_t s)
{
  return guarded([&] {
    const int* k = static_cast<const int*>(keys);
    if (w != nullptr) {
      raft::linalg::reduce_rows_by_key(static_cast<const T*>(A), int(lda), k, static_cast<const T*>(w),
                                       static_cast<char*>(nullptr), int(nrows), int(ncols), int(nkeys),
                                       static_cast<T*>(sums), s, reset != 0);
    } else {
      raft::linalg::reduce_rows_by_key(static_cast<const T*>(A), int(lda), k, static_cast<char*>(nullptr),
                                       int(nrows), int(ncols), int(nkeys), static_cast<T*>(sums), s, reset != 0);
    }
  });
}

// int32 keys; f32 or f64 data (weights, when given, of the data type)
REF_EXPORT int ref_rows_by_key(void* sums, const void* A, int64_t lda, const void* keys, const void* weights,
                               int32_t dtype, int64_t nrows, int64_t ncols, int64_t nkeys, int32_t reset,
                               cudaStream_t s)
{
  if (nrows * ncols > 0x7fffffffLL) return B2R_ERR_TOO_LARGE;  // the reference indexes with IdxT = int here
  if (dtype == B2R_F32) return rows_by_key<float>(sums, A, lda, keys, weights, nrows, ncols, nkeys, reset, s);
  if (dtype == B2R_F64) return rows_by_key<double>(sums, A, lda, keys, weights, nrows, ncols, nkeys, reset, s);
  return B2R_ERR_UNSUPPORTED;
}

REF_EXPORT int ref_cols_by_key(void* out, const void* data, const void* keys, int32_t dtype, int64_t nrows,
                               int64_t ncols, int64_t nkeys, int32_t reset, cudaStream_t s)
{
  if (nrows * ncols > 0x7fffffffLL || nrows * nkeys > 0x7fffffffLL) return B2R_ERR_TOO_LARGE;
  const int* k = static_cast<const int*>(keys);
  if (dtype == B2R_F32)
    return guarded([&] {
      raft::linalg::reduce_cols_by_key(static_cast<const float*>(data), k, static_cast<float*>(out), int(nrows),
                                       int(ncols), int(nkeys), s, reset != 0);
    });
  if (dtype == B2R_F64)
    return guarded([&] {
      raft::linalg::reduce_cols_by_key(static_cast<const double*>(data), k, static_cast<double*>(out), int(nrows),
                                       int(ncols), int(nkeys), s, reset != 0);
    });
  return B2R_ERR_UNSUPPORTED;
}
