// b2r_matrix_argmin / b2r_matrix_argmax: index of the smallest / largest element of every row
// (index-only form of the key/value row reduction; 4 or 8 output bytes per row).
#include "capi_internal.cuh"

#include <limits>

namespace raft_b200 {
namespace capi {

template <typename InT, typename IndexT, bool IsMin>
static int matrix_arg(void* out, const void* in, int64_t n_rows, int64_t n_cols, cudaStream_t s)
{
  using KV = KeyValue<int, InT>;
  // start value of the reference kernel: {0, +inf} for argmin, {0, -inf} for argmax
  // (matrix/detail/math.cuh:301)
  KV init;
  init.key   = 0;
  init.value = IsMin ? std::numeric_limits<InT>::infinity() : -std::numeric_limits<InT>::infinity();
  cudaError_t e;
  if constexpr (IsMin) {
    e = detail::launch_row_reduce<InT, KV, int64_t>(static_cast<IndexT*>(out), static_cast<const InT*>(in), n_rows,
                                                    n_cols, n_cols, init, false, op::ToKeyValue<int>{}, op::ArgMin{},
                                                    op::KeyOf<IndexT>{}, s);
  } else {
    e = detail::launch_row_reduce<InT, KV, int64_t>(static_cast<IndexT*>(out), static_cast<const InT*>(in), n_rows,
                                                    n_cols, n_cols, init, false, op::ToKeyValue<int>{}, op::ArgMax{},
                                                    op::KeyOf<IndexT>{}, s);
  }
  return set_cuda_error(e);
}

template <bool IsMin>
static int matrix_arg_any(void* out, int32_t out_dtype, const void* in, int32_t in_dtype, int64_t n_rows,
                          int64_t n_cols, b2r_stream_t stream)
{
  if (n_rows < 0 || n_cols < 0 || n_cols > int64_t(0x7fffffff)) return B2R_ERR_BAD_ARG;
  if (n_rows > 0 && (out == nullptr || (n_cols > 0 && in == nullptr))) return B2R_ERR_BAD_ARG;
  cudaStream_t s = to_stream(stream);
  if (in_dtype == B2R_F32 && out_dtype == B2R_I32) return matrix_arg<float, int, IsMin>(out, in, n_rows, n_cols, s);
  if (in_dtype == B2R_F32 && out_dtype == B2R_I64)
    return matrix_arg<float, long long, IsMin>(out, in, n_rows, n_cols, s);
  if (in_dtype == B2R_F64 && out_dtype == B2R_I32) return matrix_arg<double, int, IsMin>(out, in, n_rows, n_cols, s);
  if (in_dtype == B2R_F64 && out_dtype == B2R_I64)
    return matrix_arg<double, long long, IsMin>(out, in, n_rows, n_cols, s);
  return B2R_ERR_UNSUPPORTED;
}

}  // namespace capi
}  // namespace raft_b200

extern "C" int b2r_matrix_argmin(void* out, int32_t out_dtype, const void* in, int32_t in_dtype, int64_t n_rows,
                                 int64_t n_cols, b2r_stream_t stream)
{
  return raft_b200::capi::matrix_arg_any<true>(out, out_dtype, in, in_dtype, n_rows, n_cols, stream);
}

extern "C" int b2r_matrix_argmax(void* out, int32_t out_dtype, const void* in, int32_t in_dtype, int64_t n_rows,
                                 int64_t n_cols, b2r_stream_t stream)
{
  return raft_b200::capi::matrix_arg_any<false>(out, out_dtype, in, in_dtype, n_rows, n_cols, stream);
}
