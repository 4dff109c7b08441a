// b2r_row_normalize: rows divided by their L1 / L2 / Linf norm in one pass over the matrix.
#include "capi_internal.cuh"

#include <raft_b200/detail/row_normalize.cuh>

namespace raft_b200 {
namespace capi {

template <typename T>
static int row_normalize(void* out_v, const void* in_v, int64_t n_rows, int64_t n_cols, int32_t norm_type, double eps,
                         cudaStream_t s)
{
  T* out      = static_cast<T*>(out_v);
  const T* in = static_cast<const T*>(in_v);
  int* status = kernel_status_word();
  cudaError_t e;
  // the functor triples of linalg/normalize.cuh:94-103
  switch (norm_type) {
    case B2R_NORM_L1:
      e = detail::launch_row_normalize<T, int64_t>(out, in, n_rows, n_cols, T(0), T(eps), op::Abs{}, op::Add{},
                                                   op::Identity{}, s, status);
      break;
    case B2R_NORM_L2:
      e = detail::launch_row_normalize<T, int64_t>(out, in, n_rows, n_cols, T(0), T(eps), op::Square{}, op::Add{},
                                                   op::Sqrt{}, s, status);
      break;
    case B2R_NORM_LINF:
      e = detail::launch_row_normalize<T, int64_t>(out, in, n_rows, n_cols, T(0), T(eps), op::Abs{}, op::Max{},
                                                   op::Identity{}, s, status);
      break;
    default: return B2R_ERR_UNSUPPORTED;  // the reference fails for any other norm type (normalize.cuh:104)
  }
  return set_cuda_error(e);
}

}  // namespace capi
}  // namespace raft_b200

extern "C" int b2r_row_normalize(void* out, const void* in, int32_t dtype, int64_t n_rows, int64_t n_cols,
                                 int32_t norm_type, double eps, b2r_stream_t stream)
{
  using namespace raft_b200::capi;
  if (n_rows < 0 || n_cols < 0) return B2R_ERR_BAD_ARG;
  if (n_rows > 0 && n_cols > 0 && (out == nullptr || in == nullptr)) return B2R_ERR_BAD_ARG;
  cudaStream_t s = to_stream(stream);
  if (dtype == B2R_F32) return row_normalize<float>(out, in, n_rows, n_cols, norm_type, eps, s);
  if (dtype == B2R_F64) return row_normalize<double>(out, in, n_rows, n_cols, norm_type, eps, s);
  return B2R_ERR_UNSUPPORTED;
}
