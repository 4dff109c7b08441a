// oracle/_ref: the reference's raft::linalg::row_normalize (linalg/normalize.cuh:88-107).
#include "ref_common.cuh"

#include <raft/core/device_mdspan.hpp>
#include <raft/core/resource/cuda_stream.hpp>
#include <raft/core/resources.hpp>
#include <raft/linalg/normalize.cuh>

using namespace refwrap;

template <typename T>
static int run_normalize(void* out, const void* in, int64_t n_rows, int64_t n_cols, int norm_type, cudaStream_t s)
{
  return guarded([&] {
    raft::resources handle;
    raft::resource::set_cuda_stream(handle, rmm::cuda_stream_view(s));
    auto iv = raft::make_device_matrix_view<const T, int64_t, raft::row_major>(static_cast<const T*>(in), n_rows, n_cols);
    auto ov = raft::make_device_matrix_view<T, int64_t, raft::row_major>(static_cast<T*>(out), n_rows, n_cols);
    switch (norm_type) {
      case B2R_NORM_L1: raft::linalg::row_normalize<raft::linalg::L1Norm>(handle, iv, ov); break;
      case B2R_NORM_L2: raft::linalg::row_normalize<raft::linalg::L2Norm>(handle, iv, ov); break;
      default: raft::linalg::row_normalize<raft::linalg::LinfNorm>(handle, iv, ov); break;
    }
  });
}

REF_EXPORT int ref_row_normalize(void* out, const void* in, int32_t dtype, int64_t n_rows, int64_t n_cols,
                                 int32_t norm_type, cudaStream_t s)
{
  if (norm_type < B2R_NORM_L1 || norm_type > B2R_NORM_LINF) return B2R_ERR_UNSUPPORTED;
  if (dtype == B2R_F32) return run_normalize<float>(out, in, n_rows, n_cols, norm_type, s);
  if (dtype == B2R_F64) return run_normalize<double>(out, in, n_rows, n_cols, norm_type, s);
  return B2R_ERR_UNSUPPORTED;
}
