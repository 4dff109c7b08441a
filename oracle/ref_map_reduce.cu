// oracle/_ref: the reference's raft::linalg::mapThenSumReduce and map_reduce
// (linalg/map_then_reduce.cuh:37-53, linalg/map_reduce.cuh:82-103) with raft::identity_op as map.
#include "ref_common.cuh"

#include <raft/core/device_mdspan.hpp>
#include <raft/core/resource/cuda_stream.hpp>
#include <raft/core/resources.hpp>
#include <raft/linalg/map_reduce.cuh>
#include <raft/linalg/map_then_reduce.cuh>

#include <cuda/functional>

using namespace refwrap;

REF_EXPORT int ref_map_then_sum_reduce(void* out, const void* in, int32_t dtype, int64_t len, cudaStream_t s)
{
  return guarded([&] {
    if (dtype == B2R_F32)
      raft::linalg::mapThenSumReduce(static_cast<float*>(out), size_t(len), raft::identity_op{}, s,
                                     static_cast<const float*>(in));
    else
      raft::linalg::mapThenSumReduce(static_cast<double*>(out), size_t(len), raft::identity_op{}, s,
                                     static_cast<const double*>(in));
  });
}

// reduce_op: B2R_REDUCE_MIN or B2R_REDUCE_MAX, float only; `neutral` as the reference's test passes it
REF_EXPORT int ref_map_reduce_minmax(void* out, const void* in, int64_t len, int32_t reduce_op, float neutral,
                                     cudaStream_t s)
{
  return guarded([&] {
    raft::resources handle;
    raft::resource::set_cuda_stream(handle, rmm::cuda_stream_view(s));
    auto iv = raft::make_device_vector_view<const float, std::uint32_t>(static_cast<const float*>(in),
                                                                         static_cast<std::uint32_t>(len));
    auto ov = raft::make_device_scalar_view(static_cast<float*>(out));
    if (reduce_op == B2R_REDUCE_MIN)
      raft::linalg::map_reduce(handle, iv, ov, neutral, raft::identity_op{}, cuda::minimum{});
    else
      raft::linalg::map_reduce(handle, iv, ov, neutral, raft::identity_op{}, cuda::maximum{});
  });
}
