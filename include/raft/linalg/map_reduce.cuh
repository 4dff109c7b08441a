// raft::linalg::mapReduce / map_reduce on the B200 kernels (reference: linalg/map_reduce.cuh:43-103):
// out[0] = reduce_i map(in[i], args[i]...), `neutral` the identity of `op`.
#pragma once

#include "map_then_reduce.cuh"

#include <raft/core/device_mdspan.hpp>
#include <raft/core/resource/cuda_stream.hpp>
#include <raft/core/resources.hpp>

namespace raft {
namespace linalg {

template <typename InType,
          typename MapOp,
          typename ReduceLambda,
          typename IdxType = std::uint32_t,
          int TPB          = 256,
          typename OutType = InType,
          typename... Args>
void mapReduce(OutType* out, size_t len, OutType neutral, MapOp map, ReduceLambda op, cudaStream_t stream,
               const InType* in, Args... args)
{
  b200::map_reduce<InType, OutType>(out, len, neutral, map, op, stream, in, args...);
}

template <typename InValueType,
          typename MapOp,
          typename ReduceLambda,
          typename IndexType,
          typename OutValueType,
          typename ScalarIdxType,
          typename... Args>
void map_reduce(raft::resources const& handle,
                raft::device_vector_view<const InValueType, IndexType> in,
                raft::device_scalar_view<OutValueType, ScalarIdxType> out,
                OutValueType neutral,
                MapOp map,
                ReduceLambda op,
                Args... args)
{
  mapReduce<InValueType, MapOp, ReduceLambda, IndexType, 256, OutValueType, Args...>(
    out.data_handle(), in.extent(0), neutral, map, op, resource::get_cuda_stream(handle), in.data_handle(), args...);
}

}  // namespace linalg
}  // namespace raft
