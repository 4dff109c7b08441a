// raft::linalg::mapThenSumReduce / mapThenReduce on the B200 kernels (reference:
// linalg/map_then_reduce.cuh:37-82, kernel linalg/detail/map_then_reduce.cuh:44-94):
//     out[0] = reduce_i map(in[i], args[i]...)
// The array is treated as a 1 x len matrix reduced along its row: segments of the array go to
// persistent CTAs, their partial results are folded in a fixed order - no atomics, so the result
// is the same on every run (the reference adds one atomic per 256 elements). Sums of float
// values are carried in fp64. A named map functor without extra arrays (raft::identity_op,
// sq_op, abs_op, nz_op) on a type pair the library carries goes through the C ABI; everything
// else instantiates the kernel templates here. TPB is accepted and ignored.
#pragma once

#include "detail/b200_dispatch.cuh"

#include <cuda/std/tuple>

#include <cstdint>

namespace raft {
namespace linalg {

namespace b200 {
// main_op of the row reduction: element and its position -> map(element, args[position]...)
template <typename OutType, typename MapOp, typename... Args>
struct map_at_index {
  MapOp map;
  cuda::std::tuple<Args...> args;
  template <typename In, typename Idx>
  __host__ __device__ OutType operator()(const In& x, Idx i)
  {
    return cuda::std::apply([&](auto... a) { return OutType(map(x, a[i]...)); }, args);
  }
};

template <typename InType, typename OutType, typename MapOp, typename ReduceLambda, typename... Args>
void map_reduce(OutType* out, size_t len, OutType neutral, MapOp map, ReduceLambda op, cudaStream_t stream,
                const InType* in, Args... args)
{
  if constexpr (sizeof...(Args) == 0 && main_enum<MapOp>::value >= 0) {
    reduce<true, true, InType, OutType, int64_t>(out, in, int64_t(len), int64_t(1), neutral, stream, false, map, op,
                                                 raft::identity_op());
  } else {
    map_at_index<OutType, MapOp, Args...> main_op{map, cuda::std::tuple<Args...>(args...)};
    reduce<true, true, InType, OutType, int64_t>(out, in, int64_t(len), int64_t(1), neutral, stream, false, main_op,
                                                 op, raft::identity_op());
  }
}
}  // namespace b200

/** out[0] = sum_i map(in[i], args[i]...) */
template <typename InType,
          typename MapOp,
          typename IdxType = std::uint32_t,
          int TPB          = 256,
          typename... Args,
          typename OutType = InType>
void mapThenSumReduce(OutType* out, IdxType len, MapOp map, cudaStream_t stream, const InType* in, Args... args)
{
  b200::map_reduce<InType, OutType>(out, size_t(len), OutType(0), map, raft::add_op(), stream, in, args...);
}

/** out[0] = reduce_i map(in[i], args[i]...); `neutral` must be the identity of `op`. */
template <typename InType,
          typename MapOp,
          typename ReduceLambda,
          typename IdxType = std::uint32_t,
          int TPB          = 256,
          typename OutType = InType,
          typename... Args>
[[deprecated("Use function `mapReduce` from `raft/linalg/map_reduce.cuh")]] void mapThenReduce(
  OutType* out, size_t len, OutType neutral, MapOp map, ReduceLambda op, cudaStream_t stream, const InType* in,
  Args... args)
{
  b200::map_reduce<InType, OutType>(out, len, neutral, map, op, stream, in, args...);
}

}  // namespace linalg
}  // namespace raft
