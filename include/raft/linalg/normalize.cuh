// raft::linalg::row_normalize on the B200 kernels (reference: linalg/normalize.cuh:46-107; kernels
// linalg/detail/normalize.cuh:26-197): every row divided by final(reduce(main(x, column))); a row
// whose norm is <= eps is not written. The L1 / L2 / Linf functor triples on float or double go to
// the precompiled kernels behind b2r_row_normalize; any other functor or element type instantiates
// the same kernel templates in the caller's translation unit.
#pragma once

#include "detail/b200_dispatch.cuh"
#include "norm_types.hpp"

#include <raft/core/device_mdspan.hpp>
#include <raft/core/operators.hpp>
#include <raft/core/resource/cuda_stream.hpp>
#include <raft/core/resources.hpp>
#include <raft/util/input_validation.hpp>

#include <raft_b200/detail/row_normalize.cuh>

namespace raft {
namespace linalg {

namespace b200 {
// norm type whose (main, reduce, final) triple this is, or -1
template <typename MainLambda, typename ReduceLambda, typename FinalLambda>
constexpr int normalize_norm_type()
{
  constexpr bool abs_m = std::is_same<MainLambda, raft::abs_op>::value;
  constexpr bool sq_m  = std::is_same<MainLambda, raft::sq_op>::value;
  constexpr bool add_r = std::is_same<ReduceLambda, raft::add_op>::value;
  constexpr bool max_r = std::is_same<ReduceLambda, raft::max_op>::value;
  constexpr bool id_f  = std::is_same<FinalLambda, raft::identity_op>::value;
  constexpr bool rt_f  = std::is_same<FinalLambda, raft::sqrt_op>::value;
  return (abs_m && add_r && id_f) ? int(B2R_NORM_L1)
         : (sq_m && add_r && rt_f) ? int(B2R_NORM_L2)
         : (abs_m && max_r && id_f) ? int(B2R_NORM_LINF)
                                    : -1;
}
}  // namespace b200

/** Divide rows by their norm defined by main_op, reduce_op and fin_op. */
template <typename ElementType, typename IndexType, typename MainLambda, typename ReduceLambda, typename FinalLambda>
void row_normalize(raft::resources const& handle,
                   raft::device_matrix_view<const ElementType, IndexType, row_major> in,
                   raft::device_matrix_view<ElementType, IndexType, row_major> out,
                   ElementType init,
                   MainLambda main_op,
                   ReduceLambda reduce_op,
                   FinalLambda fin_op,
                   ElementType eps = ElementType(1e-8))
{
  RAFT_EXPECTS(raft::is_row_or_column_major(in), "Input must be contiguous");
  RAFT_EXPECTS(raft::is_row_or_column_major(out), "Output must be contiguous");
  RAFT_EXPECTS(in.extent(0) == out.extent(0), "The number of rows of the input and output should be equal");
  RAFT_EXPECTS(in.extent(1) == out.extent(1), "The number of columns of the input and output should be equal");
  cudaStream_t stream      = resource::get_cuda_stream(handle);
  constexpr int norm_type  = b200::normalize_norm_type<MainLambda, ReduceLambda, FinalLambda>();
  constexpr bool abi_dtype = std::is_same<ElementType, float>::value || std::is_same<ElementType, double>::value;
  if constexpr (norm_type >= 0 && abi_dtype) {
    if (init == ElementType(0)) {
      b200::check(b2r_row_normalize(out.data_handle(), in.data_handle(), b200::dtype_of<ElementType>::value,
                                    int64_t(in.extent(0)), int64_t(in.extent(1)), norm_type, double(eps),
                                    reinterpret_cast<b2r_stream_t>(stream)),
                  "row_normalize");
      return;
    }
  }
  b200::check_cuda(raft_b200::detail::launch_row_normalize<ElementType, IndexType>(
                     out.data_handle(), in.data_handle(), int64_t(in.extent(0)), int64_t(in.extent(1)), init, eps,
                     main_op, reduce_op, fin_op, stream),
                   "row_normalize");
}

/** Divide rows by their L1 / L2 / Linf norm. */
template <NormType norm_type, typename ElementType, typename IndexType>
void row_normalize(raft::resources const& handle,
                   raft::device_matrix_view<const ElementType, IndexType, row_major> in,
                   raft::device_matrix_view<ElementType, IndexType, row_major> out,
                   ElementType eps = ElementType(1e-8))
{
  if constexpr (norm_type == L1Norm) {
    row_normalize(handle, in, out, ElementType(0), raft::abs_op(), raft::add_op(), raft::identity_op(), eps);
  } else if constexpr (norm_type == L2Norm) {
    row_normalize(handle, in, out, ElementType(0), raft::sq_op(), raft::add_op(), raft::sqrt_op(), eps);
  } else if constexpr (norm_type == LinfNorm) {
    row_normalize(handle, in, out, ElementType(0), raft::abs_op(), raft::max_op(), raft::identity_op(), eps);
  } else {
    RAFT_FAIL("Unsupported norm type: %d", norm_type);
  }
}

}  // namespace linalg
}  // namespace raft
