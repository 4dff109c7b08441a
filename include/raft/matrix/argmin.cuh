// raft::matrix::argmin on the B200 kernels (reference: matrix/argmin.cuh:27-39, kernel
// matrix/detail/math.cuh:291-352): the column index of the minimum of every row of a row-major
// matrix; equal values resolve to the lowest index.
#pragma once

#include <raft/core/device_mdspan.hpp>
#include <raft/core/error.hpp>
#include <raft/core/resource/cuda_stream.hpp>
#include <raft/core/resources.hpp>
#include <raft/linalg/detail/b200_dispatch.cuh>

#include <limits>
#include <type_traits>

namespace raft {
namespace matrix {

template <typename math_t, typename idx_t, typename matrix_idx_t>
void argmin(raft::resources const& handle,
            raft::device_matrix_view<const math_t, matrix_idx_t, row_major> in,
            raft::device_vector_view<idx_t, matrix_idx_t> out)
{
  RAFT_EXPECTS(out.extent(0) == in.extent(0), "Size of output vector must equal number of rows in input matrix.");
  cudaStream_t stream = resource::get_cuda_stream(handle);
  constexpr bool abi_value = std::is_same<math_t, float>::value || std::is_same<math_t, double>::value;
  constexpr bool abi_index = std::is_same<idx_t, int>::value || std::is_same<idx_t, long long>::value ||
                             (std::is_same<idx_t, long>::value && sizeof(long) == 8);
  if constexpr (abi_value && abi_index) {
    // precompiled kernels behind the C ABI
    raft::linalg::b200::check(
      b2r_matrix_argmin(out.data_handle(), sizeof(idx_t) == 8 ? B2R_I64 : B2R_I32, in.data_handle(),
                        raft::linalg::b200::dtype_of<math_t>::value, int64_t(in.extent(0)), int64_t(in.extent(1)),
                        reinterpret_cast<b2r_stream_t>(stream)),
      "raft::matrix::argmin");
  } else {
    // any other value / index type: the same kernel templates, instantiated here
    using KV = raft_b200::KeyValue<int, math_t>;
    KV init;
    init.key   = 0;
    init.value = std::numeric_limits<math_t>::infinity();
    raft::linalg::b200::check_cuda(
      raft_b200::detail::launch_row_reduce<math_t, KV, matrix_idx_t>(
        out.data_handle(), in.data_handle(), int64_t(in.extent(0)), int64_t(in.extent(1)), int64_t(in.extent(1)),
        init, false, raft_b200::op::ToKeyValue<int>{}, raft_b200::op::ArgMin{}, raft_b200::op::KeyOf<idx_t>{},
        stream),
      "raft::matrix::argmin");
  }
}

}  // namespace matrix
}  // namespace raft
