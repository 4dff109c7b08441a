// raft::linalg::rowNorm / colNorm / norm on the B200 kernels (reference: linalg/norm.cuh:45-59,
// 76-90, 112-148; functor choice linalg/detail/norm.cuh:17-61): L1 = (abs, add), L2 = (sq, add) -
// the SQUARED norm unless fin_op takes the root -, Linf = (abs, max); init 0, never in place;
// any other norm type throws.
#pragma once

#include "norm_types.hpp"
#include "reduce.cuh"

namespace raft {
namespace linalg {

namespace b200 {
template <NormType norm_type, bool rowMajor, bool alongRows, typename Type, typename IdxType, typename Lambda, typename OutType>
void norm_impl(OutType* dots, const Type* data, IdxType D, IdxType N, cudaStream_t stream, Lambda fin_op)
{
  if constexpr (norm_type == L1Norm) {
    raft::linalg::reduce<rowMajor, alongRows, Type, OutType, IdxType>(
      dots, data, D, N, OutType(0), stream, false, raft::abs_op(), raft::add_op(), fin_op);
  } else if constexpr (norm_type == L2Norm) {
    raft::linalg::reduce<rowMajor, alongRows, Type, OutType, IdxType>(
      dots, data, D, N, OutType(0), stream, false, raft::sq_op(), raft::add_op(), fin_op);
  } else if constexpr (norm_type == LinfNorm) {
    raft::linalg::reduce<rowMajor, alongRows, Type, OutType, IdxType>(
      dots, data, D, N, OutType(0), stream, false, raft::abs_op(), raft::max_op(), fin_op);
  } else {
    THROW("Unsupported norm type: %d", int(norm_type));
  }
}
}  // namespace b200

/** Norm of every row: dots has N entries (D columns, N rows). */
template <NormType norm_type,
          bool rowMajor,
          typename Type,
          typename IdxType = int,
          typename Lambda  = raft::identity_op,
          typename OutType = Type>
void rowNorm(OutType* dots, const Type* data, IdxType D, IdxType N, cudaStream_t stream, Lambda fin_op = raft::identity_op())
{
  b200::norm_impl<norm_type, rowMajor, true>(dots, data, D, N, stream, fin_op);
}

/** Norm of every column: dots has D entries. */
template <NormType norm_type,
          bool rowMajor,
          typename Type,
          typename IdxType = int,
          typename Lambda  = raft::identity_op,
          typename OutType = Type>
void colNorm(OutType* dots, const Type* data, IdxType D, IdxType N, cudaStream_t stream, Lambda fin_op = raft::identity_op())
{
  b200::norm_impl<norm_type, rowMajor, false>(dots, data, D, N, stream, fin_op);
}

template <NormType norm_type,
          raft::Apply apply,
          typename ElementType,
          typename OutputType,
          typename LayoutPolicy,
          typename IndexType,
          typename Lambda = raft::identity_op>
void norm(raft::resources const& handle,
          raft::device_matrix_view<const ElementType, IndexType, LayoutPolicy> in,
          raft::device_vector_view<OutputType, IndexType> out,
          Lambda fin_op = raft::identity_op())
{
  RAFT_EXPECTS(raft::is_row_or_column_major(in), "Input must be contiguous");
  constexpr bool row_major  = std::is_same<LayoutPolicy, raft::row_major>::value;
  constexpr bool along_rows = apply == raft::Apply::ALONG_ROWS;
  if constexpr (along_rows) {
    RAFT_EXPECTS(static_cast<IndexType>(out.size()) == in.extent(0),
                 "Output should be equal to number of rows in Input");
    rowNorm<norm_type, row_major>(out.data_handle(), in.data_handle(), in.extent(1), in.extent(0),
                                  resource::get_cuda_stream(handle), fin_op);
  } else {
    RAFT_EXPECTS(static_cast<IndexType>(out.size()) == in.extent(1),
                 "Output should be equal to number of columns in Input");
    colNorm<norm_type, row_major>(out.data_handle(), in.data_handle(), in.extent(1), in.extent(0),
                                  resource::get_cuda_stream(handle), fin_op);
  }
}

}  // namespace linalg
}  // namespace raft
