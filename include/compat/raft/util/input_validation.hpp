// is_row_or_column_major for the stand-alone build (reference: util/input_validation.hpp:12-30):
// true for layout_right / layout_left views, evaluated from the strides for layout_stride.
#pragma once
#include <raft/core/device_mdspan.hpp>

namespace raft {

template <typename T, typename E, typename L>
constexpr bool is_row_or_column_major(cuda::std::mdspan<T, E, L>)
{
  return false;
}
template <typename T, typename E>
constexpr bool is_row_or_column_major(cuda::std::mdspan<T, E, cuda::std::layout_left>)
{
  return true;
}
template <typename T, typename E>
constexpr bool is_row_or_column_major(cuda::std::mdspan<T, E, cuda::std::layout_right>)
{
  return true;
}
template <typename T, typename E>
constexpr bool is_row_or_column_major(cuda::std::mdspan<T, E, cuda::std::layout_stride> m)
{
  return (m.stride(1) == 1 && m.stride(0) == m.extent(1)) || (m.stride(0) == 1 && m.stride(1) == m.extent(0));
}

}  // namespace raft
