// Device matrix / vector views for the stand-alone build, on cuda::std::mdspan (reference:
// core/mdspan_types.hpp:22-37, core/device_mdspan.hpp:76-98, 153-157, 173, 223). Same names, template
// parameters and factory functions; the accessor is the default one.
#pragma once
#include <cuda/std/mdspan>

#include <cstddef>
#include <cstdint>

namespace raft {

using row_major = cuda::std::layout_right;
using col_major = cuda::std::layout_left;

template <typename IndexType>
using matrix_extent = cuda::std::extents<IndexType, cuda::std::dynamic_extent, cuda::std::dynamic_extent>;
template <typename IndexType>
using vector_extent = cuda::std::extents<IndexType, cuda::std::dynamic_extent>;

template <typename IndexType>
using scalar_extent = cuda::std::extents<IndexType, 1>;

template <typename T, typename Extents, typename Layout = row_major>
using device_mdspan = cuda::std::mdspan<T, Extents, Layout>;

template <typename T, typename IndexType = std::uint32_t, typename Layout = row_major>
using device_matrix_view = device_mdspan<T, matrix_extent<IndexType>, Layout>;

template <typename T, typename IndexType = std::uint32_t, typename Layout = row_major>
using device_vector_view = device_mdspan<T, vector_extent<IndexType>, Layout>;

template <typename T, typename IndexType = std::uint32_t>
using device_scalar_view = device_mdspan<T, scalar_extent<IndexType>>;

template <typename T, typename IndexType = std::uint32_t>
auto make_device_scalar_view(T* ptr)
{
  return device_scalar_view<T, IndexType>{ptr, scalar_extent<IndexType>{}};
}

template <typename T, typename IndexType = std::uint32_t, typename Layout = row_major>
auto make_device_matrix_view(T* ptr, IndexType n_rows, IndexType n_cols)
{
  return device_matrix_view<T, IndexType, Layout>(ptr, n_rows, n_cols);
}

template <typename T, typename IndexType = std::uint32_t, typename Layout = row_major>
auto make_device_vector_view(T* ptr, IndexType n)
{
  return device_vector_view<T, IndexType, Layout>(ptr, n);
}

// view of the same elements as const
template <typename T, typename Extents, typename Layout>
auto make_const_mdspan(cuda::std::mdspan<T, Extents, Layout> m)
{
  return cuda::std::mdspan<const T, Extents, Layout>(m.data_handle(), m.mapping());
}

}  // namespace raft
