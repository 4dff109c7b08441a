// Tiled TMA (cp.async.bulk.tensor) plumbing: a 2-D tensor map over a row-major matrix, made on
// the host through the driver's cuTensorMapEncodeTiled (looked up at run time, so nothing links
// against libcuda), and the device-side tile load that completes on an mbarrier.
//
// Rules the callers keep (nothing checks them on the device): the matrix base and the row pitch
// are multiples of 16 bytes; the innermost coordinate of a load times the element size is a
// multiple of 16 bytes; the shared-memory destination is 128-byte aligned. Parts of a box that
// lie outside the matrix are filled with zeros and still count towards the barrier's bytes.
#pragma once

#include "col_reduce_tma.cuh"  // mbarrier helpers

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

namespace raft_b200 {
namespace detail {

template <typename T>
struct tensor_map_dtype {
  static constexpr bool supported = false;
};
template <>
struct tensor_map_dtype<float> {
  static constexpr bool supported            = true;
  static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
};
template <>
struct tensor_map_dtype<double> {
  static constexpr bool supported            = true;
  static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT64;
};
template <>
struct tensor_map_dtype<int> {
  static constexpr bool supported            = true;
  static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_INT32;
};
template <>
struct tensor_map_dtype<__half> {
  static constexpr bool supported            = true;
  static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Map of a row-major [n_rows x n_cols] matrix with row pitch `ld` elements; a box is
// box_rows x box_cols elements (each at most 256, box_cols * sizeof(T) a multiple of 16 bytes).
template <typename T>
inline cudaError_t make_tensor_map_2d(CUtensorMap* map,
                                      const T* base,
                                      int64_t n_rows,
                                      int64_t n_cols,
                                      int64_t ld,
                                      int box_rows,
                                      int box_cols)
{
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return cudaErrorNotSupported;
  const cuuint64_t dims[2]    = {cuuint64_t(n_cols), cuuint64_t(n_rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * sizeof(T)};  // bytes, dimensions 1..rank-1
  const cuuint32_t box[2]     = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
  const cuuint32_t estr[2]    = {1u, 1u};
  const CUresult r = fn(map, tensor_map_dtype<T>::value, 2u, const_cast<T*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// One box, top-left element (row y, column x), into shared memory; completes `bytes of a box` on `bar`.
B2R_DI void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
      smem_u32(smem_dst)),
    "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
    : "memory");
}

}  // namespace detail
}  // namespace raft_b200
