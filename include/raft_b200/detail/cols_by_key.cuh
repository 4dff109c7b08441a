// Keyed column sums:  out[r][keys[c]] += data[r][c]   for a row-major [nrows x ncols] matrix.
//
// Counterpart of the reference's cached / direct kernels
// (linalg/detail/reduce_cols_by_key.cuh:23-68, dispatch :89-138). Two algorithms:
//  * staged tiles for large inputs with up to a few hundred keys, no floating-point atomics: sorted column tiles
//    with a warp walking the sorted columns of its keys (cols_by_key_walk.cuh) for matrices of at least 256 rows
//    and up to 32 keys (64 for types other than fp32), a table cell per (key, row) and warp in shared memory
//    without any sort (cols_by_key_table.cuh) for fp32 with 33 to 255 keys, sorted column tiles with a lane per
//    (row, key) segment (cols_by_key_sorted.cuh) otherwise;
//  * the kernels of this file otherwise: a CTA owns a tile of RT rows and a contiguous range of
//    columns, accumulates into a privatised [RT x nkeys] table in shared memory (shared-memory
//    atomics; lanes of a warp read 128 contiguous bytes of one row per step) and flushes the
//    table once. When one CTA covers whole rows the flush is a plain store (no memset, no global
//    atomics); when the columns of a row are split across CTAs the flush uses global atomics on a
//    zeroed output. Tables too large for shared memory fall back to global atomics per element.
#pragma once

#include "common.cuh"
#include "launch.cuh"
#include "cols_by_key_sorted.cuh"
#include "cols_by_key_walk.cuh"
#include "cols_by_key_table.cuh"

namespace raft_b200 {
namespace detail {

template <typename T, typename KeyT>
__global__ void __launch_bounds__(256) cols_by_key_tile_kernel(T* __restrict__ out,
                                                              const T* __restrict__ data,
                                                              const KeyT* __restrict__ keys,
                                                              int64_t nrows,
                                                              int64_t ncols,
                                                              int64_t nkeys,
                                                              int RT,
                                                              int64_t cols_per_cta,
                                                              bool reset)
{
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* acc = reinterpret_cast<T*>(smem_raw);  // [RT][nkeys]

  const int64_t r0 = int64_t(blockIdx.x) * RT;
  int rt           = int(nrows - r0 < RT ? nrows - r0 : RT);
  const int64_t c0 = int64_t(blockIdx.y) * cols_per_cta;
  int64_t c1       = c0 + cols_per_cta;
  c1               = c1 < ncols ? c1 : ncols;
  const bool whole = gridDim.y == 1;

  const int64_t n_acc = int64_t(rt) * nkeys;
  for (int64_t i = threadIdx.x; i < n_acc; i += 256)
    acc[i] = T(0);
  __syncthreads();

  for (int64_t c = c0 + threadIdx.x; c < c1; c += 256) {
    const int64_t k = static_cast<int64_t>(keys[c]);
    const T* p      = data + r0 * ncols + c;
    int rl          = 0;
    for (; rl + 4 <= rt; rl += 4) {
      const T v0 = p[(rl + 0) * ncols];
      const T v1 = p[(rl + 1) * ncols];
      const T v2 = p[(rl + 2) * ncols];
      const T v3 = p[(rl + 3) * ncols];
      atomicAdd(&acc[(rl + 0) * nkeys + k], v0);
      atomicAdd(&acc[(rl + 1) * nkeys + k], v1);
      atomicAdd(&acc[(rl + 2) * nkeys + k], v2);
      atomicAdd(&acc[(rl + 3) * nkeys + k], v3);
    }
    for (; rl < rt; ++rl)
      atomicAdd(&acc[rl * nkeys + k], p[rl * ncols]);
  }
  __syncthreads();

  T* dst = out + r0 * nkeys;
  for (int64_t i = threadIdx.x; i < n_acc; i += 256) {
    const T v = acc[i];
    if (whole) {
      dst[i] = reset ? v : dst[i] + v;
    } else if (v != T(0)) {
      atomicAdd(&dst[i], v);
    }
  }
}

template <typename T, typename KeyT>
__global__ void __launch_bounds__(256) cols_by_key_atomic_kernel(T* __restrict__ out,
                                                                const T* __restrict__ data,
                                                                const KeyT* __restrict__ keys,
                                                                int64_t nrows,
                                                                int64_t ncols,
                                                                int64_t nkeys)
{
  const int64_t total = nrows * ncols;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int64_t r = i / ncols;
    const int64_t c = i - r * ncols;
    atomicAdd(&out[r * nkeys + static_cast<int64_t>(keys[c])], data[i]);
  }
}

// Which staged form a call takes: 0 none (the kernels of this file), 1 a lane per segment, 2 a warp walking its
// keys, 3 a table cell per (key, row) in shared memory without sorting (fp32, 65 to 255 keys).
template <typename T>
inline int cols_by_key_sorted_form(const T* data, int64_t nrows, int64_t ncols, int64_t nkeys, Cbk32Plan* p32,
                                   CbkTablePlan* ptab = nullptr)
{
  // 0: by size, 1: shared-memory atomics, 2: a lane per segment, 3: a warp walking its keys, 4: table cells
  const int algo = tuning().colkey_algo;
  if (algo == 1 || !cols_by_key_sorted_supported<T>(nrows, ncols, nkeys)) return 0;
  const bool preferred = cols_by_key_sorted_preferred<T>(nrows, ncols, nkeys);
  if (algo == 4 || (algo == 0 && preferred && nrows >= 256 && nkeys > tuning().colkey_walk_max_keys &&
                    nkeys <= tuning().colkey_table_max_keys && tensor_map_dtype<T>::supported &&
                    encode_tiled_fn() != nullptr)) {
    const CbkTablePlan p = plan_cols_by_key_table<T>(data, nrows, ncols, nkeys);
    if (p.ok) {
      if (ptab != nullptr) *ptab = p;
      return 3;
    }
  }
  // (types the table form does not take keep the walk up to 64 keys, where it still beats a lane per segment)
  const int walk_max = std::is_same<T, float>::value ? tuning().colkey_walk_max_keys
                                                      : (tuning().colkey_walk_max_keys > 64 ? tuning().colkey_walk_max_keys : 64);
  if (algo == 3 || (algo == 0 && preferred && nrows >= 256 && nkeys <= walk_max)) {
    const Cbk32Plan p = plan_cols_by_key_rows32<T>(data, nrows, ncols, nkeys, tuning().colkey32_ch, tuning().colkey32_rt);
    if (p.ok) {
      if (p32 != nullptr) *p32 = p;
      return 2;
    }
  }
  return (algo == 2 || algo == 3 || preferred) ? 1 : 0;
}

// Scratch the call will use (what a caller passes as workspace to keep it allocation-free): the sorted
// column offsets, the segment starts and - when the columns of a row are split over CTAs - the fp64 tables
// of the sorted-tile algorithm; nothing for the shared-memory-atomics kernels.
template <typename T>
inline size_t cols_by_key_scratch_bytes(const T* data, int64_t nrows, int64_t ncols, int64_t nkeys)
{
  if (nrows <= 0 || ncols <= 0 || nkeys <= 0) return 0;
  Cbk32Plan p32;
  CbkTablePlan ptab;
  const int form = cols_by_key_sorted_form<T>(data, nrows, ncols, nkeys, &p32, &ptab);
  if (form == 3) {  // should the tensor map fail at the call, the lane-per-segment form runs in the same scratch
    const size_t other = plan_cols_by_key_sorted<T>(data, nrows, ncols, nkeys).total;
    return ptab.total > other ? ptab.total : other;
  }
  if (form == 2) return p32.total;
  if (form == 1) return plan_cols_by_key_sorted<T>(data, nrows, ncols, nkeys).total;
  return 0;
}

template <typename T, typename KeyT>
cudaError_t launch_cols_by_key(T* out,
                               const T* data,
                               const KeyT* keys,
                               int64_t nrows,
                               int64_t ncols,
                               int64_t nkeys,
                               bool reset,
                               cudaStream_t stream,
                               Workspace ws = Workspace{})
{
  if (nrows <= 0 || nkeys <= 0) return cudaSuccess;
  cudaError_t e;
  const size_t out_bytes = size_t(nrows) * nkeys * sizeof(T);
  if (ncols <= 0) return reset ? cudaMemsetAsync(out, 0, out_bytes, stream) : cudaSuccess;
  // sorted column tiles where they win (large inputs, a few hundred keys at most)
  {
    Cbk32Plan p32;
    CbkTablePlan ptab;
    int form = cols_by_key_sorted_form<T>(data, nrows, ncols, nkeys, &p32, &ptab);
    if (form == 3) {
      bool unavailable = false;
      e = launch_cols_by_key_table<T, KeyT>(out, data, keys, nrows, ncols, nkeys, reset, stream, ptab, ws, &unavailable);
      if (!unavailable) return e;
      form = 1;
    }
    if (form == 2) return launch_cols_by_key_rows32<T, KeyT>(out, data, keys, nrows, ncols, nkeys, reset, stream, p32, ws);
    if (form == 1) return launch_cols_by_key_sorted<T, KeyT>(out, data, keys, nrows, ncols, nkeys, reset, stream, ws);
  }

  const size_t budget  = size_t(96) << 10;  // two CTAs per SM keep loads in flight across the flush
  const size_t per_row = size_t(nkeys) * sizeof(T);
  const int sms        = sm_count();
  if (per_row > (size_t(200) << 10)) {
    if (reset) {
      e = cudaMemsetAsync(out, 0, out_bytes, stream);
      if (e != cudaSuccess) return e;
    }
    int64_t ctas = ceil_div<int64_t>(nrows * ncols, 256);
    if (ctas > int64_t(sms) * 32) ctas = int64_t(sms) * 32;
    cols_by_key_atomic_kernel<T, KeyT><<<unsigned(ctas), 256, 0, stream>>>(out, data, keys, nrows, ncols, nkeys);
    return cudaGetLastError();
  }
  int64_t RT = per_row <= budget ? int64_t(budget / per_row) : 1;
  if (RT > 32) RT = 32;
  if (RT > nrows) RT = nrows;
  // enough row tiles to fill the machine? otherwise also split the columns
  const int64_t want = int64_t(sms) * 4;
  while (RT > 1 && ceil_div<int64_t>(nrows, RT) < want)
    RT = (RT + 1) / 2;
  const int64_t tiles = ceil_div<int64_t>(nrows, RT);
  int64_t cx          = 1;
  if (tiles < want) {
    cx                   = ceil_div<int64_t>(want, tiles);
    const int64_t max_cx = ceil_div<int64_t>(ncols, 2048);  // at least 8 columns per thread
    if (cx > max_cx) cx = max_cx;
    if (cx < 1) cx = 1;
  }
  int64_t cpc = ceil_div<int64_t>(ncols, cx);
  cpc         = ceil_div<int64_t>(cpc, 256) * 256;
  cx          = ceil_div<int64_t>(ncols, cpc);
  if (cx > 65535) cx = 65535, cpc = ceil_div<int64_t>(ceil_div<int64_t>(ncols, cx), 256) * 256, cx = ceil_div<int64_t>(ncols, cpc);
  if (cx > 1 && reset) {
    e = cudaMemsetAsync(out, 0, out_bytes, stream);
    if (e != cudaSuccess) return e;
  }
  const size_t smem = size_t(RT) * per_row;
  auto kern         = cols_by_key_tile_kernel<T, KeyT>;
  if (smem > (size_t(48) << 10)) {
    e = ensure_dynamic_smem(kern, size_t(smem));
    if (e != cudaSuccess) return e;
  }
  const dim3 grid{unsigned(tiles), unsigned(cx), 1u};
  kern<<<grid, 256, smem, stream>>>(out, data, keys, nrows, ncols, nkeys, int(RT), cpc, reset);
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
