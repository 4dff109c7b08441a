// Reduction along the strided axis of a row-major [n_rows x n_cols] matrix:
//     out[j] = final(reduce_i main(x[i][j], i)),        i over rows.
//
// Replaces the reference's three-launch scheme (init map kernel, atomic strided kernel,
// final map kernel: linalg/detail/strided_reduction.cuh:27-121, 142, 194-195) by
//
//  col_partial_kernel   grid (column tiles, row ranges). A CTA is TX x TY threads; a thread
//                       owns VEC adjacent columns (one 16-byte load per row) and walks down
//                       its rows with U loads in flight. Rows of a narrow matrix are
//                       contiguous, so for n_cols*sizeof <= 512 B a warp's load covers
//                       several whole rows. The TY partials per column are folded through
//                       shared memory in a fixed order and written to
//                       partial[row_range][n_cols] - no atomics, bit-reproducible.
//  col_finalize_kernel  folds the row-range partials in order, applies init (once),
//                       inplace and final_op, and writes out[j].
// When a single row range suffices the first kernel writes the finished output itself.
#pragma once

#include "common.cuh"
#include "ops.cuh"

namespace raft_b200 {
namespace detail {

template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          int VEC,
          int U,
          int TPB>
__global__ void __launch_bounds__(TPB, 4) col_partial_kernel(OutT* __restrict__ out,
                                                         typename state_for<OutT, ReduceOp>::type::carry_t* __restrict__ partial,
                                                         const InT* __restrict__ data,
                                                         int64_t n_rows,
                                                         int64_t n_cols,
                                                         int64_t ld,
                                                         OutT init,
                                                         bool inplace,
                                                         MainOp main_op,
                                                         ReduceOp reduce_op,
                                                         FinalOp final_op,
                                                         int TX,
                                                         int64_t rows_per_cta)
{
  grid_dep_sync();
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  State* s_part = reinterpret_cast<State*>(smem_raw);  // [TY][TX*VEC]

  const int TY        = TPB / TX;
  const int tx        = threadIdx.x & (TX - 1);
  const int ty        = threadIdx.x / TX;
  const int64_t col0  = (int64_t(blockIdx.x) * TX + tx) * VEC;
  const bool active   = col0 < n_cols;  // VEC divides n_cols on the vector path
  const int64_t r_beg = int64_t(blockIdx.y) * rows_per_cta;
  int64_t r_end       = r_beg + rows_per_cta;
  r_end               = r_end < n_rows ? r_end : n_rows;
  const bool direct   = gridDim.y == 1;

  State st[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    if constexpr (isSum) {
      st[e].init(OutT(0));
    } else {
      st[e].init(init);
    }
  }

  if (active) {
    const InT* cp = data + col0;
    int64_t r     = r_beg + ty;
    for (; r + int64_t(U - 1) * TY < r_end; r += int64_t(U) * TY) {
      VecOf<InT, VEC> v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        v[u] = load_stream<InT, VEC>(cp + (r + int64_t(u) * TY) * ld);
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          st[e].push(OutT(main_op(v[u].e[e], IdxT(r + int64_t(u) * TY))), reduce_op);
      }
    }
    for (; r < r_end; r += TY) {
      VecOf<InT, VEC> v = load_stream<InT, VEC>(cp + r * ld);
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        st[e].push(OutT(main_op(v.e[e], IdxT(r))), reduce_op);
    }
  }

  const int W = TX * VEC;
#pragma unroll
  for (int e = 0; e < VEC; ++e)
    s_part[ty * W + tx * VEC + e] = st[e];
  __syncthreads();

  for (int j = threadIdx.x; j < W; j += TPB) {
    const int64_t col = int64_t(blockIdx.x) * W + j;
    if (col < n_cols) {
      State r = s_part[j];
      for (int y = 1; y < TY; ++y)
        r.merge(s_part[y * W + j], reduce_op);
      if (direct) {
        if constexpr (isSum) { r.push(init, reduce_op); }
        OutT v = r.value();
        if (inplace) v = reduce_op(out[col], v);
        out[col] = final_op(v);
      } else {
        partial[int64_t(blockIdx.y) * n_cols + col] = r.carry();
      }
    }
  }
}

// One warp per column: the lanes fold the row-range partials p = lane, lane + 32, ... (loads of
// different lanes and steps are independent), then a butterfly merges the 32 lane states. The
// order is fixed, so the result is reproducible.
template <typename OutT, typename ReduceOp, typename FinalOp, int TPB>
__global__ void __launch_bounds__(TPB) col_finalize_kernel(OutT* __restrict__ out,
                                                          const typename state_for<OutT, ReduceOp>::type::carry_t* __restrict__ partial,
                                                          int n_parts,
                                                          int64_t n_cols,
                                                          OutT init,
                                                          bool inplace,
                                                          ReduceOp reduce_op,
                                                          FinalOp final_op,
                                                          const int* __restrict__ cta_status = nullptr)
{
  grid_dep_sync();
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  const int lane       = threadIdx.x & 31;
  const int64_t col    = int64_t(blockIdx.x) * (TPB / 32) + (threadIdx.x >> 5);
  if (col >= n_cols) return;
  State st;
  if constexpr (isSum) {
    st.init(lane == 0 ? init : OutT(0));  // init enters a sum once
  } else {
    st.init(init);
  }
  int gave_up = 0;
  for (int p = lane; p < n_parts; p += 32) {
    st.push_carry(partial[int64_t(p) * n_cols + col], reduce_op);
    if (cta_status != nullptr) gave_up |= cta_status[p];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    State got = shfl_xor_any(st, off);
    st.merge(got, reduce_op);
    gave_up |= __shfl_xor_sync(0xffffffffu, gave_up, off);
  }
  if (lane == 0) {
    OutT v = st.value();
    if constexpr (std::is_floating_point<OutT>::value) {
      if (gave_up != 0) v = OutT(NAN);  // a producer CTA abandoned a bounded wait: make it visible
    }
    if (inplace) v = reduce_op(out[col], v);
    out[col] = final_op(v);
  }
}

}  // namespace detail
}  // namespace raft_b200
