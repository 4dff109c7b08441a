// Column reduction of a WIDE row-major matrix with tiled TMA loads.
//
// The matrix is cut into column blocks of 32 16-byte vectors (128 fp32) and row ranges; a CTA
// owns one (column block, row range) pair. Its producer thread streams boxes of kBoxRows rows x
// one column block through a ring of shared-memory stages with cp.async.bulk.tensor.2d (one
// instruction per 32 KB box, strides and edges handled by the tensor map: what lies outside the
// matrix arrives as zeros); eight consumer warps read the boxes with conflict-free 16-byte
// shared-memory loads - lane = vector of the block, warp = row modulo 8 - and keep the same
// per-column accumulators as col_partial_kernel. Output protocol (partial rows per row range,
// col_finalize_kernel) is that of col_reduce.cuh.
//
// Every mbarrier wait is bounded (see col_reduce_tma.cuh); a CTA that gives up marks its row range
// in cta_status (zeroed by the host before the launch) and the finalize kernel turns it into NaN.
#pragma once

#include "col_reduce.cuh"
#include "tensor_map.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kBoxRows = 64;

template <typename InT, typename OutT, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp, int VEC>
__global__ void __launch_bounds__(kTmaThreads, 1)
  col_partial_tma2d_kernel(OutT* __restrict__ out,
                           typename state_for<OutT, ReduceOp>::type::carry_t* __restrict__ partial,
                           const __grid_constant__ CUtensorMap tmap,
                           int64_t n_rows,
                           int64_t n_cols,
                           OutT init,
                           bool inplace,
                           MainOp main_op,
                           ReduceOp reduce_op,
                           FinalOp final_op,
                           int64_t rows_per_cta,
                           int STAGES,
                           int* __restrict__ cta_status,
                           RingCtl ctl)
{
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  constexpr int BX     = 32 * VEC;                       // columns of a block
  constexpr int TY     = kTmaConsumers / 32;             // 8 row slots
  constexpr size_t kBoxBytes = size_t(kBoxRows) * BX * sizeof(InT);  // 32 KB for 16-byte vectors
  extern __shared__ __align__(128) unsigned char smem_tma[];
  unsigned char* tiles = smem_tma;                                                 // [STAGES][kBoxBytes]
  State* s_part        = reinterpret_cast<State*>(smem_tma + size_t(STAGES) * kBoxBytes);  // [TY][BX]
  __shared__ __align__(8) uint64_t s_full[kTmaMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kTmaMaxStages];
  __shared__ int s_abort;

  const int tid       = threadIdx.x;
  const bool producer = tid >= kTmaConsumers;
  const int tx        = tid & 31;
  const int ty        = tid >> 5;  // consumers: 0..7
  const int64_t col0  = int64_t(blockIdx.x) * BX;
  const int64_t r_beg = int64_t(blockIdx.y) * rows_per_cta;
  int64_t r_end       = r_beg + rows_per_cta;
  r_end               = r_end < n_rows ? r_end : n_rows;
  const int64_t rows  = r_end > r_beg ? r_end - r_beg : 0;
  const int n_tiles   = int((rows + kBoxRows - 1) / kBoxRows);
  const bool direct   = gridDim.y == 1;
  const bool col_ok   = col0 + int64_t(tx) * VEC < n_cols;  // VEC divides n_cols

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], kTmaConsumers / 32);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dep_sync();  // the set-up above touches shared memory only
  volatile int* abort_flag = &s_abort;

  State st[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    if constexpr (isSum) {
      st[e].init(OutT(0));
    } else {
      st[e].init(init);
    }
  }

  if (producer) {
    if (tid == kTmaConsumers) {  // one elected thread issues every copy
      int issued = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int s          = t % STAGES;
        const unsigned phase = (t / STAGES) & 1u;
        if (!mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag, ctl.limit_ns)) break;
        if (t == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) continue;  // test hook: never requested
        mbar_expect_tx(&s_full[s], unsigned(kBoxBytes));  // the whole box, zero fill included
        tma_load_2d(tiles + size_t(s) * kBoxBytes, &tmap, int(col0), int(r_beg + int64_t(t) * kBoxRows), &s_full[s]);
        issued = t + 1;
      }
      producer_wait_released(s_empty, issued, STAGES, abort_flag, ctl.limit_ns);
      if (*abort_flag != 0) {
        // drain: copies already issued must land before the CTA may exit
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int t = first; t < issued; ++t) {
          if (t == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) continue;
          mbar_drain_bounded(&s_full[t % STAGES], (t / STAGES) & 1u, ctl.limit_ns);
        }
        if (cta_status != nullptr) cta_status[blockIdx.y] = 1;
        ring_report_timeout(ctl);
      }
    }
  } else {
    const int lane = tid & 31;
    RingPos rp{0, 0u};
    for (int t = 0; t < n_tiles; ++t) {
      const int s          = rp.s;
      const unsigned phase = rp.phase;
      rp.advance(1, STAGES);
      if (!mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns)) break;
      const int64_t row0 = r_beg + int64_t(t) * kBoxRows;
      const int nr       = int((r_end - row0) < kBoxRows ? (r_end - row0) : kBoxRows);
      if (col_ok) {
        const unsigned char* tile = tiles + size_t(s) * kBoxBytes + size_t(tx) * VEC * sizeof(InT);
        constexpr size_t pitch    = size_t(BX) * sizeof(InT);
        int r = ty;
        for (; r + 3 * TY < nr; r += 4 * TY) {
          VecOf<InT, VEC> v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            v[u] = *reinterpret_cast<const VecOf<InT, VEC>*>(tile + size_t(r + u * TY) * pitch);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              st[e].push(OutT(main_op(v[u].e[e], IdxT(row0 + r + u * TY))), reduce_op);
          }
        }
        for (; r < nr; r += TY) {
          const VecOf<InT, VEC> v = *reinterpret_cast<const VecOf<InT, VEC>*>(tile + size_t(r) * pitch);
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            st[e].push(OutT(main_op(v.e[e], IdxT(row0 + r))), reduce_op);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
    }
  }

  // fold the TY partials per column (same as col_partial_kernel)
  if (!producer) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      s_part[ty * BX + tx * VEC + e] = st[e];
  }
  __syncthreads();
  for (int j = tid; j < BX; j += kTmaThreads) {
    const int64_t c = col0 + j;
    if (c < n_cols) {
      State r = s_part[j];
      for (int y = 1; y < TY; ++y)
        r.merge(s_part[y * BX + j], reduce_op);
      if (direct) {
        if constexpr (isSum) { r.push(init, reduce_op); }
        OutT v = r.value();
        if (inplace) v = reduce_op(out[c], v);
        out[c] = final_op(v);
      } else {
        partial[int64_t(blockIdx.y) * n_cols + c] = r.carry();
      }
    }
  }
}

}  // namespace detail
}  // namespace raft_b200
