// Row reduction of SHORT contiguous rows with TMA-staged shared-memory tiles.
//
// Rows of a contiguous row-major matrix (ld == row length) that are at most 2 KB long are
// reduced by sub-warps exactly as in row_reduce_kernel<kRows> - G lanes per row, U rows per
// group at a time, transposing sub-warp reduction, packed store - but the rows come out of a
// ring of shared-memory tiles that one producer thread fills with bulk asynchronous copies
// (cp.async.bulk + mbarrier), T consecutive rows = one contiguous block per copy. The bytes in
// flight per SM are then (stages x tile) regardless of register pressure, and the consumer warps
// spend no instruction on global addressing or on waiting for a global load.
// All mbarrier waits are bounded (see col_reduce_tma.cuh); a CTA whose wait runs out stops,
// drains its copies in flight and writes NaN to the floating-point outputs it did not finish.
#pragma once

#include "col_reduce_tma.cuh"
#include "row_reduce.cuh"

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
          typename StoreT = OutT>
__global__ void __launch_bounds__(kTmaThreads, 4) row_reduce_tma_kernel(StoreT* __restrict__ out,
                                                                       const InT* __restrict__ data,
                                                                       int64_t n_rows,
                                                                       int row_len,
                                                                       OutT init,
                                                                       bool inplace,
                                                                       MainOp main_op,
                                                                       ReduceOp reduce_op,
                                                                       FinalOp final_op,
                                                                       int G,
                                                                       int tile_rows,
                                                                       int64_t rows_per_cta,
                                                                       int STAGES,
                                                                       int* __restrict__ status)
{
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  extern __shared__ __align__(128) unsigned char smem_tma[];
  __shared__ __align__(8) uint64_t s_full[kTmaMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kTmaMaxStages];
  __shared__ int s_abort;

  const size_t row_bytes    = size_t(row_len) * sizeof(InT);
  const size_t stage_stride = (size_t(tile_rows) * row_bytes + 127) / 128 * 128;
  const int tid             = threadIdx.x;
  const bool producer       = tid >= kTmaConsumers;
  const int64_t r_beg       = int64_t(blockIdx.x) * rows_per_cta;
  int64_t r_end             = r_beg + rows_per_cta;
  r_end                     = r_end < n_rows ? r_end : n_rows;
  const int64_t rows        = r_end > r_beg ? r_end - r_beg : 0;
  const int n_tiles         = int((rows + tile_rows - 1) / tile_rows);

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], kTmaConsumers / 32);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  volatile int* abort_flag = &s_abort;

  if (producer) {
    if (tid == kTmaConsumers) {
      int issued = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int s          = t % STAGES;
        const unsigned phase = (t / STAGES) & 1u;
        if (!mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag)) break;
        const int64_t row0 = r_beg + int64_t(t) * tile_rows;
        const int64_t nr   = (r_end - row0) < tile_rows ? (r_end - row0) : tile_rows;
        const unsigned nb  = unsigned(size_t(nr) * row_bytes);
        mbar_expect_tx(&s_full[s], nb);
        bulk_load(smem_tma + s * stage_stride, reinterpret_cast<const unsigned char*>(data) + size_t(row0) * row_bytes,
                  nb, &s_full[s]);
        issued = t + 1;
      }
      if (*abort_flag != 0) {
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int t = first; t < issued; ++t) {
          unsigned spin = 0;
          while (!mbar_try_wait(&s_full[t % STAGES], (t / STAGES) & 1u) && ++spin < kSpinLimit) {}
        }
        if (status != nullptr) atomicExch(status, 1);
      }
    }
    return;
  }

  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int lg   = 31 - __clz(G);
  const int lig  = lane & (G - 1);
  const int grp  = lane >> lg;
  const int gsh  = 5 - lg;
  const int gpw  = 1 << gsh;
  const int nvec = row_len / VEC;
  const int rows_per_batch = U * gpw;
  const SubwarpLayout lay  = subwarp_layout<U>(lig, G);

  int t = 0;
  for (; t < n_tiles; ++t) {
    const int s          = t % STAGES;
    const unsigned phase = (t / STAGES) & 1u;
    if (!mbar_wait_bounded(&s_full[s], phase, abort_flag)) break;
    const int64_t tile_row0 = r_beg + int64_t(t) * tile_rows;
    const int nr            = int((r_end - tile_row0) < tile_rows ? (r_end - tile_row0) : tile_rows);
    const unsigned char* tile = smem_tma + s * stage_stride;
    const int n_batches       = (nr + rows_per_batch - 1) / rows_per_batch;
    for (int b = warp; b < n_batches; b += kTmaConsumers / 32) {
      const int lrow0 = b * rows_per_batch + grp;  // slot u -> tile row lrow0 + u*gpw
      const int left  = nr - lrow0;
      const int slots = (left + gpw - 1) >> gsh;
      const int valid = left <= 0 ? 0 : (slots < U ? slots : U);
      const unsigned char* base = tile + size_t(valid > 0 ? lrow0 : nr - 1) * row_bytes;
      const size_t step         = valid > 0 ? size_t(gpw) * row_bytes : 0;
      State st[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        init_state<OutT, State, isSum>(st[u], init, lig == 0);
      for (int c = lig; c < nvec; c += G) {
        VecOf<InT, VEC> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int uu = u < valid ? u : (valid > 0 ? valid - 1 : 0);
          v[u] = *reinterpret_cast<const VecOf<InT, VEC>*>(base + uu * step + size_t(c) * VEC * sizeof(InT));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            push_element<OutT, IdxT>(st[u], v[u].e[e], c * VEC + e, main_op, reduce_op);
        }
      }
      subwarp_transpose_reduce<U>(st, lig, G, reduce_op);
      if (lay.writer) {
#pragma unroll
        for (int i = 0; i < U; ++i) {
          if (i < lay.n_final) {
            const int slot  = lay.prefix * lay.n_final + i;
            const int lr    = lrow0 + slot * gpw;
            if (lr < nr) {
              const int64_t r = tile_row0 + lr;
              OutT v          = st[i].value();
              if constexpr (std::is_same<StoreT, OutT>::value) {
                if (inplace) v = reduce_op(out[r], v);
              }
              out[r] = final_op(v);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s_empty[s]);
  }
  if (t < n_tiles) {
    // a bounded wait ran out: make it visible - the rows this warp did not finish become NaN
    if constexpr (std::is_floating_point<StoreT>::value) {
      for (int64_t r = r_beg + int64_t(t) * tile_rows + tid; r < r_end; r += kTmaConsumers)
        out[r] = StoreT(NAN);
    }
  }
}

}  // namespace detail
}  // namespace raft_b200
