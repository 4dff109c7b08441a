// Row reduction of contiguous rows that do NOT start on 16-byte boundaries (odd widths), staged
// through shared memory.
//
// A global load can only be as wide as the alignment of a row, so a kernel that reads such rows
// directly is left with 4-byte loads. Whole blocks of rows, however, are 16-byte aligned: with
// m = 16 / gcd(16, row bytes), every m-th row starts on a boundary, and a block of a multiple of m
// rows is a multiple of 16 bytes long. One producer thread copies such blocks into a ring of
// shared-memory stages with cp.async.bulk (no register, no alignment concern per row), and the
// consumers read single elements out of shared memory, where alignment costs nothing: G lanes per
// row (G = 1 while 256 rows fit a tile - 48 fp32: a lane sums its row alone, no shuffle at all), lanes of a
// warp on consecutive rows, so that for an odd row length all 32 lanes hit different banks.
// The results of a warp are consecutive rows: one coalesced store.
//
// Rows that DO start on 16-byte boundaries take the same route with 16-byte shared-memory loads
// (VEC elements each) when their length fits the direct kernels badly (lane groups are powers of
// two there; a row of, say, 24 or 100 vectors leaves a quarter of the load slots empty). Where the
// row pitch would put the lanes of a warp into the same banks, every row slot starts a little
// further into its row and wraps around (`rot` vectors per slot, chosen by the host): a reduction
// does not care in which order the elements of a row arrive, and main_op still gets each element's
// true column.
//
// Every mbarrier wait is bounded (see col_reduce_tma.cuh); a CTA whose wait runs out stops, drains
// its copies in flight and writes NaN to the floating-point outputs it did not finish.
#pragma once

#include "col_reduce_tma.cuh"
#include "row_reduce.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kStagedShortRow = 8;  // rows up to this many elements: four rows per lane at a time

template <typename InT, typename OutT, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp, int VEC,
          typename StoreT = OutT>
__global__ void __launch_bounds__(kTmaThreads, 2) row_reduce_staged_kernel(StoreT* __restrict__ out,
                                                                          const InT* __restrict__ data,
                                                                          int64_t n_rows,
                                                                          int row_len,
                                                                          OutT init,
                                                                          bool inplace,
                                                                          MainOp main_op,
                                                                          ReduceOp reduce_op,
                                                                          FinalOp final_op,
                                                                          int G,
                                                                          int rot,
                                                                          int tile_rows,
                                                                          int64_t rows_per_cta,
                                                                          int STAGES,
                                                                          RingCtl ctl)
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
  grid_dep_sync();  // the set-up above touches shared memory only
  volatile int* abort_flag = &s_abort;

  if (producer) {
    if (tid == kTmaConsumers) {
      int issued = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int s          = t % STAGES;
        const unsigned phase = (t / STAGES) & 1u;
        if (!mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag, ctl.limit_ns)) break;
        if (t == ctl.skip_tile && blockIdx.x == 0) continue;  // test hook: this tile is never requested
        const int64_t row0 = r_beg + int64_t(t) * tile_rows;
        const int64_t nr   = (r_end - row0) < tile_rows ? (r_end - row0) : tile_rows;
        // the host makes n_rows * row_bytes, tile_rows * row_bytes and rows_per_cta * row_bytes
        // multiples of 16, so every copy starts on a boundary and has a legal size
        const unsigned nb  = unsigned(size_t(nr) * row_bytes);
        mbar_expect_tx(&s_full[s], nb);
        bulk_load(smem_tma + s * stage_stride, reinterpret_cast<const unsigned char*>(data) + size_t(row0) * row_bytes,
                  nb, &s_full[s]);
        issued = t + 1;
      }
      producer_wait_released(s_empty, issued, STAGES, abort_flag, ctl.limit_ns);
      if (*abort_flag != 0) {
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int t = first; t < issued; ++t) {
          if (t == ctl.skip_tile && blockIdx.x == 0) continue;
          mbar_drain_bounded(&s_full[t % STAGES], (t / STAGES) & 1u, ctl.limit_ns);
        }
        ring_report_timeout(ctl);
      }
    }
    return;
  }

  using Vec      = VecOf<InT, VEC>;
  const int lane = tid & 31;
  const int lg   = 31 - __clz(G);
  const int lig  = tid & (G - 1);  // lane within the group of a row
  const int slot = tid >> lg;      // row slot of this thread within a pass
  const int rpp  = kTmaConsumers >> lg;  // rows per pass of the CTA
  const int nvec = row_len / VEC;        // VEC divides row_len (VEC = 1 for rows off 16-byte boundaries)
  // every row slot starts `rot` vectors further into its row (and wraps): the host picks rot so that the
  // lanes of a warp, which sit on different rows, fall into different shared-memory banks
  const int shift = rot == 0 ? 0 : int((unsigned(slot) * unsigned(rot)) % unsigned(nvec));
  const int n_full = nvec >> lg;       // vectors that every lane of a group takes
  const int n_rem  = nvec & (G - 1);   // lanes of a group that take one more

  int t = 0;
  RingPos rp{0, 0u};
  for (; t < n_tiles; ++t) {
    const int s          = rp.s;
    const unsigned phase = rp.phase;
    rp.advance(1, STAGES);
    if (!mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns)) break;
    const int64_t tile_row0 = r_beg + int64_t(t) * tile_rows;
    const int nr            = int((r_end - tile_row0) < tile_rows ? (r_end - tile_row0) : tile_rows);
    const Vec* tile         = reinterpret_cast<const Vec*>(smem_tma + s * stage_stride);
    int lr_begin = 0;  // rows of the tile already done by the four-rows-per-lane loop
    if (G == 1 && nvec <= kStagedShortRow && (rot == 0 || (nvec & 3) != 0)) {  // at worst a two-way bank conflict
      // very short rows: a lane works on four rows at a time, so that their dependent chains overlap
      constexpr int R = 4;
      for (; lr_begin + R * kTmaConsumers <= nr; lr_begin += R * kTmaConsumers) {
        const int lr0 = lr_begin;
        State st[R];
        const Vec* row[R];
#pragma unroll
        for (int u = 0; u < R; ++u) {
          const int lr = lr0 + u * kTmaConsumers + tid;
          row[u]       = tile + size_t(lr < nr ? lr : nr - 1) * nvec;
          init_state<OutT, State, isSum>(st[u], init, true);
        }
        for (int c = 0; c < nvec; ++c) {
          Vec v[R];
#pragma unroll
          for (int u = 0; u < R; ++u)
            v[u] = row[u][c];
#pragma unroll
          for (int u = 0; u < R; ++u) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              push_element<OutT, IdxT>(st[u], v[u].e[e], c * VEC + e, main_op, reduce_op);
          }
        }
#pragma unroll
        for (int u = 0; u < R; ++u) {
          const int lr = lr0 + u * kTmaConsumers + tid;
          if (lr < nr) {
            const int64_t r = tile_row0 + lr;
            OutT v          = st[u].value();
            if constexpr (std::is_same<StoreT, OutT>::value) {
              if (inplace) v = reduce_op(out[r], v);
            }
            out[r] = final_op(v);
          }
        }
      }
    }
    {
      // whole warps walk the passes together (the shuffles below need all lanes)
      for (int lr0 = lr_begin; lr0 < nr; lr0 += rpp) {
        const int lr   = lr0 + slot;
        const bool ok  = lr < nr;
        const Vec* row = tile + size_t(ok ? lr : nr - 1) * nvec;
        State st;
        init_state<OutT, State, isSum>(st, init, lig == 0);
        // The lane's vectors: lig, lig + G, ... Steps that every lane of the group has (n_full of them,
        // the same for the whole warp) run four at a time; lanes below n_rem take one more.
        if (rot == 0) {
          int c = lig;
          int j = 0;
          for (; j + 4 <= n_full; j += 4, c += 4 * G) {
            Vec v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              v[k] = row[c + k * G];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
              for (int e = 0; e < VEC; ++e)
                push_element<OutT, IdxT>(st, v[k].e[e], (c + k * G) * VEC + e, main_op, reduce_op);
            }
          }
          for (; j < n_full + (lig < n_rem ? 1 : 0); ++j, c += G) {
            const Vec v = row[c];
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              push_element<OutT, IdxT>(st, v.e[e], c * VEC + e, main_op, reduce_op);
          }
        } else {
          // counted from the slot's starting point, wrapping at the end of the row
          int j = 0;
          for (; j + 4 <= n_full; j += 4) {
            Vec v[4];
            int c[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              c[k] = ((j + k) << lg) + lig + shift;
              c[k] = c[k] >= nvec ? c[k] - nvec : c[k];
              v[k] = row[c[k]];
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
              for (int e = 0; e < VEC; ++e)
                push_element<OutT, IdxT>(st, v[k].e[e], c[k] * VEC + e, main_op, reduce_op);
            }
          }
          for (; j < n_full + (lig < n_rem ? 1 : 0); ++j) {
            int c       = (j << lg) + lig + shift;
            c           = c >= nvec ? c - nvec : c;
            const Vec v = row[c];
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              push_element<OutT, IdxT>(st, v.e[e], c * VEC + e, main_op, reduce_op);
          }
        }
        for (int off = G >> 1; off > 0; off >>= 1) {
          State got = shfl_xor_any(st, off);
          st.merge(got, reduce_op);
        }
        if (ok && lig == 0) {
          const int64_t r = tile_row0 + lr;
          OutT v          = st.value();
          if constexpr (std::is_same<StoreT, OutT>::value) {
            if (inplace) v = reduce_op(out[r], v);
          }
          out[r] = final_op(v);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s_empty[s]);
  }
  if (t < n_tiles) {
    // a bounded wait ran out: make it visible - the rows this CTA did not finish become NaN
    if constexpr (std::is_floating_point<StoreT>::value) {
      for (int64_t r = r_beg + int64_t(t) * tile_rows + tid; r < r_end; r += kTmaConsumers)
        out[r] = StoreT(NAN);
    }
  }
}

}  // namespace detail
}  // namespace raft_b200
