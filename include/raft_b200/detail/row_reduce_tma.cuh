// Row reduction of SHORT contiguous rows out of a ring of shared-memory tiles.
//
// Rows of a contiguous row-major matrix (ld == row length) of up to 32 x CPL 16-byte vectors are
// reduced by sub-warps exactly as in row_reduce_kernel<kRows> - G lanes per row, CPL chunks of a
// row per lane, U rows per group at a time (U x CPL = 8 shared-memory loads in flight per lane),
// transposing sub-warp reduction, packed store - but the rows come out of a ring of shared-memory
// tiles that one producer thread fills with bulk asynchronous copies (cp.async.bulk + mbarrier),
// T consecutive rows = one contiguous block per copy. One CTA per SM owns a contiguous range of rows.
//
// Why a second kernel for rows the direct kernel can read: with short rows the work per row besides
// the loads (set-up, the sub-warp reduction, the store) is a large share of a warp's time, and in
// the direct kernel no new load is issued while a warp does that work. Here the producer keeps
// STAGES x tile bytes in flight whatever the consumers do. Measured on 8,388,608 x 64 fp32 row
// argmin: 6.78 TB/s against 6.3-6.5 for the direct kernel. What matters (same measurement):
// tiles of 32 KB (16 KB tiles: 4.8 TB/s - twice the barrier traffic per byte), 4 stages (2: 4.6,
// 6: 6.55 TB/s), one CTA per SM, a consumer team that takes a tile in ONE pass of its 8 warps, and
// two such teams: with 8 consumer warps per SM the kernel is bound by what those warps can issue
// (24 warp-instructions per row of 64 floats, 1.45 per clock: 5.1 TB/s).
//
// All mbarrier waits are bounded (see col_reduce_tma.cuh); a CTA whose wait runs out stops,
// drains its copies in flight, marks `status` and writes NaN to the floating-point outputs it did
// not finish.
#pragma once

#include "col_reduce_tma.cuh"
#include "row_reduce.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kRingTeams = 2;  // teams of 8 consumer warps per CTA of the ring kernel

template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          int VEC,
          int U,
          int CPL,
          int TEAMS,
          typename StoreT = OutT>
__global__ void __launch_bounds__(TEAMS * kTmaConsumers + 32, 1) row_reduce_ring_kernel(StoreT* __restrict__ out,
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
                                                                        RingCtl ctl)
{
  using State          = typename state_for<OutT, ReduceOp>::type;
  using Vec            = VecOf<InT, VEC>;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  extern __shared__ __align__(128) unsigned char smem_tma[];
  __shared__ __align__(8) uint64_t s_full[kTmaMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kTmaMaxStages];
  __shared__ int s_abort;

  const unsigned row_bytes  = unsigned(row_len) * unsigned(sizeof(InT));
  const size_t stage_stride = (size_t(tile_rows) * row_bytes + 127) / 128 * 128;
  const int tid             = threadIdx.x;
  const bool producer       = tid >= TEAMS * kTmaConsumers;
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
    if (tid == TEAMS * kTmaConsumers) {
      int issued = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int s          = t % STAGES;
        const unsigned phase = (t / STAGES) & 1u;
        if (!mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag, ctl.limit_ns)) break;
        if (t == ctl.skip_tile && blockIdx.x == 0) continue;  // test hook: this tile is never requested
        const int64_t row0 = r_beg + int64_t(t) * tile_rows;
        const int64_t nr   = (r_end - row0) < tile_rows ? (r_end - row0) : tile_rows;
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

  // TEAMS teams of 8 consumer warps take the tiles in turn (a team owns a whole tile): with short rows the
  // consumers are bound by instruction issue, and a second team doubles what an SM can issue for them.
  // STAGES must be a multiple of TEAMS, so that a stage is always served by the same team: a waiter may be
  // at most one phase behind its barrier, and a team that skips tiles would get two phases ahead of a stage
  // it shares with a slower team.
  const int lane = tid & 31;
  const int warp = (tid >> 5) & (kTmaConsumers / 32 - 1);
  const int team = tid / kTmaConsumers;
  const int lg   = 31 - __clz(G);
  const int lig  = lane & (G - 1);
  const int grp  = lane >> lg;
  const int gsh  = 5 - lg;
  const int gpw  = 1 << gsh;
  const int nvec = row_len / VEC;
  const int rows_per_batch = U * gpw;
  const bool exact         = nvec == G * CPL;  // every lane of a group holds CPL whole chunks
  const SubwarpLayout lay  = subwarp_layout<U>(lig, G);
  const unsigned step_full = unsigned(gpw) * row_bytes;

  int t = team;
  RingPos rp{team, 0u};  // STAGES is a multiple of TEAMS
  for (; t < n_tiles; t += TEAMS) {
    const int s          = rp.s;
    const unsigned phase = rp.phase;
    rp.advance(TEAMS, STAGES);
    if (!mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns)) break;
    const int64_t tile_row0 = r_beg + int64_t(t) * tile_rows;
    const int nr            = int((r_end - tile_row0) < tile_rows ? (r_end - tile_row0) : tile_rows);
    const unsigned char* tile = smem_tma + s * stage_stride;
    const int n_batches       = (nr + rows_per_batch - 1) / rows_per_batch;
    for (int b = warp; b < n_batches; b += kTmaConsumers / 32) {
      const int lrow0 = b * rows_per_batch + grp;  // slot u -> tile row lrow0 + u * gpw
      const int left  = nr - lrow0;
      const int slots = (left + gpw - 1) >> gsh;
      const int valid = left <= 0 ? 0 : (slots < U ? slots : U);
      State st[U];
      constexpr bool kWalk = kvp_walk<State, MainOp, ReduceOp>::value;  // see row_reduce.cuh
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if constexpr (kWalk) {
          st[u].v.key   = kvp_largest_key<decltype(st[u].v.key)>();
          st[u].v.value = init.value;
        } else {
          init_state<OutT, State, isSum>(st[u], init, lig == 0);
        }
      }
      Vec v[U][CPL];
      if (valid == U && exact) {
        const unsigned char* base = tile + unsigned(lrow0) * row_bytes + unsigned(lig) * unsigned(sizeof(Vec));
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int k = 0; k < CPL; ++k)
            v[u][k] = *reinterpret_cast<const Vec*>(base + u * step_full + unsigned(k * G) * unsigned(sizeof(Vec)));
        }
        if constexpr (kWalk) {
          kvp_walk_rows<kvp_walk<State, MainOp, ReduceOp>::is_min>(st, v, lig * VEC, G * VEC, init.value);
        } else {
#pragma unroll
          for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
#pragma unroll
              for (int e = 0; e < VEC; ++e)
                push_element<OutT, IdxT>(st[u], v[u][k].e[e], (lig + k * G) * VEC + e, main_op, reduce_op);
            }
          }
        }
      } else {
        // ragged batch (fewer than U real rows in the tile) or a row length below G x CPL chunks:
        // slots and chunks that do not exist re-read one that does and are ignored
        const unsigned char* base = tile + unsigned(valid > 0 ? lrow0 : nr - 1) * row_bytes;
        const unsigned step       = valid > 0 ? step_full : 0u;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int uu = u < valid ? u : (valid > 0 ? valid - 1 : 0);
#pragma unroll
          for (int k = 0; k < CPL; ++k) {
            const int c  = lig + k * G;
            const int cc = c < nvec ? c : 0;
            v[u][k]      = *reinterpret_cast<const Vec*>(base + uu * step + unsigned(cc) * unsigned(sizeof(Vec)));
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int k = 0; k < CPL; ++k) {
            if (lig + k * G < nvec) {
#pragma unroll
              for (int e = 0; e < VEC; ++e)
                push_element<OutT, IdxT>(st[u], v[u][k].e[e], (lig + k * G) * VEC + e, main_op, reduce_op);
            }
          }
        }
      }
      subwarp_transpose_reduce<U>(st, lig, G, reduce_op);
      if (lay.writer) {
#pragma unroll
        for (int i = 0; i < U; ++i) {
          if (i < lay.n_final) {
            const int slot = lay.prefix * lay.n_final + i;
            const int lr   = lrow0 + slot * gpw;
            if (lr < nr) {
              const int64_t r = tile_row0 + lr;
              OutT val        = st[i].value();
              if constexpr (kWalk) val = reduce_op(init, val);  // the lanes started from {largest key, init.value}
              if constexpr (std::is_same<StoreT, OutT>::value) {
                if (inplace) val = reduce_op(out[r], val);
              }
              out[r] = final_op(val);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s_empty[s]);
  }
  if (t < n_tiles) {
    // a bounded wait ran out: make it visible - the rows this CTA did not finish become NaN
    if constexpr (std::is_floating_point<StoreT>::value) {
      for (int64_t r = r_beg + int64_t(t) * tile_rows + (tid & (kTmaConsumers - 1)); r < r_end; r += kTmaConsumers)
        out[r] = StoreT(NAN);
    }
  }
}

// Few, very long rows (the "thick" case of the reference, coalesced_reduction-inl.cuh:481-533, and the
// full-array reductions built on it): a row is cut into segments, one CTA per (segment, row) as in
// row_split_kernel, but the segment comes through a ring of 32 KB bulk copies and the 256 consumers sum
// straight out of shared memory - a CTA keeps 128 KB in flight without a register, which is what lets a
// pure read run at 7.2-7.3 TB/s on this part where 16-byte loads stop at 6.3-6.5. The segment's partial
// goes to partial[row * n_seg + seg] (row_finalize_kernel folds them), or straight to `out` when the row
// has one segment. A row length that is no multiple of the vector: the last segment's consumers take the tail
// from global memory. Waits are bounded as everywhere (col_reduce_tma.cuh).
template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          int VEC,
          typename StoreT = OutT>
__global__ void __launch_bounds__(kTmaThreads, 1)
  row_split_ring_kernel(StoreT* __restrict__ out,
                        typename state_for<OutT, ReduceOp>::type::carry_t* __restrict__ partial,
                        const InT* __restrict__ data,
                        int64_t n_rows,
                        int64_t row_len,
                        int64_t ld,
                        OutT init,
                        bool inplace,
                        MainOp main_op,
                        ReduceOp reduce_op,
                        FinalOp final_op,
                        int64_t seg_vecs,
                        int tile_vecs,
                        int STAGES,
                        RingCtl ctl)
{
  using State          = typename state_for<OutT, ReduceOp>::type;
  using Vec            = VecOf<InT, VEC>;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  extern __shared__ __align__(128) unsigned char smem_tma[];
  __shared__ __align__(8) uint64_t s_full[kTmaMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kTmaMaxStages];
  __shared__ int s_abort;
  __shared__ State s_warp[kTmaConsumers / 32];

  const int tid        = threadIdx.x;
  const bool producer  = tid >= kTmaConsumers;
  const int n_seg      = gridDim.x;
  const int seg        = blockIdx.x;
  const int64_t nvec   = row_len / VEC;
  const int64_t v0     = int64_t(seg) * seg_vecs;
  int64_t v1           = v0 + seg_vecs;
  v1                   = v1 < nvec ? v1 : nvec;
  const int64_t n_v    = v1 > v0 ? v1 - v0 : 0;
  const int tiles_row  = int((n_v + tile_vecs - 1) / tile_vecs);  // tiles of one row's segment
  const bool direct    = n_seg == 1;
  const size_t stage_stride = size_t(tile_vecs) * sizeof(Vec);

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
      long long issued = 0;
      bool alive       = true;
      for (int64_t row = blockIdx.y; row < n_rows && alive; row += gridDim.y) {
        const Vec* rp = reinterpret_cast<const Vec*>(data + row * ld) + v0;
        for (int t = 0; t < tiles_row; ++t) {
          const int s          = int(issued % STAGES);
          const unsigned phase = unsigned(issued / STAGES) & 1u;
          if (!mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag, ctl.limit_ns)) {
            alive = false;
            break;
          }
          if (issued == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) {  // test hook: never requested
            ++issued;
            continue;
          }
          const int64_t left = n_v - int64_t(t) * tile_vecs;
          const unsigned nb  = unsigned((left < tile_vecs ? left : tile_vecs) * int64_t(sizeof(Vec)));
          mbar_expect_tx(&s_full[s], nb);
          bulk_load(smem_tma + s * stage_stride, rp + int64_t(t) * tile_vecs, nb, &s_full[s]);
          ++issued;
        }
      }
      if (alive) producer_wait_released(s_empty, issued, STAGES, abort_flag, ctl.limit_ns);
      if (*abort_flag != 0) {
        const long long first = issued > STAGES ? issued - STAGES : 0;
        for (long long t = first; t < issued; ++t) {
          if (t == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) continue;
          mbar_drain_bounded(&s_full[t % STAGES], unsigned(t / STAGES) & 1u, ctl.limit_ns);
        }
        ring_report_timeout(ctl);
      }
    }
    return;
  }

  const int lane = tid & 31;
  const int warp = tid >> 5;
  long long seq  = 0;
  bool dead      = false;
  RingPos rp{0, 0u};
  for (int64_t row = blockIdx.y; row < n_rows; row += gridDim.y) {
    constexpr int U = 4;
    State st[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      init_state<OutT, State, isSum>(st[u], init, direct && tid == 0 && u == 0);
    for (int t = 0; t < tiles_row; ++t, ++seq) {
      if (dead) continue;
      const int s          = rp.s;
      const unsigned phase = rp.phase;
      rp.advance(1, STAGES);
      if (!mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns)) {
        dead = true;
        continue;
      }
      const Vec* tile    = reinterpret_cast<const Vec*>(smem_tma + s * stage_stride);
      const int64_t base = v0 + int64_t(t) * tile_vecs;  // vector index of the tile's first vector in the row
      const int64_t left = n_v - int64_t(t) * tile_vecs;
      const int nt       = int(left < tile_vecs ? left : tile_vecs);
      int c              = tid;
      for (; c + (U - 1) * kTmaConsumers < nt; c += U * kTmaConsumers) {
        Vec v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = tile[c + u * kTmaConsumers];
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            st[u].push(OutT(main_op(v[u].e[e], IdxT((base + c + u * kTmaConsumers) * VEC + e))), reduce_op);
        }
      }
      for (; c < nt; c += kTmaConsumers) {
        const Vec v = tile[c];
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          st[0].push(OutT(main_op(v.e[e], IdxT((base + c) * VEC + e))), reduce_op);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
    }
    if constexpr (VEC > 1) {
      // a row length that is no multiple of the vector width: the last segment takes the tail
      if (seg == n_seg - 1) {
        const InT* rp = data + row * ld;
        for (int64_t i = nvec * VEC + tid; i < row_len; i += kTmaConsumers)
          st[0].push(OutT(main_op(rp[i], IdxT(i))), reduce_op);
      }
    }
#pragma unroll
    for (int u = 1; u < U; ++u)
      st[0].merge(st[u], reduce_op);
    // the 8 consumer warps meet (named barrier: the producer warp is not part of it)
    State r = st[0];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      State got = shfl_xor_any(r, off);
      r.merge(got, reduce_op);
    }
    if (lane == 0) s_warp[warp] = r;
    asm volatile("bar.sync 1, %0;" ::"n"(kTmaConsumers) : "memory");
    if (tid == 0) {
      State tot = s_warp[0];
      for (int w = 1; w < kTmaConsumers / 32; ++w)
        tot.merge(s_warp[w], reduce_op);
      const bool failed = *abort_flag != 0;
      if (direct) {
        OutT val = tot.value();
        if constexpr (std::is_same<StoreT, OutT>::value) {
          if (inplace) val = reduce_op(out[row], val);
        }
        StoreT res = final_op(val);
        if constexpr (std::is_floating_point<StoreT>::value) {
          if (failed) res = StoreT(NAN);
        }
        out[row] = res;
      } else {
        auto carry = tot.carry();
        if constexpr (std::is_floating_point<decltype(carry)>::value) {
          if (failed) carry = decltype(carry)(NAN);
        }
        partial[row * n_seg + seg] = carry;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kTmaConsumers) : "memory");  // s_warp is reused by the next row
  }
}

}  // namespace detail
}  // namespace raft_b200
