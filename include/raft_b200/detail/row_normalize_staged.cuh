// Row normalisation staged through shared memory, read AND write side by bulk asynchronous copies:
// for contiguous matrices whose rows do not start on 16-byte boundaries (a direct kernel is left
// with 4-byte loads and stores there) or whose length fits the lane groups of the direct kernels
// badly. Blocks of rows are 16-byte aligned even when single rows are not (see
// row_reduce_staged.cuh), and that holds for the output just as for the input.
//
// One producer thread per CTA owns both directions. It fills a ring of shared-memory stages with
// cp.async.bulk (global -> shared, completion on an mbarrier); 256 consumers compute the norm of
// every row of a tile from shared memory (G lanes per row), divide the row IN PLACE in shared
// memory, and report the tile done; the producer then writes the whole tile back with one
// cp.async.bulk (shared -> global), waits until the copy has read the stage, and loads the next
// tile into it. HBM sees every element once in each direction, in 16-byte-aligned bursts.
//
// Rows whose norm is <= eps must stay untouched in `out`, so a tile that contains one cannot be
// written back as a block: its consumers mark such rows in a bitmap, raise the stage's skip flag,
// and store the other rows themselves with plain stores; the producer skips the block copy.
//
// Every mbarrier wait is bounded (see col_reduce_tma.cuh). A CTA whose wait runs out raises its
// abort flag, every thread leaves at the next tile boundary, the producer waits (bounded) for its
// copies in flight, and the rows of the CTA that were not finished are filled with NaN.
#pragma once

#include "col_reduce_tma.cuh"
#include "row_reduce.cuh"

namespace raft_b200 {
namespace detail {

B2R_DI void bulk_store(void* gmem_dst, const void* smem_src, unsigned bytes)
{
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// until the bulk stores of this thread have READ their shared-memory source (it may be overwritten)
B2R_DI void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// until they are complete
B2R_DI void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// writes of this thread through the generic proxy become visible to the asynchronous proxy
B2R_DI void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// barrier among the consumer warps only (the producer warp does not take part)
B2R_DI void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kTmaConsumers) : "memory"); }
// the same barrier, returning whether ANY consumer passed a true predicate: a decision every consumer
// takes alike, whatever another thread does to the underlying flag in the meantime
B2R_DI bool consumer_sync_any(bool pred)
{
  unsigned r;
  asm volatile(
    "{\n\t.reg .pred p, q;\n\t"
    "setp.ne.u32 p, %1, 0;\n\t"
    "bar.red.or.pred q, 1, %2, p;\n\t"
    "selp.u32 %0, 1, 0, q;\n\t}"
    : "=r"(r)
    : "r"(unsigned(pred)), "n"(kTmaConsumers)
    : "memory");
  return r != 0;
}

template <typename T, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp, int VEC>
__global__ void __launch_bounds__(kTmaThreads, 2) row_normalize_staged_kernel(T* out,
                                                                             const T* in,
                                                                             int64_t n_rows,
                                                                             int row_len,
                                                                             T init,
                                                                             T eps,
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
  using State = typename state_for<T, ReduceOp>::type;
  using Vec   = VecOf<T, VEC>;
  extern __shared__ __align__(128) unsigned char smem_tma[];
  __shared__ __align__(8) uint64_t s_full[kTmaMaxStages];  // a tile has landed
  __shared__ __align__(8) uint64_t s_done[kTmaMaxStages];  // the consumers are through with it
  __shared__ int s_skip[kTmaMaxStages];                    // the tile holds rows that must not be written
  __shared__ int s_abort;

  const size_t row_bytes    = size_t(row_len) * sizeof(T);
  const size_t stage_stride = (size_t(tile_rows) * row_bytes + 127) / 128 * 128;
  const int flag_words      = (tile_rows + 31) / 32;
  unsigned* flags_base      = reinterpret_cast<unsigned*>(smem_tma + size_t(STAGES) * stage_stride);
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
      mbar_init(&s_done[s], kTmaConsumers / 32);
      s_skip[s] = 0;
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int w = tid; w < STAGES * flag_words; w += kTmaThreads)
    flags_base[w] = 0u;
  __syncthreads();
  grid_dep_sync();  // the set-up above touches shared memory only
  volatile int* abort_flag = &s_abort;
  volatile int* skip_flag  = s_skip;

  if (producer) {
    if (tid == kTmaConsumers) {
      // the host makes n_rows, tile_rows and rows_per_cta multiples of the rows between two 16-byte
      // boundaries, so every copy starts on a boundary and has a legal size
      auto load = [&](int t) {
        if (t == ctl.skip_tile && blockIdx.x == 0) return;  // test hook: this tile is never requested
        const int s        = t % STAGES;
        const int64_t row0 = r_beg + int64_t(t) * tile_rows;
        const int64_t nr   = (r_end - row0) < tile_rows ? (r_end - row0) : tile_rows;
        const unsigned nb  = unsigned(size_t(nr) * row_bytes);
        mbar_expect_tx(&s_full[s], nb);
        bulk_load(smem_tma + s * stage_stride, reinterpret_cast<const unsigned char*>(in) + size_t(row0) * row_bytes, nb,
                  &s_full[s]);
      };
      int loaded = 0;
      for (; loaded < STAGES && loaded < n_tiles; ++loaded)
        load(loaded);
      int t = 0;
      for (; t < n_tiles; ++t) {
        const int s          = t % STAGES;
        const unsigned phase = (t / STAGES) & 1u;
        if (!mbar_wait_bounded(&s_done[s], phase, abort_flag, ctl.limit_ns)) break;
        if (skip_flag[s] == 0) {
          const int64_t row0 = r_beg + int64_t(t) * tile_rows;
          const int64_t nr   = (r_end - row0) < tile_rows ? (r_end - row0) : tile_rows;
          bulk_store(reinterpret_cast<unsigned char*>(out) + size_t(row0) * row_bytes, smem_tma + s * stage_stride,
                     unsigned(size_t(nr) * row_bytes));
          bulk_store_wait_read();  // the stage may be overwritten from here on
        } else {
          skip_flag[s] = 0;  // the consumers stored the tile's rows themselves
        }
        if (t + STAGES < n_tiles) {
          load(t + STAGES);
          loaded = t + STAGES + 1;
        }
      }
      if (t < n_tiles) {
        // gave up: the loads already issued must land before the CTA may exit
        for (int u = t; u < loaded; ++u) {
          if (u == ctl.skip_tile && blockIdx.x == 0) continue;
          mbar_drain_bounded(&s_full[u % STAGES], (u / STAGES) & 1u, ctl.limit_ns);
        }
        ring_report_timeout(ctl);
      }
      bulk_store_wait_all();
    }
    return;
  }

  const int lane = tid & 31;
  const int lg   = 31 - __clz(G);
  const int lig  = tid & (G - 1);        // lane within the group of a row
  const int slot = tid >> lg;            // row slot of this thread within a pass
  const int rpp  = kTmaConsumers >> lg;  // rows per pass of the CTA
  const int nvec = row_len / VEC;        // VEC divides row_len (VEC = 1 for rows off 16-byte boundaries)
  // every row slot starts `rot` vectors further into its row and wraps (bank conflicts, see row_reduce_staged.cuh)
  const int shift  = rot == 0 ? 0 : int((unsigned(slot) * unsigned(rot)) % unsigned(nvec));
  const int n_mine = (nvec >> lg) + (lig < (nvec & (G - 1)) ? 1 : 0);  // vectors of a row this lane takes
  const int n_full = nvec >> lg;                                        // ... that every lane of the group takes

  int t = 0;
  RingPos rp{0, 0u};
  for (; t < n_tiles; ++t) {
    const int s          = rp.s;
    const unsigned phase = rp.phase;
    rp.advance(1, STAGES);
    // a wait that ran out (here, or in the producer) has raised the flag; each consumer reads it BEFORE the
    // barrier and the barrier ORs what they saw, so all of them stay or all of them leave
    mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns);
    if (consumer_sync_any(*abort_flag != 0)) break;
    const int64_t tile_row0 = r_beg + int64_t(t) * tile_rows;
    const int nr            = int((r_end - tile_row0) < tile_rows ? (r_end - tile_row0) : tile_rows);
    Vec* tile               = reinterpret_cast<Vec*>(smem_tma + s * stage_stride);
    unsigned* flags         = flags_base + s * flag_words;
    // whole warps walk the passes together (the shuffles below need all lanes)
    for (int lr0 = 0; lr0 < nr; lr0 += rpp) {
      const int lr  = lr0 + slot;
      const bool ok = lr < nr;
      Vec* row      = tile + size_t(ok ? lr : nr - 1) * nvec;
      State st;
      st.init(init);
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
              st.push(T(main_op(v[k].e[e], IdxT((c + k * G) * VEC + e))), reduce_op);
          }
        }
        for (; j < n_mine; ++j, c += G) {
          const Vec v = row[c];
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            st.push(T(main_op(v.e[e], IdxT(c * VEC + e))), reduce_op);
        }
      } else {
        for (int j = 0; j < n_mine; ++j) {
          int c       = (j << lg) + lig + shift;
          c           = c >= nvec ? c - nvec : c;
          const Vec v = row[c];
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            st.push(T(main_op(v.e[e], IdxT(c * VEC + e))), reduce_op);
        }
      }
      for (int off = G >> 1; off > 0; off >>= 1) {
        State got = shfl_xor_any(st, off);
        st.merge(got, reduce_op);
      }
      // every lane of the row divides by the SAME value: the one of the group's first lane
      const T norm = shfl_idx_any(T(final_op(st.value())), lane & ~(G - 1));
      if (ok) {
        if (!(norm <= eps)) {
          for (int j = 0; j < n_mine; ++j) {
            int c = (j << lg) + lig + shift;
            c     = c >= nvec ? c - nvec : c;
            Vec v = row[c];
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              v.e[e] = v.e[e] / norm;
            row[c] = v;
          }
        } else if (lig == 0) {
          atomicOr(&flags[lr >> 5], 1u << (lr & 31));
          skip_flag[s] = 1;
        }
      }
    }
    fence_proxy_async();  // the divided rows, for the producer's block copy
    consumer_sync();
    if (skip_flag[s] != 0) {
      // some row of this tile must stay untouched in `out`: no block copy, every other row by plain stores
      for (int lr0 = 0; lr0 < nr; lr0 += rpp) {
        const int lr = lr0 + slot;
        if (lr < nr && ((flags[lr >> 5] >> (lr & 31)) & 1u) == 0u) {
          const T* src = reinterpret_cast<const T*>(tile + size_t(lr) * nvec);
          T* dst       = out + (tile_row0 + lr) * int64_t(row_len);
          for (int c = lig; c < row_len; c += G)
            dst[c] = src[c];
        }
      }
      consumer_sync();  // every thread has read the bitmap
      for (int w = tid; w < flag_words; w += kTmaConsumers)
        flags[w] = 0u;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s_done[s]);
  }
  if (t < n_tiles) {
    // a bounded wait ran out: make it visible - the rows this CTA did not finish become NaN
    if constexpr (std::is_floating_point<T>::value) {
      const int64_t e_beg = (r_beg + int64_t(t) * tile_rows) * row_len;
      const int64_t e_end = r_end * int64_t(row_len);
      for (int64_t i = e_beg + tid; i < e_end; i += kTmaConsumers)
        out[i] = T(NAN);
    }
  }
}

}  // namespace detail
}  // namespace raft_b200
