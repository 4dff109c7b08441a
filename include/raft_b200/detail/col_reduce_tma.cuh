// Column reduction of a NARROW contiguous row-major matrix with TMA-staged shared-memory tiles.
//
// When a row is at most a few KB and rows are contiguous (ld == n_cols), T consecutive rows are
// one contiguous block of memory. A producer warp streams such blocks into a ring of shared-memory
// stages with bulk asynchronous copies (cp.async.bulk, completion on an mbarrier), so the bytes in
// flight per SM are set by the ring (stages x tile bytes) instead of by registers, and the
// consumer warps spend no instructions on global addresses: they read the tile with conflict-free
// 16-byte shared-memory loads and keep the same per-column accumulators as col_partial_kernel.
// Output protocol (partial rows, finalize kernel) is that of col_reduce.cuh.
//
// Every wait on an mbarrier is bounded by TIME (RingCtl::limit_ns of the global timer, a second by
// default): a thread whose wait runs out raises the CTA's abort flag; all threads then leave their
// loops, the producer drains the copies it still has in flight (bounded as well), marks
// cta_status[cta] = 1 and the call's status word, and the CTA finishes normally. The finalize kernel
// turns any marked CTA into NaN outputs and the host can read the status word afterwards
// (b2r_last_kernel_status), so a give-up is loud, not a silently wrong sum.
#pragma once

#include "col_reduce.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kTmaConsumers = 256;              // consumer threads (8 warps)
constexpr int kTmaThreads   = kTmaConsumers + 32;  // + one producer warp
constexpr int kTmaMaxStages   = 8;

// What every ring kernel is told about its waits. `status` is a device word shared by the calls of one
// device (null: none): a CTA that gives up stores 1 there. `skip_tile` is a test hook: the producer of
// CTA 0 does not issue the copy of that tile (-1: none), so the consumers' wait for it runs out with no
// copy of that tile in flight - the one way to see the give-up path work without a fault.
struct RingCtl {
  int* status;
  unsigned long long limit_ns;
  int skip_tile;
};
constexpr unsigned long long kDefaultWaitLimitNs = 1000ull * 1000ull * 1000ull;
B2R_HDI RingCtl default_ring_ctl()
{
  RingCtl c;
  c.status    = nullptr;
  c.limit_ns  = kDefaultWaitLimitNs;
  c.skip_tile = -1;
  return c;
}

B2R_DI unsigned long long ring_timer_ns()
{
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

B2R_DI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

B2R_DI void mbar_init(uint64_t* bar, unsigned count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
B2R_DI void mbar_expect_tx(uint64_t* bar, unsigned bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
B2R_DI void mbar_arrive(uint64_t* bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
B2R_DI bool mbar_try_wait(uint64_t* bar, unsigned parity)
{
  unsigned ok;
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(ok)
    : "r"(smem_u32(bar)), "r"(parity)
    : "memory");
  return ok != 0;
}
// A consumer's place in a ring of `stages` stages - stage index and parity of the round - advanced without a
// division: tile t sits in stage t % stages in round t / stages, and a division by a run-time stage count costs
// a warp some thirty instructions per tile (a hundred in 64 bits), as much as the tile's own work where tiles are small.
struct RingPos {
  int s;
  unsigned phase;
  B2R_DI void advance(int by, int stages)  // by <= stages
  {
    s += by;
    if (s >= stages) {
      s -= stages;
      phase ^= 1u;
    }
  }
};
// Bounded wait. Returns false (and raises the abort flag) when `limit_ns` has passed or another
// thread has already aborted. The clock is only read once a first batch of polls has failed.
B2R_DI bool mbar_wait_bounded(uint64_t* bar, unsigned parity, volatile int* abort_flag, unsigned long long limit_ns)
{
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = ring_timer_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (ring_timer_ns() - t0 > limit_ns) break;
  }
  *abort_flag = 1;
  return false;
}
// The producer's last duty after a give-up: the copies it has issued must land before the CTA may exit.
// Bounded as well (twice the limit); returns false if even that ran out.
B2R_DI bool mbar_drain_bounded(uint64_t* bar, unsigned parity, unsigned long long limit_ns)
{
  const unsigned long long t0 = ring_timer_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (ring_timer_ns() - t0 > 2 * limit_ns) return false;
  }
}
// After its last copy the producer stays until the consumers have released every tile it issued, or
// somebody has given up: it is the thread that lets copies in flight land and reports, so it leaves last.
B2R_DI void producer_wait_released(uint64_t* s_empty, long long issued, int STAGES, volatile int* abort_flag,
                                   unsigned long long limit_ns)
{
  const long long first = issued > STAGES ? issued - STAGES : 0;
  for (long long t = first; t < issued; ++t)
    if (!mbar_wait_bounded(&s_empty[t % STAGES], unsigned(t / STAGES) & 1u, abort_flag, limit_ns)) return;
}
B2R_DI void ring_report_timeout(const RingCtl& ctl)
{
  if (ctl.status != nullptr) atomicExch(ctl.status, 1);
}
B2R_DI void bulk_load(void* smem_dst, const void* gmem_src, unsigned bytes, uint64_t* bar)
{
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
    "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
    : "memory");
}

template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          int VEC>
__global__ void __launch_bounds__(kTmaThreads, 1)
  col_partial_tma_kernel(OutT* __restrict__ out,
                         typename state_for<OutT, ReduceOp>::type::carry_t* __restrict__ partial,
                         const InT* __restrict__ data,
                         int64_t n_rows,
                         int n_cols,
                         OutT init,
                         bool inplace,
                         MainOp main_op,
                         ReduceOp reduce_op,
                         FinalOp final_op,
                         int TX,
                         int tile_rows,
                         int64_t rows_per_cta,
                         int STAGES,
                         int* __restrict__ cta_status,
                         RingCtl ctl)
{
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  extern __shared__ __align__(128) unsigned char smem_tma[];
  const size_t row_bytes  = size_t(n_cols) * sizeof(InT);
  const size_t tile_bytes = size_t(tile_rows) * row_bytes;  // multiple of 16
  unsigned char* tiles    = smem_tma;                                              // [STAGES][tile_bytes]
  State* s_part           = reinterpret_cast<State*>(smem_tma + STAGES * ((tile_bytes + 127) / 128 * 128));
  __shared__ __align__(8) uint64_t s_full[kTmaMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kTmaMaxStages];
  __shared__ int s_abort;

  const int tid       = threadIdx.x;
  const bool producer = tid >= kTmaConsumers;
  const int TY        = kTmaConsumers / TX;
  const int tx        = tid & (TX - 1);
  const int ty        = tid / TX;  // meaningful for consumers
  const int64_t r_beg = int64_t(blockIdx.x) * rows_per_cta;
  int64_t r_end       = r_beg + rows_per_cta;
  r_end               = r_end < n_rows ? r_end : n_rows;
  const int64_t rows  = r_end > r_beg ? r_end - r_beg : 0;
  const int n_tiles   = int((rows + tile_rows - 1) / tile_rows);
  const bool direct   = gridDim.x == 1;
  const size_t stage_stride = (tile_bytes + 127) / 128 * 128;

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
  // 1 if this CTA gave up on a wait (set by the same thread)
  if (tid == kTmaConsumers && cta_status != nullptr) cta_status[blockIdx.x] = 0;
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
        if (t == ctl.skip_tile && blockIdx.x == 0) continue;  // test hook: this tile is never requested
        const int64_t row0 = r_beg + int64_t(t) * tile_rows;
        const int64_t nr   = (r_end - row0) < tile_rows ? (r_end - row0) : tile_rows;
        const unsigned nb  = unsigned(size_t(nr) * row_bytes);
        mbar_expect_tx(&s_full[s], nb);
        bulk_load(tiles + s * stage_stride, reinterpret_cast<const unsigned char*>(data) + size_t(row0) * row_bytes, nb,
                  &s_full[s]);
        issued = t + 1;
      }
      producer_wait_released(s_empty, issued, STAGES, abort_flag, ctl.limit_ns);
      if (*abort_flag != 0) {
        // drain: copies already issued must land before the CTA may exit
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int t = first; t < issued; ++t) {
          if (t == ctl.skip_tile && blockIdx.x == 0) continue;
          mbar_drain_bounded(&s_full[t % STAGES], (t / STAGES) & 1u, ctl.limit_ns);
        }
        if (cta_status != nullptr) cta_status[blockIdx.x] = 1;
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
      const int64_t row0 = r_beg + int64_t(t) * tile_rows;
      const int nr       = int((r_end - row0) < tile_rows ? (r_end - row0) : tile_rows);
      if (tx * VEC < n_cols) {
        const unsigned char* tile = tiles + s * stage_stride + size_t(tx) * VEC * sizeof(InT);
        int r = ty;
        for (; r + 3 * TY < nr; r += 4 * TY) {
          VecOf<InT, VEC> v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            v[u] = *reinterpret_cast<const VecOf<InT, VEC>*>(tile + size_t(r + u * TY) * row_bytes);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              st[e].push(OutT(main_op(v[u].e[e], IdxT(row0 + r + u * TY))), reduce_op);
          }
        }
        for (; r < nr; r += TY) {
          const VecOf<InT, VEC> v = *reinterpret_cast<const VecOf<InT, VEC>*>(tile + size_t(r) * row_bytes);
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
  const int W = TX * VEC;
  if (!producer) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      s_part[ty * W + tx * VEC + e] = st[e];
  }
  __syncthreads();
  for (int j = tid; j < W; j += kTmaThreads) {
    if (j < n_cols) {
      State r = s_part[j];
      for (int y = 1; y < TY; ++y)
        r.merge(s_part[y * W + j], reduce_op);
      if (direct) {
        if constexpr (isSum) { r.push(init, reduce_op); }
        OutT v = r.value();
        if (inplace) v = reduce_op(out[j], v);
        out[j] = final_op(v);
      } else {
        partial[int64_t(blockIdx.x) * n_cols + j] = r.carry();
      }
    }
  }
}

}  // namespace detail
}  // namespace raft_b200
