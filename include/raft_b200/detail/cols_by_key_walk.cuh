// Keyed column sums, "walk" form of "sort the columns, then stream tiles" (cols_by_key_sorted.cuh):
//     out[r][keys[c]] += data[r][c]          data row-major [nrows x ncols], rows on 16-byte boundaries
//
// The tile kernel of cols_by_key_sorted.cuh gives a lane a (row, key) SEGMENT of the tile; segments of one
// chunk differ in length, the lanes of a warp wait for the longest, and every segment pays its own set-up: with
// 128 keys that kernel executes 24 lane-instructions per matrix element and is bound by instruction issue at
// 4.2 TB/s. Here the whole WARP walks the sorted columns of the keys it owns (of (key, slice) items when there
// are fewer keys than warps) one segment after the other: lane (r, q) takes row r of the tile and every Q-th
// sorted column of the segment, Q = 32 / RT, so all lanes run the same loop on the same segment - no
// divergence beyond a last, partly filled step - summing in fp64 registers that live for a whole row tile; only at its end do the Q
// partial sums of a row meet by shuffles and go into the table cell (item, row) in shared memory. The sorted column offsets are read as broadcasts.
// Tiles are RT rows x CH columns with FEW, LONG row pieces (16 x 1024 by default): what bounds a ring of bulk
// copies is their number, not their bytes - 32 pieces of 2 KB per tile ran at the same tiles per second as 32
// pieces of 1 KB (5.4 against 2.9 TB/s with 8 keys).
// Measured, fp32 2000 x 200000, TB/s (this form / lane per segment): 8 keys 6.7 / 5.5, 32 keys 6.4 / 4.8, 64 keys
// 5.3 / 4.5, 128 keys 3.4 / 4.15, 256 keys 2.2 / 3.75 - with many keys a warp owns many short segments per tile
// and pays a chain of shared-memory latencies for each, so the host takes this form up to 32 keys (64 for
// fp64, which the table form of cols_by_key_table.cuh does not take). (With fp32 partial sums it is 1-10 %
// faster, but then a repeated call can differ in the last bit: see the walk below.)
// Nothing else changes: the columns are counting-sorted by key once per call, chunk by chunk (cbk_sort_kernel),
// a producer WARP streams the RT row pieces of a tile (one bulk copy per lane), the chunk's sorted offsets and
// its segment starts into a ring of shared-memory stages, one CTA per SM walks a range of row tiles x a range
// of chunks, and per-CTA tables are merged in a fixed order when the columns are split (cbk_merge_kernel).
// No floating-point atomics. Every mbarrier wait is bounded (col_reduce_tma.cuh); a CTA that gives up writes
// NaN and sets the status word.
#pragma once

#include "cols_by_key_sorted.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kCbk32Warps     = 16;                      // consumer warps
constexpr int kCbk32Consumers = kCbk32Warps * 32;
constexpr int kCbk32Threads   = kCbk32Consumers + 32;    // + the producer warp
constexpr int kCbk32MaxStages = 6;

// one element of a staged tile, in its own type (fp32 segments are summed in fp32, fp64 ones in fp64)
B2R_DI float lds_val(uint32_t addr, float)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
B2R_DI double lds_val(uint32_t addr, double)
{
  double v;
  asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(addr));
  return v;
}

struct Cbk32Plan {
  bool ok;
  int RT;             // rows per tile: 8, 16 or 32
  int acc_pitch;      // doubles per item in the table (RT + 1: the flush reads columns of it)
  int CH;
  int S;              // slices per key (a power of two; > 1 only with fewer keys than consumer warps)
  int n_items;        // nkeys x S
  int items_per_warp;
  int n_chunks;
  int offs_stride;
  int stages;
  int y_split;
  int chunks_per_cta;
  int64_t n_row_tiles;
  int64_t row_tiles_per_cta;
  size_t acc_bytes, off_tile, off_perm, off_offs, stage_bytes, smem;
  size_t off_perm_g, off_offs_g, off_part_g, total;  // scratch in global memory
};

template <typename T>
inline Cbk32Plan plan_cols_by_key_rows32(const T* data, int64_t nrows, int64_t ncols, int64_t nkeys, int ch_knob,
                                         int rt_knob)
{
  Cbk32Plan p = {};
  const int RT = (rt_knob == 8 || rt_knob == 16 || rt_knob == 32) ? rt_knob : 16;
  p.RT         = RT;
  p.acc_pitch  = RT + 1;
  constexpr int V16 = vec16<T>::value;
  if (!(V16 > 1 && ncols % V16 == 0 && aligned16(data)) || nkeys < 1 || nkeys > 16 * kCbk32Warps || ncols < 1 || nrows < 1) return p;
  int S = 1;
  while (nkeys * S < kCbk32Warps)
    S <<= 1;
  p.S              = S;
  p.n_items        = int(nkeys) * S;
  p.items_per_warp = ceil_div<int>(p.n_items, kCbk32Warps);
  p.acc_bytes      = align_up(size_t(p.n_items) * size_t(p.acc_pitch) * sizeof(double), 128);
  p.offs_stride    = int(ceil_div<int64_t>(nkeys + 1, 8) * 8);
  const size_t budget = size_t(218) << 10;
  // the longest chunks that leave room for at least two stages (longer segments: less set-up per element;
  // longer row pieces: fewer copies per byte), a 64 KB tile at most unless the knob says otherwise
  int CH = ch_knob > 0 ? ch_knob : int(65536 / (RT * sizeof(T)));
  if (CH > 4096) CH = 4096;
  for (;; CH >>= 1) {
    if (CH < 64) return p;
    size_t o   = 0;
    p.off_tile = o;
    o += align_up(size_t(RT) * (CH + kCbkPad) * sizeof(T), 128);
    p.off_perm = o;
    o += align_up(size_t(CH) * sizeof(unsigned short), 128);
    p.off_offs = o;
    o += align_up(size_t(p.offs_stride) * sizeof(unsigned short), 128);
    p.stage_bytes = o;
    if (p.acc_bytes + 2 * p.stage_bytes <= budget) break;
  }
  while (CH > 64 && CH / 2 >= ncols)
    CH >>= 1;
  {
    size_t o   = 0;
    p.off_tile = o;
    o += align_up(size_t(RT) * (CH + kCbkPad) * sizeof(T), 128);
    p.off_perm = o;
    o += align_up(size_t(CH) * sizeof(unsigned short), 128);
    p.off_offs = o;
    o += align_up(size_t(p.offs_stride) * sizeof(unsigned short), 128);
    p.stage_bytes = o;
  }
  p.CH     = CH;
  int st   = int((budget - p.acc_bytes) / p.stage_bytes);
  p.stages = st > kCbk32MaxStages ? kCbk32MaxStages : st;
  if (p.stages < 2) return p;
  p.smem        = p.acc_bytes + size_t(p.stages) * p.stage_bytes;
  p.n_chunks    = int(ceil_div<int64_t>(ncols, CH));
  p.n_row_tiles = ceil_div<int64_t>(nrows, RT);
  if (p.n_row_tiles > int64_t(0x7fffffff)) return p;
  // the split of the columns that needs the fewest waves of one CTA per SM; splitting costs a merge
  const int slots   = sm_count();
  int64_t best_cost = 0;
  for (int y = 1; y <= 2 * slots && y <= p.n_chunks; ++y) {
    const int cpc       = int(ceil_div<int64_t>(p.n_chunks, y));
    const int ys        = int(ceil_div<int64_t>(p.n_chunks, cpc));
    const int64_t per_x = p.n_row_tiles * ys > slots ? ceil_div<int64_t>(p.n_row_tiles * ys, slots) : 1;
    const int64_t rtpc  = per_x < p.n_row_tiles ? per_x : p.n_row_tiles;
    const int64_t gx    = ceil_div<int64_t>(p.n_row_tiles, rtpc);
    const int64_t waves = ceil_div<int64_t>(gx * ys, slots);
    const int64_t cost  = waves * rtpc * cpc * (ys > 1 ? 51 : 50) + (ys > 1 ? 50 : 0);
    if (best_cost == 0 || cost < best_cost) {
      best_cost           = cost;
      p.y_split           = ys;
      p.chunks_per_cta    = cpc;
      p.row_tiles_per_cta = rtpc;
    }
  }
  size_t o     = 0;
  p.off_perm_g = o;
  o += align_up(size_t(p.n_chunks) * size_t(CH) * sizeof(unsigned short), 256);
  p.off_offs_g = o;
  o += align_up(size_t(p.n_chunks) * size_t(p.offs_stride) * sizeof(unsigned short), 256);
  p.off_part_g = o;
  if (p.y_split > 1) o += align_up(size_t(p.y_split) * size_t(nrows) * size_t(nkeys) * sizeof(double), 256);
  p.total = o;
  p.ok    = true;
  return p;
}

// IPW: items a warp owns at most (compile-time, so that their running sums are registers)
template <typename T, int IPW>
__global__ void __launch_bounds__(kCbk32Threads, 1) cbk_rows32_kernel(T* __restrict__ out,
                                                                     double* __restrict__ partial,
                                                                     const T* __restrict__ data,
                                                                     const unsigned short* __restrict__ perm16,
                                                                     const unsigned short* __restrict__ offs16,
                                                                     int64_t nrows,
                                                                     int64_t ncols,
                                                                     int nkeys,
                                                                     bool reset,
                                                                     Cbk32Plan P,
                                                                     RingCtl ctl)
{
  extern __shared__ __align__(128) unsigned char smem_tma[];
  double* acc               = reinterpret_cast<double*>(smem_tma);  // [n_items][RT + 1]
  unsigned char* stages     = smem_tma + P.acc_bytes;
  const uint32_t stages_u32 = smem_u32(stages);
  __shared__ __align__(8) uint64_t s_full[kCbk32MaxStages];
  __shared__ __align__(8) uint64_t s_empty[kCbk32MaxStages];
  __shared__ int s_abort;

  const int tid       = threadIdx.x;
  const bool producer = tid >= kCbk32Consumers;
  const int CH        = P.CH;
  const int RT        = P.RT;
  const int STAGES    = P.stages;
  const int64_t rt0   = int64_t(blockIdx.x) * P.row_tiles_per_cta;
  int64_t rt1         = rt0 + P.row_tiles_per_cta;
  rt1                 = rt1 < P.n_row_tiles ? rt1 : P.n_row_tiles;
  const int ch0       = blockIdx.y * P.chunks_per_cta;
  int ch1             = ch0 + P.chunks_per_cta;
  ch1                 = ch1 < P.n_chunks ? ch1 : P.n_chunks;
  const int n_ch      = ch1 > ch0 ? ch1 - ch0 : 0;
  const unsigned pitch = unsigned(CH + kCbkPad) * unsigned(sizeof(T));  // bytes between the rows of a staged tile

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], kCbk32Warps);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dep_sync();  // the set-up above touches shared memory only
  volatile int* abort_flag = &s_abort;

  if (producer) {
    const int plane  = tid - kCbk32Consumers;
    long long issued = 0;
    bool alive       = true;
    for (int64_t rti = rt0; rti < rt1 && alive; ++rti) {
      const int64_t r0 = rti * RT;
      const int rt     = int(nrows - r0 < RT ? nrows - r0 : RT);
      for (int c = 0; c < n_ch; ++c) {
        const int s          = int(issued % STAGES);
        const unsigned phase = unsigned(issued / STAGES) & 1u;
        int ok               = 1;
        if (plane == 0) ok = mbar_wait_bounded(&s_empty[s], phase ^ 1u, abort_flag, ctl.limit_ns) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          alive = false;
          break;
        }
        if (issued == ctl.skip_tile && blockIdx.x == 0 && blockIdx.y == 0) {  // test hook: never requested
          ++issued;
          continue;
        }
        const int ch      = ch0 + c;
        const int64_t c0  = int64_t(ch) * CH;
        const int cw      = int(ncols - c0 < CH ? ncols - c0 : CH);
        unsigned char* st = stages + size_t(s) * P.stage_bytes;
        const unsigned rb = unsigned(cw) * unsigned(sizeof(T));  // a multiple of 16
        const unsigned pb = unsigned(CH) * unsigned(sizeof(unsigned short));
        const unsigned ob = unsigned(P.offs_stride) * unsigned(sizeof(unsigned short));
        if (plane == 0) mbar_expect_tx(&s_full[s], rb * unsigned(rt) + pb + ob);
        __syncwarp();  // the bytes are announced before any copy can complete
        if (plane < rt) bulk_load(st + P.off_tile + size_t(plane) * pitch, data + (r0 + plane) * ncols + c0, rb, &s_full[s]);
        if (plane == (rt & 31)) bulk_load(st + P.off_perm, perm16 + size_t(ch) * CH, pb, &s_full[s]);
        if (plane == ((rt + 1) & 31)) bulk_load(st + P.off_offs, offs16 + size_t(ch) * P.offs_stride, ob, &s_full[s]);
        ++issued;
      }
    }
    if (plane == 0) {
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

  const int lane   = tid & 31;
  const int warp   = tid >> 5;
  const int ls     = 31 - __clz(P.S);
  const int it0    = warp * P.items_per_warp;
  int it1          = it0 + P.items_per_warp;
  it1              = it1 < P.n_items ? it1 : P.n_items;
  const int lrt    = 31 - __clz(RT);
  const int my_r   = lane & (RT - 1);          // row of the tile
  const int my_q   = lane >> lrt;              // which of every Q sorted columns
  const unsigned step = unsigned(32 >> lrt) * 2u;  // bytes between this lane's consecutive offsets
  // This lane's share (row my_r, sorted columns my_q, my_q + Q, ...) of the sum of every item of the warp, for
  // the current row tile: registers. Nothing is exchanged or stored per segment; the Q shares of a row meet by
  // shuffles once per row tile.
  double run[IPW];
#pragma unroll
  for (int ii = 0; ii < IPW; ++ii)
    run[ii] = 0.0;

  long long seq = 0;
  RingPos rp{0, 0u};
  bool dead     = false;
  for (int64_t rti = rt0; rti < rt1; ++rti) {
    const int64_t r0 = rti * RT;
    const int rt     = int(nrows - r0 < RT ? nrows - r0 : RT);
    for (int c = 0; c < n_ch; ++c, ++seq) {
      if (dead) continue;
      const int s          = rp.s;
      const unsigned phase = rp.phase;
      rp.advance(1, STAGES);
      if (!mbar_wait_bounded(&s_full[s], phase, abort_flag, ctl.limit_ns)) {
        dead = true;
        continue;
      }
      const uint32_t st   = stages_u32 + uint32_t(s) * uint32_t(P.stage_bytes);
      const uint32_t perm = st + uint32_t(P.off_perm);                               // u16 [CH], sorted by key
      const uint32_t offs = st + uint32_t(P.off_offs);                               // u16 [nkeys + 1]
      const uint32_t row  = st + uint32_t(P.off_tile) + uint32_t(my_r) * pitch;      // this lane's row piece
      // the segment bounds of all items first (independent loads), then the walks
      unsigned j0s[IPW], j1s[IPW];
#pragma unroll
      for (int ii = 0; ii < IPW; ++ii) {
        const int it = it0 + ii;
        j0s[ii] = j1s[ii] = 0u;
        if (it < it1) {
          const int k         = it >> ls;
          const int sl        = it & (P.S - 1);
          const unsigned seg0 = lds_u16(offs + 2u * unsigned(k));
          const unsigned len  = lds_u16(offs + 2u * unsigned(k) + 2u) - seg0;
          j0s[ii]             = seg0 + ((len * unsigned(sl)) >> ls);
          j1s[ii]             = seg0 + ((len * unsigned(sl + 1)) >> ls);
        }
      }
      // (Masking the ragged ends of the segments instead - fixed steps of four columns per lane, two items
      // interleaved - was measured: 2-6 % slower up to 64 keys, 5-15 % faster from 128 keys on, where the
      // lane-per-segment kernel is faster than either.)
#pragma unroll
      for (int ii = 0; ii < IPW; ++ii) {
        // fp64 partial sums also for fp32 data: the order of a key's columns inside a chunk comes from integer
        // atomics in the sort and may differ between runs; sums carried in fp64 hide that below the rounding
        // of the fp32 result, so a repeated call gives the same bits
        double f0 = 0.0, f1 = 0.0, f2 = 0.0, f3 = 0.0;
        uint32_t pa       = perm + 2u * (j0s[ii] + unsigned(my_q));
        const uint32_t pe = perm + 2u * j1s[ii];
        for (; pa + 3u * step < pe; pa += 4u * step) {
          const unsigned a = lds_u16(pa), b = lds_u16(pa + step), c2 = lds_u16(pa + 2u * step), d = lds_u16(pa + 3u * step);
          f0 += double(lds_val(row + a * unsigned(sizeof(T)), T()));
          f1 += double(lds_val(row + b * unsigned(sizeof(T)), T()));
          f2 += double(lds_val(row + c2 * unsigned(sizeof(T)), T()));
          f3 += double(lds_val(row + d * unsigned(sizeof(T)), T()));
        }
        for (; pa < pe; pa += step)
          f0 += double(lds_val(row + lds_u16(pa) * unsigned(sizeof(T)), T()));
        run[ii] += (f0 + f1) + (f2 + f3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
    }
    // end of the row tile: the Q shares of every (item, row) meet, the first lane of a row puts the sum into
    // the table in shared memory
#pragma unroll
    for (int ii = 0; ii < IPW; ++ii) {
      double v = run[ii];
      for (int off = RT; off < 32; off <<= 1)
        v += __shfl_xor_sync(0xffffffffu, v, off);
      if (my_q == 0 && it0 + ii < it1) acc[(it0 + ii) * P.acc_pitch + my_r] = v;
      run[ii] = 0.0;
    }
    // ... which goes out as [row][key]
    asm volatile("bar.sync 1, %0;" ::"n"(kCbk32Consumers) : "memory");
    const bool failed = *abort_flag != 0;
    const double nan  = __longlong_as_double(0x7ff8000000000000ll);
    for (int i = tid; i < rt * nkeys; i += kCbk32Consumers) {
      const int r = i / nkeys;
      const int k = i - r * nkeys;
      double v    = 0.0;
      for (int sl = 0; sl < P.S; ++sl)
        v += acc[((k << ls) + sl) * P.acc_pitch + r];
      if (failed) v = nan;
      if (gridDim.y == 1) {
        T* dst = out + (r0 + r) * nkeys + k;
        *dst   = T(reset ? v : double(*dst) + v);
      } else {
        partial[(size_t(blockIdx.y) * nrows + r0) * nkeys + i] = v;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kCbk32Consumers) : "memory");  // the table is rewritten by the next row tile
  }
}

template <typename T, typename KeyT>
cudaError_t launch_cols_by_key_rows32(T* out,
                                      const T* data,
                                      const KeyT* keys,
                                      int64_t nrows,
                                      int64_t ncols,
                                      int64_t nkeys,
                                      bool reset,
                                      cudaStream_t stream,
                                      const Cbk32Plan& p,
                                      Workspace ws)
{
  Scratch scratch(ws, p.total, stream);
  if (scratch.error() != cudaSuccess) return scratch.error();
  unsigned char* base    = static_cast<unsigned char*>(scratch.get());
  unsigned short* perm16 = reinterpret_cast<unsigned short*>(base + p.off_perm_g);
  unsigned short* offs16 = reinterpret_cast<unsigned short*>(base + p.off_offs_g);
  double* partial        = reinterpret_cast<double*>(base + p.off_part_g);
  const int nk           = int(nkeys);
  (void)launch_dep(cbk_sort_kernel<KeyT>, dim3(unsigned(p.n_chunks)), dim3(kCbkTpb), size_t(nk) * sizeof(int), stream,
                   keys, ncols, nk, p.CH, p.offs_stride, perm16, offs16);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const dim3 grid{unsigned(ceil_div<int64_t>(p.n_row_tiles, p.row_tiles_per_cta)), unsigned(p.y_split), 1u};
#define B2R_LAUNCH_WALK(IPW_)                                                                                      \
  do {                                                                                                             \
    auto kern = cbk_rows32_kernel<T, IPW_>;                                                                        \
    e         = ensure_dynamic_smem(kern, p.smem);                                                                 \
    if (e != cudaSuccess) return e;                                                                                \
    (void)launch_dep(kern, dim3(grid), dim3(kCbk32Threads), p.smem, stream,                                        \
                     out, partial, data, perm16, offs16, nrows, ncols, nk, reset, p,                               \
                                                 ring_ctl(ws.status));                                             \
  } while (0)
  if (p.items_per_warp <= 1) {
    B2R_LAUNCH_WALK(1);
  } else if (p.items_per_warp <= 2) {
    B2R_LAUNCH_WALK(2);
  } else if (p.items_per_warp <= 4) {
    B2R_LAUNCH_WALK(4);
  } else if (p.items_per_warp <= 8) {
    B2R_LAUNCH_WALK(8);
  } else {
    B2R_LAUNCH_WALK(16);  // the plan admits no more
  }
#undef B2R_LAUNCH_WALK
  e = cudaGetLastError();
  if (e != cudaSuccess || p.y_split == 1) return e;
  const int64_t cells = nrows * nkeys;
  (void)launch_dep(cbk_merge_kernel<T>, dim3(unsigned(ceil_div<int64_t>(cells, 256))), dim3(256), 0, stream, out,
                   partial, cells, p.y_split, reset);
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
