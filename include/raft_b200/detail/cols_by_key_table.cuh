// Keyed column sums, "table" form for 33 to 255 keys (fp32):
//     out[r][keys[c]] += data[r][c]          data row-major [nrows x ncols], rows on 16-byte boundaries
//
// With many keys a chunk of columns holds only a few columns per key, and the two sorted forms
// (cols_by_key_sorted.cuh, cols_by_key_walk.cuh) pay their per-segment set-up on ever shorter segments: 4.15 and
// 3.4 TB/s with 128 keys, bound by instruction issue. This form does not sort at all. The key of a column is
// the same for every row, so a LANE takes a ROW of the tile and the warp walks the columns: the accumulator of
// (key, row) lives in shared memory at table[warp][key][lane] - the bank is the lane, whatever the key, so the
// read-add-write of an element never conflicts and needs no atomic: the cell belongs to one lane. Per element
// that is a key extraction, an address, two loads, an add and a store - 10 lane-instructions as compiled, whatever
// the number of keys (the lane-per-segment kernel: 24 with 128 keys). Measured, fp32 2000 x 200000: 64 keys 6.1
// TB/s, 128 keys 5.9, 255 keys 4.6.
//
//  * Tiles are boxes of 32 rows x 228 columns (188 with eight consumer warps: more stages beside the tables)
//    fetched by ONE tiled-TMA instruction each (a ring of bulk row copies is bound by the number of
//    copies, and 32 pieces of 912 bytes would be far too many); 228 because the box lands densely in shared
//    memory and a pitch of 4 (mod 8) words lets lane r, which reads row r, avoid its neighbours: the lanes of a
//    warp are four groups of eight rows, group g reads column 4m + (g + s) % 4 in step s of column group m, so a
//    step touches 32 different banks (eight multiples of four from r % 8, plus (g + s) % 4), and after four steps
//    every lane has seen the four columns of the group.
//  * Keys travel as one byte per column (cbk_keys8_kernel: key, or the dummy slot `nkeys` for a key outside
//    [0, nkeys) and for the columns past the end) plus one flag per column group that holds a key twice, 240 bytes
//    per box beside it in the stage; a lane fetches the four keys of a column group with one broadcast load.
//  * The consumer warps (eight; four above 136 keys, where eight tables no longer leave room for three stages)
//    share the 32 rows and split the 47 or 57 column groups of a box; each has its own table ((nkeys + 1) x 32
//    floats), so nothing is shared while streaming. The four columns of a group are added all at once - four
//    cell loads in flight, four adds, four stores - when their keys differ (the flag; with no flagged group in a
//    warp's share of the box, 7 boxes of 10 with 128 keys, a copy of the walk without any branch runs), otherwise
//    two at a time with a same-cell check: if both are the same cell the second add takes the first sum.
//  * At the end of a row tile the tables are added in warp order in fp64 and written as [row][key] (or as an
//    fp64 partial when the columns are split over CTAs: cbk_merge_kernel).
//    fp32 cells see at most kCbkTableMaxAdds additions between two flushes (the planner splits the columns
//    accordingly), and the order of all additions is fixed: results repeat bit for bit.
//
// One CTA per SM; every mbarrier wait is bounded (col_reduce_tma.cuh); a CTA that gives up writes NaN and sets
// the status word.
#pragma once

#include "cols_by_key_sorted.cuh"
#include "tensor_map.cuh"

#include <utility>

namespace raft_b200 {
namespace detail {

constexpr int kCbkTableRows    = 32;                  // rows of a box: one per lane
constexpr int kCbkTableCols    = 228;                 // columns of a box; 228 words = 4 (mod 8): see above
constexpr int kCbkTableColsNarrow = 188;              // ... of the narrow box (eight consumer warps)
constexpr int kCbkTableKeyB    = 240;                 // key bytes per box, a multiple of 16
constexpr int kCbkTableDupByte = 232;                // first of the 8 bytes of duplicate flags in them
constexpr int kCbkTableMaxKeys = 255;                 // keys and the dummy slot fit a byte
constexpr int kCbkTableMaxAdds = 128;                 // fp32 additions into one cell between flushes
constexpr int kCbkTableMaxStages = 6;
constexpr size_t cbk_table_box_bytes(int cols) { return size_t(kCbkTableRows) * size_t(cols) * sizeof(float); }

B2R_DI float lds_f32(uint32_t addr)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
// f(integral_constant<int, 0>), ..., f(integral_constant<int, N - 1>): a loop whose index is a compile-time constant
template <typename F, int... I>
B2R_DI void static_for_impl(F&& f, std::integer_sequence<int, I...>)
{
  (f(std::integral_constant<int, I>{}), ...);
}
template <int N, typename F>
B2R_DI void static_for(F&& f)
{
  static_for_impl(f, std::make_integer_sequence<int, N>{});
}

template <int OFF>
B2R_DI float lds_f32_at(uint32_t addr)  // [addr + OFF] with the offset in the instruction
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
B2R_DI unsigned lds_u32_at(uint32_t addr)
{
  unsigned v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
B2R_DI void sts_f32(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
B2R_DI unsigned lds_u32(uint32_t addr)
{
  unsigned v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// cells a0 / a1 += x0 / x1, in this order, with both cell loads in flight together
B2R_DI void table_add_pair(uint32_t a0, float x0, uint32_t a1, float x1)
{
  const float c0 = lds_f32(a0);
  const float c1 = lds_f32(a1);
  const float v0 = c0 + x0;
  const float v1 = (a1 == a0 ? v0 : c1) + x1;
  sts_f32(a0, v0);
  sts_f32(a1, v1);  // the same cell: the later store holds both additions
}

struct CbkTablePlan {
  bool ok;
  int warps;   // consumer warps: 8 while their tables leave room for three stages, 4 above
  int cols;    // columns of a box: 228, or 188 when that makes room for a fourth stage
  int stages;
  int n_chunks;
  int y_split;
  int chunks_per_cta;
  int64_t n_row_tiles;
  int64_t row_tiles_per_cta;
  size_t table_bytes;  // per warp
  size_t stage_bytes;
  size_t smem;
  size_t off_keys_g, off_part_g, total;  // scratch in global memory
};

template <typename T>
inline CbkTablePlan plan_cols_by_key_table(const T* data, int64_t nrows, int64_t ncols, int64_t nkeys)
{
  CbkTablePlan p = {};
  if (!std::is_same<T, float>::value || nkeys < 1 || nkeys > kCbkTableMaxKeys || nrows < 1 ||
      ncols < kCbkTableCols || ncols % 4 != 0 || !aligned16(data) || ncols > (int64_t(1) << 30))
    return p;
  p.cols = kCbkTableCols;
  p.warps       = nkeys <= tuning().colkey_table_w8_max ? 8 : 4;
  p.table_bytes = size_t(nkeys + 1) * 32 * sizeof(float);
  const size_t budget = size_t(224) << 10;
  const size_t tables = size_t(p.warps) * p.table_bytes;
  auto stages_with    = [&](int cols) {
    const size_t sb = align_up(cbk_table_box_bytes(cols) + kCbkTableKeyB, 128);
    return tables + 2 * sb > budget ? 0 : int((budget - tables) / sb);
  };
  // With eight consumer warps the narrow box: more, smaller stages for the same bytes in flight, and four stages
  // instead of three beside the tables of 128 keys (measured, 228 / 188 columns: 64 keys 5.93 / 6.08 TB/s, 100
  // keys 6.05 / 6.14, 128 keys 5.65 / 5.9; 148 columns lose - 5.3 to 5.6 - their row pieces are too short; two
  // stages instead of three cost a fifth). With four warps the stages do not matter: the warps bound the kernel.
  const int knob = tuning().colkey_table_cols;
  if (knob == kCbkTableColsNarrow || (knob == 0 && p.warps == 8 && stages_with(kCbkTableColsNarrow) >= 4))
    p.cols = kCbkTableColsNarrow;
  p.stage_bytes = align_up(cbk_table_box_bytes(p.cols) + kCbkTableKeyB, 128);
  int st        = stages_with(p.cols);
  if (st < 2) return p;
  p.stages = st > kCbkTableMaxStages ? kCbkTableMaxStages : st;
  p.smem   = tables + size_t(p.stages) * p.stage_bytes;
  p.n_chunks    = int(ceil_div<int64_t>(ncols, p.cols));
  p.n_row_tiles = ceil_div<int64_t>(nrows, kCbkTableRows);
  if (p.n_row_tiles > int64_t(0x7fffffff) / kCbkTableRows) return p;
  // columns between two flushes of a table: at most kCbkTableMaxAdds additions into a cell on average
  const int64_t max_cpc = std::max<int64_t>(1, int64_t(kCbkTableMaxAdds) * p.warps * nkeys / p.cols);
  int y_min             = int(ceil_div<int64_t>(p.n_chunks, max_cpc));
  if (int64_t(y_min) > 65535) return p;
  const int y_knob = tuning().colkey_table_y;  // experiments: this many column splits at least
  if (y_knob > y_min && y_knob <= p.n_chunks) y_min = y_knob;
  // the split of the columns that needs the fewest waves of one CTA per SM; a row tile costs its boxes plus a
  // flush (about six boxes' worth), a split costs the merge
  const int slots   = sm_count();
  int64_t best_cost = 0;
  for (int y = y_min; y <= (y_knob > 0 ? y_min : std::max(y_min, 2 * slots)) && y <= p.n_chunks; ++y) {
    const int cpc       = int(ceil_div<int64_t>(p.n_chunks, y));
    const int ys        = int(ceil_div<int64_t>(p.n_chunks, cpc));
    const int64_t per_x = p.n_row_tiles * ys > slots ? ceil_div<int64_t>(p.n_row_tiles * ys, slots) : 1;
    const int64_t rtpc  = per_x < p.n_row_tiles ? per_x : p.n_row_tiles;
    const int64_t gx    = ceil_div<int64_t>(p.n_row_tiles, rtpc);
    const int64_t waves = ceil_div<int64_t>(gx * ys, slots);
    const int64_t cost  = waves * rtpc * (cpc + 6) + (ys > 1 ? 50 : 0);
    if (best_cost == 0 || cost < best_cost) {
      best_cost           = cost;
      p.y_split           = ys;
      p.chunks_per_cta    = cpc;
      p.row_tiles_per_cta = rtpc;
    }
  }
  if (best_cost == 0) return p;
  size_t o     = 0;
  p.off_keys_g = o;
  o += align_up(size_t(p.n_chunks) * kCbkTableKeyB, 256);
  p.off_part_g = o;
  if (p.y_split > 1) o += align_up(size_t(p.y_split) * size_t(nrows) * size_t(nkeys) * sizeof(double), 256);
  p.total = o;
  p.ok    = true;
  return p;
}

// keys8[chunk][240]: bytes 0..227 the key of every column of the chunk, `nkeys` (a slot nobody reads) for keys
// outside [0, nkeys) - their columns are dropped, as in the other forms - and past the last column; bytes 232..239
// one bit per column group of four: set when two of its columns have the same key (the consumers then add the
// four one after the other instead of all at once)
template <typename KeyT>
B2R_DI int cbk_table_key(const KeyT* __restrict__ keys, int64_t c, int64_t ncols, int nkeys)
{
  if (c >= ncols) return nkeys;
  const long long kv = static_cast<long long>(keys[c]);
  return (kv >= 0 && kv < nkeys) ? int(kv) : nkeys;
}

template <typename KeyT>
__global__ void __launch_bounds__(256) cbk_keys8_kernel(unsigned char* __restrict__ keys8,
                                                       const KeyT* __restrict__ keys,
                                                       int64_t ncols,
                                                       int nkeys,
                                                       int n_chunks,
                                                       int cols)
{
  grid_dep_sync();
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= int64_t(n_chunks) * kCbkTableKeyB) return;
  const int ch     = int(i / kCbkTableKeyB);
  const int j      = int(i - int64_t(ch) * kCbkTableKeyB);
  const int64_t c0 = int64_t(ch) * cols;
  int v            = nkeys;
  if (j < cols) {
    v = cbk_table_key(keys, c0 + j, ncols, nkeys);
  } else if (j >= kCbkTableDupByte) {
    v = 0;
    for (int b = 0; b < 8; ++b) {
      const int m = (j - kCbkTableDupByte) * 8 + b;
      if (m >= cols / 4) break;
      const int k0 = cbk_table_key(keys, c0 + 4 * m, ncols, nkeys), k1 = cbk_table_key(keys, c0 + 4 * m + 1, ncols, nkeys);
      const int k2 = cbk_table_key(keys, c0 + 4 * m + 2, ncols, nkeys), k3 = cbk_table_key(keys, c0 + 4 * m + 3, ncols, nkeys);
      if (k0 == k1 || k0 == k2 || k0 == k3 || k1 == k2 || k1 == k3 || k2 == k3) v |= 1 << b;
    }
  }
  keys8[i] = static_cast<unsigned char>(v);
}

template <typename T, int W, int COLS>
__global__ void __launch_bounds__(W * 32 + 32, 1) cbk_table_kernel(T* __restrict__ out,
                                                                 double* __restrict__ partial,
                                                                 const __grid_constant__ CUtensorMap tmap,
                                                                 const unsigned char* __restrict__ keys8,
                                                                 int64_t nrows,
                                                                 int nkeys,
                                                                 bool reset,
                                                                 CbkTablePlan P,
                                                                 RingCtl ctl)
{
  extern __shared__ __align__(128) unsigned char smem_tma[];
  constexpr int n_cons      = W * 32;
  constexpr int NG          = COLS / 4;            // column groups of a box
  constexpr int NC          = NG / W;              // groups every warp has
  constexpr int EX          = NG % W;              // the first EX warps have one more
  constexpr int GPW         = NC + (EX != 0 ? 1 : 0);
  constexpr size_t kBoxBytes = cbk_table_box_bytes(COLS);
  static_assert(COLS % 8 == 4 && COLS + 8 <= kCbkTableDupByte + 8 && GPW <= 16, "pitch = 4 (mod 8) words; flags behind the keys");
  unsigned char* stages     = smem_tma + size_t(W) * P.table_bytes;
  const uint32_t tables_u32 = smem_u32(smem_tma);
  const uint32_t stages_u32 = smem_u32(stages);
  __shared__ __align__(8) uint64_t s_full[kCbkTableMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kCbkTableMaxStages];
  __shared__ int s_abort;

  const int tid       = threadIdx.x;
  const bool producer = tid >= n_cons;
  const int STAGES    = P.stages;
  const int64_t rt0   = int64_t(blockIdx.x) * P.row_tiles_per_cta;
  int64_t rt1         = rt0 + P.row_tiles_per_cta;
  rt1                 = rt1 < P.n_row_tiles ? rt1 : P.n_row_tiles;
  // The CTAs that share a row tile take its boxes in turn (box y, y + gridDim.y, ...): running at the same pace
  // they fetch neighbouring 912-byte pieces of the same 32 matrix rows at about the same time, which is what
  // DRAM pages want - a contiguous range of boxes per CTA ran at 4.4 TB/s.
  const int ch0       = blockIdx.y;
  const int ch_step   = gridDim.y;
  const int n_ch      = ch0 < P.n_chunks ? (P.n_chunks - ch0 + ch_step - 1) / ch_step : 0;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], W);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the tables start at zero
  for (uint32_t i = uint32_t(tid) * 16u; i < uint32_t(W) * uint32_t(P.table_bytes); i += blockDim.x * 16u)
    *reinterpret_cast<float4*>(smem_tma + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  grid_dep_sync();  // the set-up above touches shared memory only
  volatile int* abort_flag = &s_abort;

  if (producer) {
    if (tid == n_cons) {  // one elected thread issues every copy
      long long issued = 0;
      bool alive       = true;
      for (int64_t rti = rt0; rti < rt1 && alive; ++rti) {
        for (int c = 0; c < n_ch; ++c) {
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
          const int ch      = ch0 + c * ch_step;
          unsigned char* st = stages + size_t(s) * P.stage_bytes;
          mbar_expect_tx(&s_full[s], unsigned(kBoxBytes) + unsigned(kCbkTableKeyB));  // zero fill included
          tma_load_2d(st, &tmap, ch * COLS, int(rti * kCbkTableRows), &s_full[s]);
          bulk_load(st + kBoxBytes, keys8 + size_t(ch) * kCbkTableKeyB, unsigned(kCbkTableKeyB), &s_full[s]);
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
  const int grp  = lane >> 3;  // which of the four columns of a group this lane reads first
  // this warp's column groups of every box
  const int g0         = warp * NC + (warp < EX ? warp : EX);
  const bool has_extra = warp < EX;
  const uint32_t cell0 = tables_u32 + uint32_t(warp) * uint32_t(P.table_bytes) + uint32_t(lane) * 4u;  // (key 0, lane)
  unsigned sel[4], dcol[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const unsigned q = unsigned(grp + s) & 3u;
    sel[s]           = q | 0x4440u;  // byte q of the four keys, zero-extended
    dcol[s]          = uint32_t(lane) * uint32_t(COLS * sizeof(float)) + q * 4u + 16u * unsigned(g0);
  }

  long long seq = 0;
  RingPos rp{0, 0u};
  bool dead     = false;
  for (int64_t rti = rt0; rti < rt1; ++rti) {
    const int64_t r0 = rti * kCbkTableRows;
    const int rt     = int(nrows - r0 < kCbkTableRows ? nrows - r0 : kCbkTableRows);
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
      const uint32_t keys = st + uint32_t(kBoxBytes) + 4u * unsigned(g0);
      const uint32_t rb0 = st + dcol[0], rb1 = st + dcol[1], rb2 = st + dcol[2], rb3 = st + dcol[3];
      // the keys of all groups of the warp and the duplicate flags first: one latency per box, not per group
      unsigned kk[GPW];
      static_for<GPW>([&](auto jc) { kk[decltype(jc)::value] = lds_u32_at<4 * decltype(jc)::value>(keys); });  // (the last one only counts for a warp with an extra group)
      const unsigned dlo = lds_u32(st + uint32_t(kBoxBytes) + uint32_t(kCbkTableDupByte));
      const unsigned dhi = lds_u32(st + uint32_t(kBoxBytes) + uint32_t(kCbkTableDupByte) + 4u);
      const unsigned dup = unsigned(((static_cast<unsigned long long>(dhi) << 32) | dlo) >> g0);
      float x[2][4];
      x[0][0] = lds_f32(rb0);
      x[0][1] = lds_f32(rb1);
      x[0][2] = lds_f32(rb2);
      x[0][3] = lds_f32(rb3);
      // every warp has NC groups, the first EX warps one more (57 = 8 x 7 + 1, 47 = 8 x 5 + 7). Two copies of the
      // walk: when no group of the warp has two columns of one key (7 boxes of 10 with 128 keys) the first runs,
      // straight-line code that adds the four columns of a group all at once; a branch per group would cost
      // three control instructions per four elements.
      const unsigned mine = has_extra ? (1u << GPW) - 1u : (1u << NC) - 1u;
      auto walk = [&](auto fast_c) {
        constexpr bool kFast = decltype(fast_c)::value;
        static_for<GPW>([&](auto jc) {
          constexpr int j = decltype(jc)::value;
          if (j < NC || has_extra) {
            const float* xc = x[j & 1];
            if constexpr (j + 1 < GPW) {  // the next group's elements are on their way while this one is added
              float* xn = x[(j + 1) & 1];
              xn[0]     = lds_f32_at<16 * (j + 1)>(rb0);
              xn[1]     = lds_f32_at<16 * (j + 1)>(rb1);
              xn[2]     = lds_f32_at<16 * (j + 1)>(rb2);
              xn[3]     = lds_f32_at<16 * (j + 1)>(rb3);
            }
            const uint32_t a0 = cell0 + __byte_perm(kk[j], 0u, sel[0]) * 128u;
            const uint32_t a1 = cell0 + __byte_perm(kk[j], 0u, sel[1]) * 128u;
            const uint32_t a2 = cell0 + __byte_perm(kk[j], 0u, sel[2]) * 128u;
            const uint32_t a3 = cell0 + __byte_perm(kk[j], 0u, sel[3]) * 128u;
            if (kFast || ((dup >> j) & 1u) == 0u) {  // four different cells (the same for every lane): all at once
              const float c0 = lds_f32(a0), c1 = lds_f32(a1), c2 = lds_f32(a2), c3 = lds_f32(a3);
              sts_f32(a0, c0 + xc[0]);
              sts_f32(a1, c1 + xc[1]);
              sts_f32(a2, c2 + xc[2]);
              sts_f32(a3, c3 + xc[3]);
            } else {
              table_add_pair(a0, xc[0], a1, xc[1]);
              table_add_pair(a2, xc[2], a3, xc[3]);
            }
          }
        });
      };
      if (__all_sync(0xffffffffu, (dup & mine) == 0u)) {
        walk(std::true_type{});
      } else {
        walk(std::false_type{});
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
    }
    // end of the row tile: cell (key, row) = the W tables added in warp order, in fp64. Thread (warp, lane) takes
    // row `lane` of the keys warp, warp + W, ... - conflict-free table reads - clears what it read and writes the
    // sum straight out: at any moment the W warps write W neighbouring keys of the same 32 rows, which the L2
    // puts together into whole sectors.
    asm volatile("bar.sync 1, %0;" ::"r"(n_cons) : "memory");
    const bool failed = *abort_flag != 0;
    const double nan  = __longlong_as_double(0x7ff8000000000000ll);
    for (int k = warp; k < nkeys; k += W) {
      double v = 0.0;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        const uint32_t a = tables_u32 + uint32_t(w) * uint32_t(P.table_bytes) + uint32_t(k) * 128u + uint32_t(lane) * 4u;
        v += double(lds_f32(a));
        sts_f32(a, 0.f);
      }
      if (failed) v = nan;
      if (lane < rt) {
        if (gridDim.y == 1) {
          T* dst = out + (r0 + lane) * nkeys + k;
          *dst   = T(reset ? v : double(*dst) + v);
        } else {
          partial[(size_t(blockIdx.y) * nrows + r0 + lane) * nkeys + k] = v;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(n_cons) : "memory");  // the tables are zero again for the next row tile
  }
}

template <typename T, typename KeyT>
cudaError_t launch_cols_by_key_table(T* out,
                                     const T* data,
                                     const KeyT* keys,
                                     int64_t nrows,
                                     int64_t ncols,
                                     int64_t nkeys,
                                     bool reset,
                                     cudaStream_t stream,
                                     const CbkTablePlan& p,
                                     Workspace ws,
                                     bool* unavailable)
{
  *unavailable = false;
  if constexpr (!std::is_same<T, float>::value) {
    *unavailable = true;
    return cudaSuccess;
  } else {
    CUtensorMap tmap;
    if (make_tensor_map_2d<float>(&tmap, data, nrows, ncols, ncols, kCbkTableRows, p.cols) != cudaSuccess) {
      *unavailable = true;  // no tensor map (driver entry point missing): the caller takes another form
      return cudaSuccess;
    }
    Scratch scratch(ws, p.total, stream);
    if (scratch.error() != cudaSuccess) return scratch.error();
    unsigned char* base  = static_cast<unsigned char*>(scratch.get());
    unsigned char* keys8 = base + p.off_keys_g;
    double* partial      = reinterpret_cast<double*>(base + p.off_part_g);
    const int nk         = int(nkeys);
    const int64_t nb     = int64_t(p.n_chunks) * kCbkTableKeyB;
    (void)launch_dep(cbk_keys8_kernel<KeyT>, dim3(unsigned(ceil_div<int64_t>(nb, 256))), dim3(256), 0, stream, keys8,
                     keys, ncols, nk, p.n_chunks, p.cols);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    auto kern = p.cols == kCbkTableCols
                  ? (p.warps == 8 ? cbk_table_kernel<T, 8, kCbkTableCols> : cbk_table_kernel<T, 4, kCbkTableCols>)
                  : (p.warps == 8 ? cbk_table_kernel<T, 8, kCbkTableColsNarrow> : cbk_table_kernel<T, 4, kCbkTableColsNarrow>);
    e         = ensure_dynamic_smem(kern, p.smem);
    if (e != cudaSuccess) return e;
    const dim3 grid{unsigned(ceil_div<int64_t>(p.n_row_tiles, p.row_tiles_per_cta)), unsigned(p.y_split), 1u};
    (void)launch_dep(kern, dim3(grid), dim3(p.warps * 32 + 32), p.smem, stream, out, partial, tmap, keys8, nrows, nk,
                     reset, p, ring_ctl(ws.status));
    e = cudaGetLastError();
    if (e != cudaSuccess || p.y_split == 1) return e;
    const int64_t cells = nrows * nkeys;
    (void)launch_dep(cbk_merge_kernel<T>, dim3(unsigned(ceil_div<int64_t>(cells, 256))), dim3(256), 0, stream, out,
                     partial, cells, p.y_split, reset);
    return cudaGetLastError();
  }
}

}  // namespace detail
}  // namespace raft_b200
