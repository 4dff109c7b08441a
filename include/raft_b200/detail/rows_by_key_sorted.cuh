// Keyed row sums, "sort then stream" formulation:
//     sums[keys[i]][:] += w[i] * A[i][:]
//
// Five kernels, no floating-point atomics, every matrix row read from HBM once:
//
//  rbk_sort_kernel     one CTA per window of W consecutive rows (W <= 65536, sized so that the
//                      windows fill whole waves of resident CTAs). Counting sort of the window's row
//                      offsets by key with integer shared-memory atomics: perm[window][.] (16-bit
//                      offsets staged in shared memory, written out coalesced) and offs[window][k].
//  rbk_units_kernel    one CTA per GROUP of consecutive windows (the group size is chosen so that a key
//                      has about kUnitTarget rows per group, whatever the number of keys): rows of every
//                      key in the group, prefix sum over the keys -> the work units (at most
//                      1.5 x that many rows of one key each, split evenly) and the list of (group, key)
//                      pairs that got more than one unit.
//  rbk_stream_kernel   one warp per work unit, units handed out dynamically: the warp finds the
//                      unit's rows through the sorted windows (a search over at most 32 segment
//                      counts held one per lane), streams them (a sub-warp of G lanes per row, 8 row
//                      loads in flight per lane), keeps a wide / compensated sum per column in
//                      REGISTERS and writes ONE partial row per unit. Nothing is shared between
//                      warps, so occupancy - and with it the bytes in flight - is not limited by an
//                      accumulator table; long runs of one key are spread over many warps
//                      (skew-proof); a handful of keys is as fast as tens of thousands.
//  rbk_fold_kernel     one warp per listed (group, key): folds its units' partial rows into the
//                      first of them.
//  rbk_merge_kernel    one warp (many keys) or one CTA (few keys) per key: folds the key's partial
//                      rows over all groups in a fixed order, adds to or overwrites sums, and derives
//                      the exact int64 row counts from the sort's offsets.
//
// Extra memory traffic over the matrix itself: the keys are read twice, one 4-byte index per row
// is written and read once, and one fp64 partial row per ~128 matrix rows is written and read -
// about 4 % for 128 fp32 columns.
#pragma once

#include "common.cuh"
#include "launch.cuh"
#include "ops.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kUnitTarget  = 128;    // rows per work unit aimed for, at least (B2R_KEY_UNIT_ROWS sets it)
constexpr int kMaxGroup    = 32;     // windows per group at most (one lane per window)
constexpr int kSortTpb     = 1024;
constexpr int kMaxSortKeys = 24576;  // histogram + cursors (8 bytes per key) must fit shared memory

// Rows of one key that a warp sums into one partial row. Every unit costs a 8-byte-per-column partial row that is
// written and read once more, so long units save traffic (10^7 x 128, 1024 keys: 128 rows 760 + 25 us in the
// stream and merge kernels, 384 rows 746 + 16); short ones keep enough units per resident warp for the queue to
// level the warps out at the end. Eight units per resident warp, between 128 and 384 rows.
inline int rbk_unit_target(int64_t nrows)
{
  const int knob = tuning().key_unit_rows;
  if (knob >= 16 && knob <= 4096) return knob;
  int64_t t = nrows / (int64_t(sm_count()) * 24 * 8);
  t         = t / 32 * 32;
  return int(t < kUnitTarget ? kUnitTarget : (t > 384 ? 384 : t));
}
inline int rbk_unit_cap(int64_t nrows) { return rbk_unit_target(nrows) * 3 / 2; }  // rows per work unit at most

struct SortedPlan {
  int vec;
  int window_rows;  // W, a multiple of 1024, at most 65536
  int n_windows;
  int group;        // windows per group
  int n_groups;
  int max_units;    // per group
  int max_fold;     // (group, key) pairs with more than one unit, at most
  size_t off_perm, off_offs, off_gcnt, off_uoffs, off_ukey, off_ufirst, off_ulen, off_fold, off_counter, off_part,
    total;
};

// STAGED: the window's permutation is built in shared memory as 16-bit offsets (W <= 65536) and
// written out with coalesced stores; otherwise every row's slot is stored straight to global
// memory (32 sectors per warp store).
template <typename KeyT, bool STAGED>
__global__ void __launch_bounds__(kSortTpb) rbk_sort_kernel(const KeyT* __restrict__ keys,
                                                           int64_t nrows,
                                                           int nkeys,
                                                           int W,
                                                           unsigned* __restrict__ perm,
                                                           int* __restrict__ offs,
                                                           int* __restrict__ unit_counter)
{
  grid_dep_sync();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unit_counter[0] = 0;  // the stream kernel's work queue
    unit_counter[1] = 0;  // length of the fold list
  }
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* s_cnt             = reinterpret_cast<int*>(smem_raw);                  // [nkeys] counts
  int* s_cur             = s_cnt + nkeys;                                     // [nkeys] scatter cursors
  unsigned short* s_perm = reinterpret_cast<unsigned short*>(s_cur + nkeys);  // [W] when STAGED
  __shared__ int s_warp[kSortTpb / 32];

  const int win      = blockIdx.x;
  const int64_t row0 = int64_t(win) * W;
  int64_t n          = nrows - row0;
  n                  = n < W ? n : W;
  const int tid      = threadIdx.x;
  const int lane     = tid & 31;
  const int warp     = tid >> 5;
  const KeyT* wkeys  = keys + row0;
  unsigned* wperm    = perm + row0;
  int* w_offs        = offs + size_t(win) * (nkeys + 1);

  for (int k = tid; k < nkeys; k += kSortTpb)
    s_cnt[k] = 0;
  __syncthreads();
  constexpr int KU = 8;  // independent key loads in flight per thread
  for (int64_t i0 = 0; i0 < n; i0 += int64_t(KU) * kSortTpb) {
    int kk[KU];
#pragma unroll
    for (int j = 0; j < KU; ++j) {
      const int64_t i = i0 + int64_t(j) * kSortTpb + tid;
      kk[j]           = i < n ? static_cast<int>(wkeys[i]) : -1;
      if (unsigned(kk[j]) >= unsigned(nkeys)) kk[j] = -1;  // a key outside [0, nkeys) drops its row
    }
#pragma unroll
    for (int j = 0; j < KU; ++j)
      if (kk[j] >= 0) atomicAdd(&s_cnt[kk[j]], 1);
  }
  __syncthreads();

  // exclusive scan of the counts over [0, nkeys)
  const int per = (nkeys + kSortTpb - 1) / kSortTpb;
  const int b0  = tid * per;
  int local     = 0;
  for (int i = 0; i < per; ++i)
    if (b0 + i < nkeys) local += s_cnt[b0 + i];
  int incl = local;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += a;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < warp; ++w)
    base += s_warp[w];
  int run = base + incl - local;
  for (int i = 0; i < per; ++i) {
    const int k = b0 + i;
    if (k < nkeys) {
      w_offs[k] = run;
      s_cur[k]  = run;
      run += s_cnt[k];
    }
  }
  if (tid == kSortTpb - 1) w_offs[nkeys] = run;
  __syncthreads();
  for (int64_t i0 = 0; i0 < n; i0 += int64_t(KU) * kSortTpb) {
    int kk[KU];
#pragma unroll
    for (int j = 0; j < KU; ++j) {
      const int64_t i = i0 + int64_t(j) * kSortTpb + tid;
      kk[j]           = i < n ? static_cast<int>(wkeys[i]) : -1;
      if (unsigned(kk[j]) >= unsigned(nkeys)) kk[j] = -1;  // a key outside [0, nkeys) drops its row
    }
#pragma unroll
    for (int j = 0; j < KU; ++j) {
      if (kk[j] >= 0) {
        const int pos = atomicAdd(&s_cur[kk[j]], 1);
        if constexpr (STAGED) {
          s_perm[pos] = static_cast<unsigned short>(i0 + int64_t(j) * kSortTpb + tid);
        } else {
          wperm[pos] = static_cast<unsigned>(i0 + int64_t(j) * kSortTpb + tid);
        }
      }
    }
  }
  if constexpr (STAGED) {
    __syncthreads();
    for (int64_t i = tid; i < n; i += kSortTpb)
      wperm[i] = s_perm[i];
  }
}

// One CTA per group, keys taken TPB at a time so that loads and stores coalesce. First the rows of every key in
// the group's windows, gcnt[g][k] (the merge adds them up to the exact row counts), then from them:
//   uoffs[g][nkeys + 1]            first work unit of each key
//   ukey / ufirst / ulen [max_units]  per unit: key, ordinal of its first row among the key's rows
//                                  of the group, and row count (an even split into
//                                  ceil(rows / unit_cap) units)
//   fold_list                      (g * nkeys + k) of every key that got more than one unit
template <int TPB>
__global__ void __launch_bounds__(TPB) rbk_units_kernel(const int* __restrict__ offs,
                                                       int n_windows,
                                                       int group,
                                                       int* __restrict__ gcnt,
                                                       int nkeys,
                                                       int max_units,
                                                       int unit_cap,
                                                       int* __restrict__ uoffs,
                                                       int* __restrict__ ukey,
                                                       int* __restrict__ ufirst,
                                                       int* __restrict__ ulen,
                                                       int* __restrict__ fold_list,
                                                       int* __restrict__ fold_count)
{
  grid_dep_sync();
  static_assert(TPB / 32 <= 32, "one warp scans the warp totals");
  __shared__ int s_warp[TPB / 32];
  __shared__ int s_total;
  const int g    = blockIdx.x;
  const int tid  = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  int* cnt       = gcnt + size_t(g) * nkeys;
  const int w0   = g * group;
  int nw         = n_windows - w0;
  nw             = nw < group ? nw : group;
  int* g_uoffs   = uoffs + size_t(g) * (nkeys + 1);
  int* g_ukey    = ukey + size_t(g) * max_units;
  int* g_ufirst  = ufirst + size_t(g) * max_units;
  int* g_ulen    = ulen + size_t(g) * max_units;

  int run = 0;  // units of the keys before this tile
  for (int k0 = 0; k0 < nkeys; k0 += TPB) {
    const int k  = k0 + tid;
    int t        = 0;
    if (k < nkeys) {
      const int* wo = offs + size_t(w0) * (nkeys + 1) + k;
#pragma unroll 8
      for (int w = 0; w < nw; ++w)
        t += wo[size_t(w) * (nkeys + 1) + 1] - wo[size_t(w) * (nkeys + 1)];
      cnt[k] = t;
    }
    const int nu = (t + unit_cap - 1) / unit_cap;
    int inc      = nu;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += a;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int v = lane < TPB / 32 ? s_warp[lane] : 0;
      int wi      = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += a;
      }
      if (lane < TPB / 32) s_warp[lane] = wi - v;  // exclusive
      if (lane == 31) s_total = wi;
    }
    __syncthreads();
    const int u_first = run + s_warp[warp] + inc - nu;
    if (k < nkeys) {
      g_uoffs[k] = u_first;
      if (nu > 0) {
        const int each = t / nu, extra = t % nu;  // even split: `extra` units get one more row
        for (int j = 0; j < nu; ++j) {
          g_ukey[u_first + j]   = k;
          g_ufirst[u_first + j] = j * each + (j < extra ? j : extra);
          g_ulen[u_first + j]   = each + (j < extra ? 1 : 0);
        }
        if (nu > 1) fold_list[atomicAdd(fold_count, 1)] = g * nkeys + k;
      }
    }
    run += s_total;
    __syncthreads();  // s_warp and s_total are rewritten by the next tile
  }
  if (tid == 0) g_uoffs[nkeys] = run;
}

// One warp per work unit; units are handed out through a global counter (zeroed by the sort
// kernel), in (group, key) order, so that the warps finish within one unit of each other.
//
// The unit's rows are ordinals [first, first + len) in the concatenation, over the group's
// windows, of the key's segments of the sorted windows. Lane j holds the segment of window j
// (start and inclusive running count); an ordinal finds its window by a five-step search over the
// lanes' running counts (shuffles), then its row through the window's sorted list. With eight or
// more lanes per row the warp translates 32 ordinals at once, one per lane, and hands the row
// numbers out by shuffle; narrower matrices translate per load.
// (Four CTAs per SM: the kernel fits 64 registers without spills, and 32 warps x 8 rows of 512 bytes are 128 KB in
// flight per SM instead of 96 KB with three - 10^7 x 128: 6.39 -> 6.42-6.52 TB/s end to end.)
template <typename DataT, typename WeightT, typename SumT, int VEC>
__global__ void __launch_bounds__(256, 4) rbk_stream_kernel(typename sum_state<SumT>::type::carry_t* __restrict__ partial,
                                                        const DataT* __restrict__ A,
                                                        int64_t lda,
                                                        const WeightT* __restrict__ weights,
                                                        int ncols,
                                                        int nkeys,
                                                        int W,
                                                        int n_windows,
                                                        int group,
                                                        int n_groups,
                                                        int max_units,
                                                        int G,
                                                        int col_split,
                                                        const unsigned* __restrict__ perm,
                                                        const int* __restrict__ offs,
                                                        const int* __restrict__ uoffs,
                                                        const int* __restrict__ ukey,
                                                        const int* __restrict__ ufirst,
                                                        const int* __restrict__ ulen,
                                                        int* __restrict__ unit_counter)
{
  grid_dep_sync();
  using State     = typename sum_state<SumT>::type;
  using CarryT    = typename State::carry_t;
  constexpr int Q = 8;  // row loads in flight per lane
  const op::Add add{};
  const int lane = threadIdx.x & 31;
  const int lg   = 31 - __clz(G);
  const int lig  = lane & (G - 1);
  const int grp  = lane >> lg;
  const int gpw  = 32 >> lg;
  const int nvec = ncols / VEC;  // VEC divides ncols on the vector path
  // a queue item is (unit, part of the columns): with few rows but long ones the columns of a unit
  // are cut into col_split parts, so that there are enough items for every warp
  const int64_t total_items = int64_t(n_groups) * max_units * col_split;
  const int passes          = (nvec + G - 1) / G;
  const int passes_per_part = (passes + col_split - 1) / col_split;
  while (true) {
    long long item = 0;
    if (lane == 0) item = atomicAdd(unit_counter, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= total_items) break;
    const long long slot = col_split > 1 ? item / col_split : item;
    const int part       = col_split > 1 ? int(item - slot * col_split) : 0;
    const int g = int(slot / max_units);
    const int u = int(slot - int64_t(g) * max_units);
    if (u >= uoffs[size_t(g) * (nkeys + 1) + nkeys]) continue;  // this group has fewer units
    const int key   = ukey[slot];
    const int first = ufirst[slot];
    const int len   = ulen[slot];
    const int w0    = g * group;
    int nw          = n_windows - w0;
    nw              = nw < group ? nw : group;
    int my_beg = 0, my_cnt = 0;
    if (lane < nw) {
      const int* wo = offs + size_t(w0 + lane) * (nkeys + 1);
      my_beg        = wo[key];
      my_cnt        = wo[key + 1] - my_beg;
    }
    int my_end = my_cnt;  // rows of the key in windows 0..lane of the group
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, my_end, off);
      if (lane >= off) my_end += a;
    }
    const int64_t grow0   = int64_t(w0) * W;  // first matrix row of the group
    const unsigned* gperm = perm + grow0;
    // row (relative to grow0) of the unit's i-th row; every lane must call it (shuffles inside)
    auto translate = [&](int i) -> unsigned {
      const int o = first + (i < len ? i : len - 1);
      int lo      = 0;  // first window whose running count exceeds o
#pragma unroll
      for (int step = 16; step > 0; step >>= 1) {
        const int probe = __shfl_sync(0xffffffffu, my_end, lo + step - 1);
        if (probe <= o) lo += step;
      }
      const int w_end = __shfl_sync(0xffffffffu, my_end, lo);
      const int w_cnt = __shfl_sync(0xffffffffu, my_cnt, lo);
      const int w_beg = __shfl_sync(0xffffffffu, my_beg, lo);
      const unsigned in_win = unsigned(lo) * unsigned(W);
      return in_win + gperm[in_win + unsigned(w_beg + (o - (w_end - w_cnt)))];
    };
    CarryT* dst = partial + size_t(slot) * ncols;
    const int cv_beg = part * passes_per_part * G;
    int cv_end       = cv_beg + passes_per_part * G;
    cv_end           = cv_end < nvec ? cv_end : nvec;
    for (int cv0 = cv_beg; cv0 < cv_end; cv0 += G) {
      const int cv      = cv0 + lig;
      const bool col_ok = cv < nvec;
      const DataT* col  = A + grow0 * lda + int64_t(col_ok ? cv : 0) * VEC;
      State acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        acc[e].init(SumT(0));
      // one pass of Q loads per lane: rows i0 + k * gpw + grp, k = 0..Q-1, taken from `row_of(k)`
      auto pass = [&](int i0, int limit, auto row_of) {
        VecOf<DataT, VEC> v[Q];
        SumT w[Q];
#pragma unroll
        for (int k = 0; k < Q; ++k) {
          const int64_t r = int64_t(row_of(k));
          v[k]            = load_stream<DataT, VEC>(col + r * lda);
          w[k]            = weights != nullptr ? SumT(weights[grow0 + r]) : SumT(1);
        }
#pragma unroll
        for (int k = 0; k < Q; ++k) {
          if (i0 + k * gpw + grp < limit) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              SumT x = SumT(v[k].e[e]);
              if (weights != nullptr) x *= w[k];
              acc[e].push(x, add);
            }
          }
        }
      };
      if (G >= 8) {  // Q * gpw divides 32: translate 32 rows, then hand them out
        // the look-up of the NEXT 32 rows is issued before the loads of these 32, so that its latency (a
        // dependent read of the sorted list) is hidden behind them instead of leaving the warp without a
        // load in flight once per batch
        unsigned next_row = translate(lane);
        for (int tb = 0; tb < len; tb += 32) {
          const unsigned my_row = next_row;
          if (tb + 32 < len) next_row = translate(tb + 32 + lane);
          const int nb = len - tb < 32 ? len - tb : 32;
          for (int i0 = 0; i0 < nb; i0 += Q * gpw)
            pass(i0, nb, [&](int k) { return __shfl_sync(0xffffffffu, my_row, i0 + k * gpw + grp); });
        }
      } else {
        for (int i0 = 0; i0 < len; i0 += Q * gpw)
          pass(i0, len, [&](int k) { return translate(i0 + k * gpw + grp); });
      }
      // fold the row groups of the warp (they hold different rows of the same columns)
      for (int off = G; off < 32; off <<= 1) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          State got = shfl_xor_any(acc[e], off);
          acc[e].merge(got, add);
        }
      }
      if (grp == 0 && col_ok) {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          dst[size_t(cv) * VEC + e] = acc[e].carry();
      }
    }
  }
}

// One warp per (group, key) that owns more than one work unit (the units kernel lists them):
// folds the units' partial rows, in unit order and eight rows in flight, into the FIRST of them,
// so that the final merge reads one row per group and key however many rows a key has (a single
// key may own most of the matrix).
template <typename SumT>
__global__ void __launch_bounds__(256) rbk_fold_kernel(typename sum_state<SumT>::type::carry_t* __restrict__ partial,
                                                      const int* __restrict__ uoffs,
                                                      const int* __restrict__ fold_list,
                                                      const int* __restrict__ fold_count,
                                                      int max_units,
                                                      int ncols,
                                                      int nkeys)
{
  grid_dep_sync();
  using State  = typename sum_state<SumT>::type;
  using CarryT = typename State::carry_t;
  constexpr int R = 8;
  const op::Add add{};
  const int lane  = threadIdx.x & 31;
  const int n     = *fold_count;
  for (int idx = blockIdx.x * 8 + (threadIdx.x >> 5); idx < n; idx += gridDim.x * 8) {
    const int gk  = fold_list[idx];
    const int g   = gk / nkeys;
    const int k   = gk - g * nkeys;
    const int* gu = uoffs + size_t(g) * (nkeys + 1);
    const int u0  = gu[k];
    const int u1  = gu[k + 1];
    CarryT* rows = partial + size_t(g) * max_units * ncols;
    for (int c0 = 0; c0 < ncols; c0 += 128) {
      State acc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        acc[e].init(SumT(0));
      for (int u = u0; u < u1; u += R) {
        CarryT v[R][4];
#pragma unroll
        for (int j = 0; j < R; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c0 + e * 32 + lane;
            v[j][e]     = (u + j < u1 && c < ncols) ? rows[size_t(u + j) * ncols + c] : CarryT(0);
          }
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            acc[e].push_carry(v[j][e], add);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = c0 + e * 32 + lane;
        if (c < ncols) rows[size_t(u0) * ncols + c] = acc[e].carry();
      }
    }
  }
}

// WPK warps per key (8 for few keys, so that the merge has enough loads in flight; 1 otherwise).
// Lanes run over the columns (four per lane and pass); warp s of a key folds the unit rows of
// groups s, s + WPK, ... (one row per group after rbk_fold_kernel), four loaded before any is
// consumed, and the WPK partial results are added in warp order through shared memory: the order
// of the additions is fixed.
// The last warp of the key also adds up the key's exact row count from the per-group counts.
template <typename SumT, int WPK>
__global__ void __launch_bounds__(256) rbk_merge_kernel(SumT* __restrict__ sums,
                                                       long long* __restrict__ counts,
                                                       const typename sum_state<SumT>::type::carry_t* __restrict__ partial,
                                                       const int* __restrict__ gcnt,
                                                       const int* __restrict__ uoffs,
                                                       int n_groups,
                                                       int max_units,
                                                       int ncols,
                                                       int nkeys,
                                                       bool reset)
{
  grid_dep_sync();
  using State  = typename sum_state<SumT>::type;
  using CarryT = typename State::carry_t;
  static_assert(WPK == 1 || WPK == 8, "one warp or one CTA per key");
  __shared__ CarryT s_part[WPK > 1 ? WPK : 1][128];
  const op::Add add{};
  const int lane   = threadIdx.x & 31;
  const int warp   = threadIdx.x >> 5;
  const int sub    = WPK > 1 ? warp : 0;                        // this warp's share of the groups
  const int k      = WPK > 1 ? int(blockIdx.x) : int(blockIdx.x) * 8 + warp;
  const bool valid = k < nkeys;  // uniform per CTA when WPK > 1, so the barriers below are safe

  if (valid && sub == WPK - 1 && counts != nullptr) {  // the warp that has the fewest groups to fold
    long long n = 0;
    for (int g = lane; g < n_groups; g += 32)
      n += gcnt[size_t(g) * nkeys + k];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      n += __shfl_xor_sync(0xffffffffu, n, off);
    if (lane == 0) counts[k] = (reset ? 0ll : counts[k]) + n;
  }

  for (int c0 = 0; c0 < ncols; c0 += 128) {
    State acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = c0 + e * 32 + lane;
      acc[e].init((!valid || sub != 0 || reset || c >= ncols) ? SumT(0) : sums[size_t(k) * ncols + c]);
    }
    for (int g0 = sub; valid && g0 < n_groups; g0 += 4 * WPK) {
      int u0[4], u1[4];
      CarryT first[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int g = g0 + j * WPK;
        u0[j] = u1[j] = 0;
        if (g < n_groups) {
          const int* gu = uoffs + size_t(g) * (nkeys + 1);
          u0[j]         = gu[k];
          u1[j]         = gu[k + 1];
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = c0 + e * 32 + lane;
          first[j][e] = (u1[j] > u0[j] && c < ncols)
                          ? partial[(size_t(g0 + j * WPK) * max_units + u0[j]) * ncols + c]
                          : CarryT(0);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          acc[e].push_carry(first[j][e], add);
      }
    }
    if constexpr (WPK > 1) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        s_part[warp][e * 32 + lane] = acc[e].carry();
      __syncthreads();
      if (sub == 0) {
        for (int s = 1; s < WPK; ++s) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            acc[e].push_carry(s_part[s][e * 32 + lane], add);
        }
      }
      __syncthreads();
    }
    if (valid && sub == 0) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = c0 + e * 32 + lane;
        if (c < ncols) sums[size_t(k) * ncols + c] = acc[e].value();
      }
    }
  }
}

// Shared memory of one sort CTA: histogram + cursors, and the staged 16-bit permutation.
inline size_t rbk_sort_smem(int64_t nkeys, int64_t W, bool staged)
{
  return size_t(nkeys) * 2 * sizeof(int) + (staged ? size_t(W) * sizeof(unsigned short) : 0);
}

template <typename DataT>
inline SortedPlan plan_rows_by_key_sorted(const DataT* A, int64_t lda, int64_t nrows, int64_t ncols, int64_t nkeys,
                                          size_t carry_size)
{
  constexpr int V16 = vec16<DataT>::value;
  SortedPlan p      = {};
  const bool vec_ok = V16 > 1 && ncols % V16 == 0 && lda % V16 == 0 && aligned16(A);
  p.vec             = vec_ok ? V16 : 1;

  // Window size: the sort runs one CTA per window, so the windows should fill whole waves of
  // (SMs x resident CTAs). Two CTAs of 1024 threads fit an SM when their shared memory does.
  const int64_t sm_smem = int64_t(228) << 10;  // per SM; every CTA also reserves 1 KB
  const int64_t fixed   = 1024 + 256;          // reserve + static shared memory
  const int sms         = sm_count();
  int64_t w_floor       = ceil_div<int64_t>(nkeys, 1024) * 1024;  // histogram work <= row work
  if (w_floor < 4096) w_floor = 4096;
  int64_t best_w = 0, best_cost = 0;
  for (int cps = 2; cps >= 1; --cps) {
    int64_t w_max = ((sm_smem / cps - fixed - nkeys * 8) / 2) / 1024 * 1024;
    if (w_max > 65536) w_max = 65536;
    if (w_max < 4096) continue;
    const int64_t slots = int64_t(sms) * cps;
    const int64_t waves = ceil_div<int64_t>(nrows, slots * w_max);
    int64_t W           = ceil_div<int64_t>(ceil_div<int64_t>(nrows, waves * slots), 1024) * 1024;
    if (W < w_floor) W = w_floor;
    if (W > w_max) W = w_max;
    const int64_t real_waves = ceil_div<int64_t>(ceil_div<int64_t>(nrows, W), slots);
    const int64_t cost       = real_waves * (2 * W + nkeys) * (cps == 2 ? 4 : 3);  // co-resident CTAs share an SM
    if (best_w == 0 || cost < best_cost) {
      best_w    = W;
      best_cost = cost;
    }
  }
  if (best_w == 0) best_w = 65536;  // not staged (the launcher falls back to direct stores)
  const int knob = tuning().key_window_rows;
  if (knob >= 1024 && knob <= 65536) best_w = knob;
  const int64_t W    = best_w;
  p.window_rows      = int(W);
  p.n_windows        = int(ceil_div<int64_t>(nrows, W));
  // windows per group: a key should own about kUnitTarget rows of a group
  int64_t group = (int64_t(rbk_unit_target(nrows)) * nkeys + W / 2) / W;
  if (group > kMaxGroup) group = kMaxGroup;
  if (group > p.n_windows) group = p.n_windows;
  if (group < 1) group = 1;
  p.group    = int(group);
  p.n_groups = int(ceil_div<int64_t>(p.n_windows, group));
  const int64_t group_rows    = group * W;
  const int64_t rows_in_group = nrows < group_rows ? nrows : group_rows;
  // every key present adds at most one ragged unit on top of the full ones
  const int64_t present = nkeys < rows_in_group ? nkeys : rows_in_group;
  p.max_units           = int(present + rows_in_group / rbk_unit_cap(nrows) + 1);
  const int64_t heavy   = rows_in_group / rbk_unit_cap(nrows) + 1;  // keys with more than a unit's rows in a group
  p.max_fold            = int(int64_t(p.n_groups) * (heavy < nkeys ? heavy : nkeys));
  const size_t per_key  = size_t(nkeys + 1) * sizeof(int);
  const size_t per_unit = size_t(p.n_groups) * p.max_units * sizeof(int);
  size_t o              = 0;
  p.off_perm            = o;
  o += align_up(size_t(nrows) * sizeof(unsigned), 256);
  p.off_offs = o;
  o += align_up(size_t(p.n_windows) * per_key, 256);
  p.off_gcnt = o;
  o += align_up(size_t(p.n_groups) * nkeys * sizeof(int), 256);
  p.off_uoffs = o;
  o += align_up(size_t(p.n_groups) * per_key, 256);
  p.off_ukey = o;
  o += align_up(per_unit, 256);
  p.off_ufirst = o;
  o += align_up(per_unit, 256);
  p.off_ulen = o;
  o += align_up(per_unit, 256);
  p.off_fold = o;
  o += align_up(size_t(p.max_fold) * sizeof(int), 256);
  p.off_counter = o;
  o += 256;
  p.off_part = o;
  o += align_up(size_t(p.n_groups) * p.max_units * size_t(ncols) * carry_size, 256);
  p.total = o;
  return p;
}

// The unit queue is a 32-bit counter and offsets inside a group are 32-bit: 2^30 rows at most.
inline bool rows_by_key_sorted_supported(int64_t nrows, int64_t ncols, int64_t nkeys)
{
  return nkeys <= kMaxSortKeys && ncols <= int64_t(0x7fffffff) && nrows > 0 && nrows <= (int64_t(1) << 30);
}

template <typename DataT, typename KeyT, typename WeightT, typename SumT>
cudaError_t launch_rows_by_key_sorted(SumT* sums,
                                      long long* counts,
                                      const DataT* A,
                                      int64_t lda,
                                      const KeyT* keys,
                                      const WeightT* weights,
                                      int64_t nrows,
                                      int64_t ncols,
                                      int64_t nkeys,
                                      bool reset,
                                      cudaStream_t stream,
                                      Workspace ws)
{
  constexpr int V16  = vec16<DataT>::value;
  using CarryT       = typename sum_state<SumT>::type::carry_t;
  const SortedPlan p = plan_rows_by_key_sorted<DataT>(A, lda, nrows, ncols, nkeys, sizeof(CarryT));
  Scratch scratch(ws, p.total, stream);
  if (scratch.error() != cudaSuccess) return scratch.error();
  unsigned char* base = static_cast<unsigned char*>(scratch.get());
  unsigned* perm      = reinterpret_cast<unsigned*>(base + p.off_perm);
  int* offs           = reinterpret_cast<int*>(base + p.off_offs);
  int* gcnt           = reinterpret_cast<int*>(base + p.off_gcnt);
  int* uoffs          = reinterpret_cast<int*>(base + p.off_uoffs);
  int* ukey           = reinterpret_cast<int*>(base + p.off_ukey);
  int* ufirst         = reinterpret_cast<int*>(base + p.off_ufirst);
  int* ulen           = reinterpret_cast<int*>(base + p.off_ulen);
  int* fold_list      = reinterpret_cast<int*>(base + p.off_fold);
  int* counter        = reinterpret_cast<int*>(base + p.off_counter);  // [0] unit queue, [1] fold list length
  CarryT* partial     = reinterpret_cast<CarryT*>(base + p.off_part);
  const int nk        = int(nkeys);
  const int sms       = sm_count();
  cudaError_t e;

  // 1. per-window counting sort
  const size_t smem_cap  = (size_t(227) << 10) - 256;  // most a CTA may opt into, less the static part
  const bool staged      = rbk_sort_smem(nkeys, p.window_rows, true) <= smem_cap;
  const size_t sort_smem = rbk_sort_smem(nkeys, p.window_rows, staged);
  auto sort_kern         = staged ? rbk_sort_kernel<KeyT, true> : rbk_sort_kernel<KeyT, false>;
  if (sort_smem + 1024 > (size_t(48) << 10)) {  // static shared memory counts against the 48 KB too
    e = ensure_dynamic_smem(sort_kern, size_t(sort_smem));
    if (e != cudaSuccess) return e;
  }
  e = launch_dep(sort_kern, dim3(unsigned(p.n_windows)), dim3(kSortTpb), sort_smem, stream, keys, nrows, nk,
                 p.window_rows, perm, offs, counter);
  if (e != cudaSuccess) return e;

  // 2. rows per (group, key), unit tables and the list of keys to fold
  e = launch_dep(rbk_units_kernel<1024>, dim3(unsigned(p.n_groups)), dim3(1024), 0, stream, offs, p.n_windows, p.group,
                 gcnt, nk, p.max_units, rbk_unit_cap(nrows), uoffs, ukey, ufirst, ulen, fold_list, counter + 1);
  if (e != cudaSuccess) return e;

  // 4. stream the matrix, one warp per (unit, part of the columns)
  const int nvec      = int(ncols / p.vec);
  const unsigned g    = next_pow2(unsigned(nvec > 0 ? nvec : 1));
  const int G         = int(g > 32u ? 32u : g);
  const int64_t slots = int64_t(p.n_groups) * p.max_units;
  const int passes    = (nvec + G - 1) / G;
#define B2R_LAUNCH_STREAM(VEC_)                                                                              \
  do {                                                                                                       \
    auto kern      = rbk_stream_kernel<DataT, WeightT, SumT, VEC_>;                                          \
    static int occ = resident_ctas(kern, 256, 0);                                                            \
    int64_t ctas   = int64_t(sms) * occ;                                                                     \
    /* about four items per resident warp: cut the columns when the rows alone give fewer */                \
    const int64_t est_units = ceil_div<int64_t>(nrows, rbk_unit_target(nrows));                                        \
    int64_t split           = ceil_div<int64_t>(ctas * 8 * 4, est_units);                                    \
    if (split > passes) split = passes;                                                                      \
    while (split > 1 && slots * split >= (int64_t(1) << 30))                                                 \
      --split;                                                                                               \
    if (split < 1) split = 1;                                                                                \
    if (ctas > ceil_div<int64_t>(slots * split, 8)) ctas = ceil_div<int64_t>(slots * split, 8);              \
    (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(256), 0, stream, partial, A, lda, weights, int(ncols), \
                     nk, p.window_rows, p.n_windows, p.group, p.n_groups, p.max_units, G, int(split), perm,  \
                     offs, uoffs, ukey, ufirst, ulen, counter);                                              \
  } while (0)
  if (p.vec > 1) {
    B2R_LAUNCH_STREAM(V16);
  } else {
    B2R_LAUNCH_STREAM(1);
  }
#undef B2R_LAUNCH_STREAM
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  // 5. one partial row per (group, key); 6. fold the groups of every key
  int64_t fold_ctas = ceil_div<int64_t>(p.max_fold, 8);
  if (fold_ctas > int64_t(sms) * 8) fold_ctas = int64_t(sms) * 8;
  if (fold_ctas < 1) fold_ctas = 1;
  (void)launch_dep(rbk_fold_kernel<SumT>, dim3(unsigned(fold_ctas)), dim3(256), 0, stream, partial, uoffs, fold_list,
                   counter + 1, p.max_units, int(ncols), nk);
  if (nkeys <= 2048) {  // few keys: a CTA per key
    (void)launch_dep(rbk_merge_kernel<SumT, 8>, dim3(unsigned(nkeys)), dim3(256), 0, stream, sums, counts, partial,
                     gcnt, uoffs, p.n_groups, p.max_units, int(ncols), nk, reset);
  } else {
    (void)launch_dep(rbk_merge_kernel<SumT, 1>, dim3(unsigned(ceil_div<int64_t>(nkeys, 8))), dim3(256), 0, stream, sums,
                     counts, partial, gcnt, uoffs, p.n_groups, p.max_units, int(ncols), nk, reset);
  }
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
