// Keyed row sums, "sort then stream" formulation:
//     sums[keys[i]][:] += w[i] * A[i][:]
//
// Three kernels, no floating-point atomics, every matrix row read from HBM exactly once:
//
//  rbk_sort_kernel     one CTA per window of W consecutive rows. Counting sort of the window's
//                      row indices by key in shared memory (integer atomics only): writes
//                        perm[window][.]        row offsets inside the window, grouped by key
//                        unit tables            the grouped list cut into work units of at most
//                                               kUnitRows rows that all carry one key
//  rbk_stream_kernel   one warp per work unit, persistent grid: the warp streams the unit's
//                      rows (a sub-warp of G lanes per row, 8 row loads in flight per lane),
//                      keeps a compensated sum per column in REGISTERS, and writes one partial
//                      row per unit. Nothing is shared between warps, so occupancy - and with
//                      it the bytes in flight - is not limited by an accumulator table, long
//                      runs of one key are spread over many warps (skew-proof), and a handful
//                      of keys is as fast as thousands.
//  rbk_merge_kernel    per (key, column): folds the partial rows of the key's units over all
//                      windows in a fixed order (compensated), adds to or overwrites sums, and
//                      derives the exact int64 row counts from the sort's offsets.
//
// Extra memory traffic over the matrix itself: the keys are read twice, the 4-byte permutation
// is written and read once, and one partial row per unit is written and read - about 3 % for
// 128 fp32 columns.
#pragma once

#include "common.cuh"
#include "launch.cuh"
#include "ops.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kUnitRows   = 256;    // rows per work unit (one key each)
constexpr int kSortTpb    = 1024;
constexpr int kMaxSortKeys = 49152;  // histogram + cursors must fit shared memory

struct SortedPlan {
  int vec;
  int window_rows;   // W
  int n_windows;
  int max_units;     // per window
  size_t off_perm, off_offs, off_uoffs, off_ukey, off_ubeg, off_ulen, off_part, total;
};

// Work-unit tables of one window (global memory):
//   offs [nkeys + 1]  first sorted position of each key          (exclusive prefix of counts)
//   uoffs[nkeys + 1]  first unit of each key                     (exclusive prefix of unit counts)
//   ukey/ubeg/ulen[max_units]  key, first sorted position and row count of each unit
// STAGED: the window's permutation is built in shared memory as 16-bit offsets (W <= 65536) and
// written out with coalesced stores; otherwise every row's slot is stored straight to global
// memory (32 sectors per warp store).
template <typename KeyT, bool STAGED>
__global__ void __launch_bounds__(kSortTpb) rbk_sort_kernel(const KeyT* __restrict__ keys,
                                                           int64_t nrows,
                                                           int nkeys,
                                                           int W,
                                                           int max_units,
                                                           unsigned* __restrict__ perm,
                                                           int* __restrict__ offs,
                                                           int* __restrict__ uoffs,
                                                           int* __restrict__ ukey,
                                                           int* __restrict__ ubeg,
                                                           int* __restrict__ ulen)
{
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* s_cnt   = reinterpret_cast<int*>(smem_raw);  // [nkeys] counts, then cursors
  int* s_cur   = s_cnt + nkeys;                     // [nkeys] scatter cursors
  unsigned short* s_perm = reinterpret_cast<unsigned short*>(s_cur + nkeys);  // [W] when STAGED
  __shared__ int s_warp[2][kSortTpb / 32];

  const int win        = blockIdx.x;
  const int64_t row0   = int64_t(win) * W;
  int64_t n            = nrows - row0;
  n                    = n < W ? n : W;
  const int tid        = threadIdx.x;
  const int lane       = tid & 31;
  const int warp       = tid >> 5;
  const KeyT* wkeys    = keys + row0;
  unsigned* wperm      = perm + row0;
  int* w_offs          = offs + size_t(win) * (nkeys + 1);
  int* w_uoffs         = uoffs + size_t(win) * (nkeys + 1);
  int* w_ukey          = ukey + size_t(win) * max_units;
  int* w_ubeg          = ubeg + size_t(win) * max_units;
  int* w_ulen          = ulen + size_t(win) * max_units;

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
    }
#pragma unroll
    for (int j = 0; j < KU; ++j)
      if (kk[j] >= 0) atomicAdd(&s_cnt[kk[j]], 1);
  }
  __syncthreads();

  // exclusive scans of the counts and of the per-key unit counts, both over [0, nkeys)
  const int per = (nkeys + kSortTpb - 1) / kSortTpb;
  const int b0  = tid * per;
  int loc_c = 0, loc_u = 0;
  for (int i = 0; i < per; ++i) {
    if (b0 + i < nkeys) {
      const int c = s_cnt[b0 + i];
      loc_c += c;
      loc_u += (c + kUnitRows - 1) / kUnitRows;
    }
  }
  int inc_c = loc_c, inc_u = loc_u;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, inc_c, off);
    const int b = __shfl_up_sync(0xffffffffu, inc_u, off);
    if (lane >= off) {
      inc_c += a;
      inc_u += b;
    }
  }
  if (lane == 31) {
    s_warp[0][warp] = inc_c;
    s_warp[1][warp] = inc_u;
  }
  __syncthreads();
  int base_c = 0, base_u = 0;
  for (int w = 0; w < warp; ++w) {
    base_c += s_warp[0][w];
    base_u += s_warp[1][w];
  }
  int run_c = base_c + inc_c - loc_c;
  int run_u = base_u + inc_u - loc_u;
  for (int i = 0; i < per; ++i) {
    const int k = b0 + i;
    if (k < nkeys) {
      const int c  = s_cnt[k];
      const int nu = (c + kUnitRows - 1) / kUnitRows;
      w_offs[k]    = run_c;
      w_uoffs[k]   = run_u;
      for (int u = 0; u < nu; ++u) {
        w_ukey[run_u + u] = k;
        w_ubeg[run_u + u] = run_c + u * kUnitRows;
        w_ulen[run_u + u] = (c - u * kUnitRows) < kUnitRows ? (c - u * kUnitRows) : kUnitRows;
      }
      s_cur[k]     = run_c;
      run_c += c;
      run_u += nu;
    }
  }
  if (tid == kSortTpb - 1) {
    w_offs[nkeys]  = run_c;
    w_uoffs[nkeys] = run_u;
  }
  __syncthreads();
  for (int64_t i0 = 0; i0 < n; i0 += int64_t(KU) * kSortTpb) {
    int kk[KU];
#pragma unroll
    for (int j = 0; j < KU; ++j) {
      const int64_t i = i0 + int64_t(j) * kSortTpb + tid;
      kk[j]           = i < n ? static_cast<int>(wkeys[i]) : -1;
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

template <typename DataT, typename WeightT, typename SumT, int VEC>
__global__ void __launch_bounds__(256) rbk_stream_kernel(typename sum_state<SumT>::type::carry_t* __restrict__ partial,
                                                        const DataT* __restrict__ A,
                                                        int64_t lda,
                                                        const WeightT* __restrict__ weights,
                                                        int64_t nrows,
                                                        int ncols,
                                                        int nkeys,
                                                        int W,
                                                        int n_windows,
                                                        int max_units,
                                                        int G,
                                                        const unsigned* __restrict__ perm,
                                                        const int* __restrict__ uoffs,
                                                        const int* __restrict__ ubeg,
                                                        const int* __restrict__ ulen)
{
  using State     = typename sum_state<SumT>::type;
  using CarryT    = typename State::carry_t;
  constexpr int Q = 8;
  const op::Add add{};
  const int lane  = threadIdx.x & 31;
  const int lig   = lane & (G - 1);
  const int grp   = lane / G;
  const int gpw   = 32 / G;
  const int nvec  = ncols / VEC;
  const int64_t total_slots = int64_t(n_windows) * max_units;
  const int64_t warps       = int64_t(gridDim.x) * 8;
  for (int64_t slot = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5); slot < total_slots; slot += warps) {
    const int win = int(slot / max_units);
    const int u   = int(slot - int64_t(win) * max_units);
    if (u >= uoffs[size_t(win) * (nkeys + 1) + nkeys]) continue;  // this window has fewer units
    const int beg         = ubeg[slot];
    const int len         = ulen[slot];
    const int64_t row0    = int64_t(win) * W;
    const unsigned* uperm = perm + row0 + beg;
    CarryT* dst           = partial + size_t(slot) * ncols;
    for (int cv0 = 0; cv0 < nvec; cv0 += G) {
      const int cv      = cv0 + lig;
      const bool col_ok = cv < nvec;
      State acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        acc[e].init(SumT(0));
      for (int i0 = 0; i0 < len; i0 += Q * gpw) {
        VecOf<DataT, VEC> v[Q];
        SumT w[Q];
#pragma unroll
        for (int k = 0; k < Q; ++k) {
          int i           = i0 + k * gpw + grp;
          i               = i < len ? i : len - 1;  // duplicate, masked below
          const int64_t r = row0 + uperm[i];
          v[k]            = load_stream<DataT, VEC>(A + r * lda + int64_t(col_ok ? cv : 0) * VEC);
          w[k]            = weights != nullptr ? SumT(weights[r]) : SumT(1);
        }
#pragma unroll
        for (int k = 0; k < Q; ++k) {
          if (i0 + k * gpw + grp < len) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              SumT x = SumT(v[k].e[e]);
              if (weights != nullptr) x *= w[k];
              acc[e].push(x, add);
            }
          }
        }
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

// One CTA per key: warp j folds the key's partial rows of windows j, j+8, ... (lanes over the
// columns, unit rows loaded four at a time), then the eight warps are folded in order through
// shared memory. Also derives the key's row count from the sort offsets.
template <typename SumT>
__global__ void __launch_bounds__(256) rbk_merge_kernel(SumT* __restrict__ sums,
                                                       long long* __restrict__ counts,
                                                       const typename sum_state<SumT>::type::carry_t* __restrict__ partial,
                                                       const int* __restrict__ offs,
                                                       const int* __restrict__ uoffs,
                                                       int n_windows,
                                                       int max_units,
                                                       int ncols,
                                                       int nkeys,
                                                       bool reset)
{
  using State  = typename sum_state<SumT>::type;
  using CarryT = typename State::carry_t;
  const op::Add add{};
  extern __shared__ __align__(16) unsigned char smem_raw[];
  State* s_acc     = reinterpret_cast<State*>(smem_raw);            // [8][chunk]
  int2* s_rng      = reinterpret_cast<int2*>(s_acc + 8 * 128);      // [n_windows] unit range of key k
  __shared__ long long s_n[8];
  const int k      = blockIdx.x;
  const int lane   = threadIdx.x & 31;
  const int warp   = threadIdx.x >> 5;
  constexpr int CH = 128;  // columns per pass: 4 per lane

  long long n_rows_k = 0;
  for (int w = warp * 32 + lane; w < n_windows; w += 256) {
    const int* wo = offs + size_t(w) * (nkeys + 1);
    const int* wu = uoffs + size_t(w) * (nkeys + 1);
    n_rows_k += wo[k + 1] - wo[k];
    s_rng[w] = make_int2(wu[k], wu[k + 1]);
  }
  __syncthreads();
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    n_rows_k += __shfl_xor_sync(0xffffffffu, n_rows_k, off);
  if (lane == 0) s_n[warp] = n_rows_k;

  for (int c0 = 0; c0 < ncols; c0 += CH) {
    State acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      acc[e].init(SumT(0));
    // four windows per step: the first unit row of each (most keys have one or two units per
    // window) is loaded before any of them is consumed, so four loads per lane are in flight
    for (int w0 = warp; w0 < n_windows; w0 += 32) {
      int2 rng[4];
      CarryT first[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int w = w0 + 8 * j;
        rng[j]      = w < n_windows ? s_rng[w] : make_int2(0, 0);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = c0 + e * 32 + lane;
          first[j][e] = (rng[j].y > rng[j].x && c < ncols)
                          ? partial[(size_t(w) * max_units + rng[j].x) * ncols + c]
                          : CarryT(0);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          acc[e].push_carry(first[j][e], add);
        const CarryT* wpart = partial + size_t(w0 + 8 * j) * max_units * ncols;
        for (int u = rng[j].x + 1; u < rng[j].y; ++u) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c0 + e * 32 + lane;
            if (c < ncols) acc[e].push_carry(wpart[size_t(u) * ncols + c], add);
          }
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      s_acc[warp * CH + e * 32 + lane] = acc[e];
    __syncthreads();
    if (threadIdx.x < CH) {
      const int c = c0 + threadIdx.x;
      if (c < ncols) {
        State t;
        t.init(reset ? SumT(0) : sums[size_t(k) * ncols + c]);
        for (int j = 0; j < 8; ++j)
          t.merge(s_acc[j * CH + threadIdx.x], add);
        sums[size_t(k) * ncols + c] = t.value();
      }
    }
    __syncthreads();
  }
  if (counts != nullptr && threadIdx.x == 0) {
    long long n = reset ? 0ll : counts[k];
    for (int j = 0; j < 8; ++j)
      n += s_n[j];
    counts[k] = n;
  }
}

template <typename DataT>
inline SortedPlan plan_rows_by_key_sorted(const DataT* A, int64_t lda, int64_t nrows, int64_t ncols, int64_t nkeys,
                                          size_t sum_size)
{
  constexpr int V16 = vec16<DataT>::value;
  SortedPlan p      = {};
  const bool vec_ok = V16 > 1 && ncols % V16 == 0 && lda % V16 == 0 && aligned16(A);
  p.vec             = vec_ok ? V16 : 1;
  // windows: about two per SM, between 16 Ki and 128 Ki rows
  int64_t W = int64_t(next_pow2(unsigned(ceil_div<int64_t>(nrows, int64_t(sm_count()) * 2))));
  const int knob = tuning().key_window_rows;
  if (knob > 0 && (knob & (knob - 1)) == 0) W = knob;
  if (W < 16384) W = 16384;
  if (W > 131072) W = 131072;
  p.window_rows = int(W);
  p.n_windows   = int(ceil_div<int64_t>(nrows, W));
  const int64_t rows_in_win = nrows < W ? nrows : W;
  int64_t mu    = nkeys + rows_in_win / kUnitRows;  // every key may have one ragged unit
  if (mu > rows_in_win) mu = rows_in_win;           // a unit holds at least one row
  if (mu < 1) mu = 1;
  p.max_units   = int(mu);
  size_t o      = 0;
  p.off_perm    = o;
  o += align_up(size_t(nrows) * sizeof(unsigned), 256);
  p.off_offs = o;
  o += align_up(size_t(p.n_windows) * (nkeys + 1) * sizeof(int), 256);
  p.off_uoffs = o;
  o += align_up(size_t(p.n_windows) * (nkeys + 1) * sizeof(int), 256);
  p.off_ukey = o;
  o += align_up(size_t(p.n_windows) * p.max_units * sizeof(int), 256);
  p.off_ubeg = o;
  o += align_up(size_t(p.n_windows) * p.max_units * sizeof(int), 256);
  p.off_ulen = o;
  o += align_up(size_t(p.n_windows) * p.max_units * sizeof(int), 256);
  p.off_part = o;
  o += align_up(size_t(p.n_windows) * p.max_units * size_t(ncols) * sum_size, 256);
  p.total = o;
  return p;
}

inline bool rows_by_key_sorted_supported(int64_t nrows, int64_t ncols, int64_t nkeys)
{
  return nkeys <= kMaxSortKeys && ncols <= int64_t(0x7fffffff) && nrows > 0;
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
  int* uoffs          = reinterpret_cast<int*>(base + p.off_uoffs);
  int* ukey           = reinterpret_cast<int*>(base + p.off_ukey);
  int* ubeg           = reinterpret_cast<int*>(base + p.off_ubeg);
  int* ulen           = reinterpret_cast<int*>(base + p.off_ulen);
  CarryT* partial     = reinterpret_cast<CarryT*>(base + p.off_part);
  cudaError_t e;

  const size_t hist_smem   = size_t(nkeys) * 2 * sizeof(int);
  const size_t staged_smem = hist_smem + size_t(p.window_rows) * sizeof(unsigned short);
  const bool staged        = p.window_rows <= 65536 && staged_smem <= (size_t(220) << 10);
  const size_t sort_smem   = staged ? staged_smem : hist_smem;
  auto sort_kern           = staged ? rbk_sort_kernel<KeyT, true> : rbk_sort_kernel<KeyT, false>;
  if (sort_smem + 1024 > (size_t(48) << 10)) {  // static shared memory counts against the 48 KB too
    e = cudaFuncSetAttribute(sort_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sort_smem));
    if (e != cudaSuccess) return e;
  }
  sort_kern<<<unsigned(p.n_windows), kSortTpb, sort_smem, stream>>>(
    keys, nrows, int(nkeys), p.window_rows, p.max_units, perm, offs, uoffs, ukey, ubeg, ulen);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  const int nvec           = int(ncols / p.vec);
  unsigned g               = next_pow2(unsigned(nvec > 0 ? nvec : 1));
  const int G              = int(g > 32u ? 32u : g);
  const int64_t slots      = int64_t(p.n_windows) * p.max_units;
  const int sms            = sm_count();
#define B2R_LAUNCH_STREAM(VEC_)                                                                        \
  do {                                                                                                 \
    auto kern      = rbk_stream_kernel<DataT, WeightT, SumT, VEC_>;                                    \
    static int occ = resident_ctas(kern, 256, 0);                                                      \
    int64_t ctas   = int64_t(sms) * occ;                                                               \
    if (ctas > ceil_div<int64_t>(slots, 8)) ctas = ceil_div<int64_t>(slots, 8);                        \
    kern<<<unsigned(ctas), 256, 0, stream>>>(partial, A, lda, weights, nrows, int(ncols), int(nkeys),  \
                                             p.window_rows, p.n_windows, p.max_units, G, perm, uoffs,  \
                                             ubeg, ulen);                                              \
  } while (0)
  if (p.vec > 1) {
    B2R_LAUNCH_STREAM(V16);
  } else {
    B2R_LAUNCH_STREAM(1);
  }
#undef B2R_LAUNCH_STREAM
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  const size_t merge_smem =
    size_t(8) * 128 * sizeof(typename sum_state<SumT>::type) + size_t(p.n_windows) * sizeof(int2);
  if (merge_smem + 1024 > (size_t(48) << 10)) {
    e = cudaFuncSetAttribute(rbk_merge_kernel<SumT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(merge_smem));
    if (e != cudaSuccess) return e;
  }
  rbk_merge_kernel<SumT><<<unsigned(nkeys), 256, merge_smem, stream>>>(
    sums, counts, partial, offs, uoffs, p.n_windows, p.max_units, int(ncols), int(nkeys), reset);
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
