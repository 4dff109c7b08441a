// Keyed row sums:  sums[keys[i]][:] += w[i] * A[i][:]   (k-means centroid accumulation).
//
// The reference issues one global atomicAdd per matrix element
// (linalg/detail/reduce_rows_by_key.cuh:279-300, launcher :302-326), so it is bound by
// atomic throughput on an L2-resident table and its result depends on scheduling.
// Here every matrix row is read from HBM once, with 16-byte loads, and no atomic touches a
// floating-point value:
//
//  rows_by_key_partial_kernel   grid (key slices S, row groups R), one CTA per SM.
//     A CTA owns the accumulator rows of one slice of the key space in shared memory
//     (compensated sums, kept for the whole row group) and walks its row group in blocks
//     of B rows:
//       1. the keys of the block are counting-sorted by key in shared memory (integer
//          shared-memory atomics give each row its rank inside its key);
//       2. warps pull work items dynamically. An item is the sorted entries of a few
//          consecutive keys (about 32 rows): the warp streams these rows with 8 row loads
//          in flight per lane, sums each key's rows in registers with a compensated sum,
//          and merges the result into the key's accumulator row ONCE per key - so
//          shared-memory traffic is a fraction of a byte per matrix byte and no two warps
//          ever touch the same accumulator.
//       When the whole table is small enough to give every warp a private copy, an item
//       is instead a fixed-size piece of the sorted list (it may cut a key's run), which
//       keeps the warps balanced when there are only a handful of keys.
//     Rows whose key falls outside the CTA's slice are skipped, so across the S CTAs of a
//     row group every row is loaded exactly once. At the end the slice is written to
//     partial[row group][key][col] together with the exact per-key row counts.
//  rows_by_key_merge_kernel     folds the R partial tables in a fixed order (compensated),
//     adds to or overwrites sums, and accumulates the int64 counts.
#pragma once

#include "common.cuh"
#include "launch.cuh"
#include "ops.cuh"
#include "rows_by_key_small.cuh"
#include "rows_by_key_sorted.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kKeyTpb       = 512;  // 16 warps
constexpr int kKeyMaxPerThr = 16;   // keys staged per thread per block -> B <= 8192
constexpr int kKeyChunk     = 16;   // sorted entries per work item in private mode

struct RowsByKeyPlan {
  int vec;
  int kps;           // keys per slice
  int n_slices;      // S
  int n_groups;      // R
  int block_rows;    // B
  int repl;          // 1 or number of warps
  int64_t rows_per_group;
  size_t smem;
  size_t scratch_sums;    // bytes
  size_t scratch_counts;  // bytes
};

template <typename SumT>
struct RowsByKeySmem {
  // byte offsets inside dynamic shared memory
  size_t table, cnt, hist, offs, sorted, misc, total;
};

template <typename SumT>
inline RowsByKeySmem<SumT> rows_by_key_smem(int kps, int ncols, int repl, int B)
{
  using State = CompensatedState<SumT>;
  RowsByKeySmem<SumT> s;
  size_t o = 0;
  s.table  = o;
  o += align_up(size_t(repl) * kps * ncols * sizeof(State), 16);
  s.cnt = o;
  o += align_up(size_t(kps) * sizeof(unsigned long long), 16);
  s.hist = o;
  o += align_up(size_t(kps) * sizeof(int), 16);
  s.offs = o;
  o += align_up(size_t(kps + 1) * sizeof(int), 16);
  s.sorted = o;
  o += align_up(size_t(B) * sizeof(unsigned short), 16);
  s.misc = o;
  o += 64 * sizeof(int);
  s.total = o;
  return s;
}

template <typename DataT, typename KeyT, typename WeightT, typename SumT, int VEC>
__global__ void __launch_bounds__(kKeyTpb, 1)
  rows_by_key_partial_kernel(SumT* __restrict__ partial_sums,
                             unsigned long long* __restrict__ partial_counts,
                             const DataT* __restrict__ A,
                             int64_t lda,
                             const KeyT* __restrict__ keys,
                             const WeightT* __restrict__ weights,
                             int64_t nrows,
                             int ncols,
                             int nkeys,
                             int kps,
                             int64_t rows_per_group,
                             int B,
                             int repl,
                             RowsByKeySmem<SumT> lay)
{
  using State      = CompensatedState<SumT>;
  constexpr int Q  = 8;  // row loads in flight per lane
  extern __shared__ __align__(16) unsigned char smem_raw[];
  State* table              = reinterpret_cast<State*>(smem_raw + lay.table);
  unsigned long long* s_cnt = reinterpret_cast<unsigned long long*>(smem_raw + lay.cnt);
  int* s_hist               = reinterpret_cast<int*>(smem_raw + lay.hist);
  int* s_offs               = reinterpret_cast<int*>(smem_raw + lay.offs);
  unsigned short* s_sorted  = reinterpret_cast<unsigned short*>(smem_raw + lay.sorted);
  int* s_misc               = reinterpret_cast<int*>(smem_raw + lay.misc);  // [0] next item, [1] total, [2..2+NW] scan

  const int tid  = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const op::Add add{};

  const int slice      = blockIdx.x;
  const int key_base   = slice * kps;
  int my_keys          = nkeys - key_base;
  my_keys              = my_keys < kps ? my_keys : kps;
  const int64_t g_row0 = int64_t(blockIdx.y) * rows_per_group;
  int64_t g_row1       = g_row0 + rows_per_group;
  g_row1               = g_row1 < nrows ? g_row1 : nrows;
  const int nvec       = ncols / VEC;  // VEC divides ncols on the vector path

  for (int i = tid; i < repl * kps * ncols; i += kKeyTpb)
    table[i].init(SumT(0));
  for (int i = tid; i < kps; i += kKeyTpb) {
    s_cnt[i]  = 0ull;
    s_hist[i] = 0;
  }
  __syncthreads();

  // keys of the first block, held in registers (-1: row absent or key not in this slice)
  int lk[kKeyMaxPerThr];
  auto fetch_keys = [&](int64_t row0, int (&dst)[kKeyMaxPerThr]) {
#pragma unroll
    for (int i = 0; i < kKeyMaxPerThr; ++i) {
      const int j     = i * kKeyTpb + tid;
      const int64_t r = row0 + j;
      int v           = -1;
      if (j < B && r < g_row1) {
        const long long k = static_cast<long long>(keys[r]) - key_base;
        if (k >= 0 && k < my_keys) v = int(k);
      }
      dst[i] = v;
    }
  };
  if (g_row0 < g_row1) fetch_keys(g_row0, lk);

  for (int64_t row0 = g_row0; row0 < g_row1; row0 += B) {
    // ---- 1. counting sort of this block's rows by key ------------------------------
    int rank[kKeyMaxPerThr];
#pragma unroll
    for (int i = 0; i < kKeyMaxPerThr; ++i)
      rank[i] = lk[i] >= 0 ? atomicAdd(&s_hist[lk[i]], 1) : 0;
    __syncthreads();
    // exclusive scan of s_hist[0..my_keys) -> s_offs, total -> s_misc[1]
    {
      const int per = (my_keys + kKeyTpb - 1) / kKeyTpb;
      const int b0  = tid * per;
      int local     = 0;
      for (int i = 0; i < per; ++i)
        if (b0 + i < my_keys) local += s_hist[b0 + i];
      int incl = local;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
      }
      if (lane == 31) s_misc[2 + warp] = incl;
      __syncthreads();
      int warp_base = 0;
      for (int w = 0; w < warp; ++w)
        warp_base += s_misc[2 + w];
      int run = warp_base + incl - local;
      for (int i = 0; i < per; ++i) {
        if (b0 + i < my_keys) {
          s_offs[b0 + i] = run;
          run += s_hist[b0 + i];
        }
      }
      if (tid == kKeyTpb - 1) {
        s_offs[my_keys] = run;
        s_misc[1]       = run;
        s_misc[0]       = 0;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kKeyMaxPerThr; ++i)
      if (lk[i] >= 0) s_sorted[s_offs[lk[i]] + rank[i]] = static_cast<unsigned short>(i * kKeyTpb + tid);
    // prefetch the next block's keys while this block's rows are summed
    if (row0 + B < g_row1) fetch_keys(row0 + B, lk);
    __syncthreads();

    // ---- 2. dynamic work items ---------------------------------------------------------
    // An item is a range [p_beg, p_end) of the sorted list. With one shared table the
    // range is the entries of `kg` consecutive keys (so a key is never split between
    // warps); with private tables it is a fixed-size piece.
    const int total = s_misc[1];
    int kg          = 1;
    if (total > 0) {
      kg = (kKeyChunk * my_keys + total - 1) / total;
      kg = kg < 1 ? 1 : kg;
    }
    const int n_items = repl == 1 ? (my_keys + kg - 1) / kg : (total + kKeyChunk - 1) / kKeyChunk;
    State* my_table   = table + (repl == 1 ? size_t(0) : size_t(warp) * kps * ncols);
    while (total > 0) {
      int item = 0;
      if (lane == 0) item = atomicAdd(&s_misc[0], 1);
      item = __shfl_sync(0xffffffffu, item, 0);
      if (item >= n_items) break;
      int p_beg, p_end, key0;
      if (repl == 1) {
        key0         = item * kg;
        int key_last = key0 + kg;
        key_last     = key_last < my_keys ? key_last : my_keys;
        p_beg        = s_offs[key0];
        p_end        = s_offs[key_last];
      } else {
        p_beg = item * kKeyChunk;
        p_end = p_beg + kKeyChunk < total ? p_beg + kKeyChunk : total;
        int lo = 0, hi = my_keys - 1;  // last key whose first entry is <= p_beg
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (s_offs[mid] <= p_beg) {
            lo = mid;
          } else {
            hi = mid - 1;
          }
        }
        key0 = lo;
      }
      if (p_beg >= p_end) continue;
      for (int cv = lane; cv < nvec; cv += 32) {
        State acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          acc[e].init(SumT(0));
        int key = key0;
        while (s_offs[key + 1] <= p_beg)
          ++key;
        int next_bound = s_offs[key + 1];
        auto flush     = [&](int k) {
          State* dst = my_table + size_t(k) * ncols + size_t(cv) * VEC;
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            State t = dst[e];
            t.merge(acc[e], add);
            dst[e] = t;
            acc[e].init(SumT(0));
          }
        };
        for (int i0 = p_beg; i0 < p_end; i0 += Q) {
          VecOf<DataT, VEC> v[Q];
          SumT w[Q];
#pragma unroll
          for (int k = 0; k < Q; ++k) {
            const int i     = i0 + k < p_end ? i0 + k : p_end - 1;  // duplicate, masked below
            const int64_t r = row0 + s_sorted[i];
            v[k]            = load_stream<DataT, VEC>(A + r * lda + int64_t(cv) * VEC);
            w[k]            = weights != nullptr ? SumT(weights[r]) : SumT(1);
          }
#pragma unroll
          for (int k = 0; k < Q; ++k) {
            if (i0 + k < p_end) {
              if (i0 + k >= next_bound) {  // uniform across the warp
                flush(key);
                do {
                  ++key;
                } while (s_offs[key + 1] <= i0 + k);
                next_bound = s_offs[key + 1];
              }
#pragma unroll
              for (int e = 0; e < VEC; ++e) {
                SumT x = SumT(v[k].e[e]);
                if (weights != nullptr) x *= w[k];
                acc[e].push(x, add);
              }
            }
          }
        }
        flush(key);
      }
    }
    __syncthreads();
    for (int i = tid; i < my_keys; i += kKeyTpb) {
      s_cnt[i] += static_cast<unsigned long long>(s_hist[i]);
      s_hist[i] = 0;
    }
    __syncthreads();
  }

  // ---- write this slice of the row group's partial table ---------------------------------
  SumT* dst_sums = partial_sums + (size_t(blockIdx.y) * nkeys + key_base) * ncols;
  for (int i = tid; i < my_keys * ncols; i += kKeyTpb) {
    State t = table[i];
    for (int r = 1; r < repl; ++r)
      t.merge(table[size_t(r) * kps * ncols + i], add);
    dst_sums[i] = t.value();
  }
  if (partial_counts != nullptr) {
    for (int i = tid; i < my_keys; i += kKeyTpb)
      partial_counts[size_t(blockIdx.y) * nkeys + key_base + i] = s_cnt[i];
  }
}

template <typename SumT>
__global__ void __launch_bounds__(256) rows_by_key_merge_kernel(SumT* __restrict__ sums,
                                                               long long* __restrict__ counts,
                                                               const SumT* __restrict__ partial_sums,
                                                               const unsigned long long* __restrict__ partial_counts,
                                                               int n_groups,
                                                               int64_t table_elems,
                                                               int nkeys,
                                                               bool reset)
{
  const op::Add add{};
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < table_elems) {
    CompensatedState<SumT> st;
    st.init(reset ? SumT(0) : sums[i]);
    for (int g = 0; g < n_groups; ++g)
      st.push(partial_sums[size_t(g) * table_elems + i], add);
    sums[i] = st.value();
  }
  if (counts != nullptr && i < nkeys) {
    long long c = reset ? 0ll : counts[i];
    for (int g = 0; g < n_groups; ++g)
      c += static_cast<long long>(partial_counts[size_t(g) * nkeys + i]);
    counts[i] = c;
  }
}

// Fallback for tables whose single key row does not fit in shared memory (hundreds of
// thousands of columns): one 16-byte load per thread and global atomics, as the reference.
template <typename DataT, typename KeyT, typename WeightT, typename SumT>
__global__ void __launch_bounds__(256) rows_by_key_atomic_kernel(SumT* __restrict__ sums,
                                                                unsigned long long* __restrict__ counts,
                                                                const DataT* __restrict__ A,
                                                                int64_t lda,
                                                                const KeyT* __restrict__ keys,
                                                                const WeightT* __restrict__ weights,
                                                                int64_t nrows,
                                                                int64_t ncols)
{
  const int64_t total = nrows * ncols;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int64_t r = i / ncols;
    const int64_t c = i - r * ncols;
    const int64_t k = static_cast<int64_t>(keys[r]);
    SumT x          = SumT(A[r * lda + c]);
    if (weights != nullptr) x *= SumT(weights[r]);
    atomicAdd(&sums[k * ncols + c], x);
    if (c == 0 && counts != nullptr) atomicAdd(&counts[k], 1ull);
  }
}

template <typename DataT, typename SumT>
inline RowsByKeyPlan plan_rows_by_key(const DataT* A, int64_t lda, int64_t nrows, int64_t ncols, int64_t nkeys)
{
  using State          = CompensatedState<SumT>;
  constexpr int NW     = kKeyTpb / 32;
  constexpr int V16    = vec16<DataT>::value;
  const size_t budget  = size_t(225) << 10;  // of the 227 KB a CTA may opt into
  RowsByKeyPlan p      = {};
  const bool vec_ok    = V16 > 1 && ncols % V16 == 0 && lda % V16 == 0 && aligned16(A);
  p.vec                = vec_ok ? V16 : 1;
  int B                = tuning().key_block_rows;
  if (B > kKeyMaxPerThr * kKeyTpb) B = kKeyMaxPerThr * kKeyTpb;
  if (B < 32) B = 32;
  if (int64_t(B) > nrows) B = int(ceil_div<int64_t>(nrows > 0 ? nrows : 1, 32) * 32);
  p.block_rows = B;
  // fixed shared memory besides the table, per key and per CTA
  const size_t per_cta = align_up(size_t(B) * 2, 16) + 64 * 4 + 64;
  const size_t per_key = size_t(ncols) * sizeof(State) + 8 + 4 + 4;
  if (per_cta + per_key + 64 > budget) {
    p.kps = 0;  // not even one key row fits: atomic fallback
    return p;
  }
  int64_t kps = int64_t((budget - per_cta - 64) / per_key);
  if (kps > nkeys) kps = nkeys;
  if (kps > 32767) kps = 32767;
  // private copies per warp when the whole table fits NW times
  const size_t private_need = per_cta + 64 + size_t(nkeys) * (size_t(NW) * ncols * sizeof(State) + 16);
  p.repl                    = (kps == nkeys && private_need <= budget) ? NW : 1;
  p.n_slices                = int(ceil_div<int64_t>(nkeys, kps));
  p.kps                     = int(ceil_div<int64_t>(nkeys, p.n_slices));  // even slices
  const int sms             = sm_count();
  int64_t R                 = sms / p.n_slices;
  if (R < 1) R = 1;
  const int64_t max_R = ceil_div<int64_t>(nrows > 0 ? nrows : 1, B);
  if (R > max_R) R = max_R;
  p.n_groups       = int(R);
  int64_t rpg      = ceil_div<int64_t>(nrows > 0 ? nrows : 1, R);
  rpg              = ceil_div<int64_t>(rpg, B) * B;
  p.rows_per_group = rpg;
  p.n_groups       = int(ceil_div<int64_t>(nrows > 0 ? nrows : 1, rpg));
  p.smem           = rows_by_key_smem<SumT>(p.kps, int(ncols), p.repl, B).total;
  p.scratch_sums   = align_up(size_t(p.n_groups) * nkeys * ncols * sizeof(SumT), 256);
  p.scratch_counts = align_up(size_t(p.n_groups) * nkeys * sizeof(unsigned long long), 256);
  return p;
}

template <typename DataT, typename SumT>
inline size_t rows_by_key_scratch_bytes(const DataT* A, int64_t lda, int64_t nrows, int64_t ncols, int64_t nkeys)
{
  if (nrows <= 0 || ncols <= 0 || nkeys <= 0) return 0;
  if (rows_by_key_small_supported(nrows, ncols, nkeys) &&
      (tuning().key_algo == 3 ||
       (tuning().key_algo == 0 && rows_by_key_small_preferred(nrows, ncols, nkeys, sizeof(DataT)))))
    return 0;  // one launch, no scratch
  if (tuning().key_algo != 1 && rows_by_key_sorted_supported(nrows, ncols, nkeys))
    return plan_rows_by_key_sorted<DataT>(A, lda, nrows, ncols, nkeys,
                                          sizeof(typename sum_state<SumT>::type::carry_t)).total;
  const RowsByKeyPlan p = plan_rows_by_key<DataT, SumT>(A, lda, nrows, ncols, nkeys);
  return p.kps == 0 ? 0 : p.scratch_sums + p.scratch_counts;
}

// counts may be null. When it is not, it receives (reset) or accumulates (!reset) the
// number of rows per key as int64 - an extension; the reference has no count output.
template <typename DataT, typename KeyT, typename WeightT, typename SumT>
cudaError_t launch_rows_by_key(SumT* sums,
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
                               Workspace ws = Workspace{})
{
  if (ncols <= 0 || nkeys <= 0) return cudaSuccess;
  cudaError_t e;
  if (nrows <= 0) {
    if (reset) {
      e = cudaMemsetAsync(sums, 0, size_t(nkeys) * ncols * sizeof(SumT), stream);
      if (e != cudaSuccess) return e;
      if (counts != nullptr) return cudaMemsetAsync(counts, 0, size_t(nkeys) * sizeof(long long), stream);
    }
    return cudaSuccess;
  }
  // small inputs: one launch (key_algo 0 = by size; forced: 1 = shared-memory table, 2 = sorted pipeline,
  // 3 = one-launch kernel)
  if (rows_by_key_small_supported(nrows, ncols, nkeys) &&
      (tuning().key_algo == 3 ||
       (tuning().key_algo == 0 && rows_by_key_small_preferred(nrows, ncols, nkeys, sizeof(DataT)))))
    return launch_rows_by_key_small<DataT, KeyT, WeightT, SumT>(sums, counts, A, lda, keys, weights, nrows, ncols,
                                                                nkeys, reset, stream);
  if (tuning().key_algo != 1 && rows_by_key_sorted_supported(nrows, ncols, nkeys))
    return launch_rows_by_key_sorted<DataT, KeyT, WeightT, SumT>(sums, counts, A, lda, keys, weights, nrows, ncols,
                                                                 nkeys, reset, stream, ws);
  constexpr int V16     = vec16<DataT>::value;
  const RowsByKeyPlan p = plan_rows_by_key<DataT, SumT>(A, lda, nrows, ncols, nkeys);
  if (p.kps == 0 || ncols > int64_t(0x7fffffff) || nkeys > int64_t(0x7fffffff)) {
    if (reset) {
      e = cudaMemsetAsync(sums, 0, size_t(nkeys) * ncols * sizeof(SumT), stream);
      if (e != cudaSuccess) return e;
      if (counts != nullptr) {
        e = cudaMemsetAsync(counts, 0, size_t(nkeys) * sizeof(long long), stream);
        if (e != cudaSuccess) return e;
      }
    }
    int64_t ctas = ceil_div<int64_t>(nrows * ncols, 256);
    const int64_t cap = int64_t(sm_count()) * 32;
    if (ctas > cap) ctas = cap;
    rows_by_key_atomic_kernel<DataT, KeyT, WeightT, SumT><<<unsigned(ctas), 256, 0, stream>>>(
      sums, reinterpret_cast<unsigned long long*>(counts), A, lda, keys, weights, nrows, ncols);
    return cudaGetLastError();
  }

  Scratch scratch(ws, p.scratch_sums + p.scratch_counts, stream);
  if (scratch.error() != cudaSuccess) return scratch.error();
  SumT* partial_sums = static_cast<SumT*>(scratch.get());
  unsigned long long* partial_counts =
    reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(scratch.get()) + p.scratch_sums);
  const RowsByKeySmem<SumT> lay = rows_by_key_smem<SumT>(p.kps, int(ncols), p.repl, p.block_rows);
  const dim3 grid{unsigned(p.n_slices), unsigned(p.n_groups), 1u};

#define B2R_LAUNCH_RBK(VEC_)                                                                        \
  do {                                                                                              \
    auto kern = rows_by_key_partial_kernel<DataT, KeyT, WeightT, SumT, VEC_>;                       \
    e = ensure_dynamic_smem(kern, size_t(lay.total));    \
    if (e != cudaSuccess) return e;                                                                 \
    kern<<<grid, kKeyTpb, lay.total, stream>>>(partial_sums, partial_counts, A, lda, keys, weights, \
                                               nrows, int(ncols), int(nkeys), p.kps,                \
                                               p.rows_per_group, p.block_rows, p.repl, lay);        \
  } while (0)
  if (p.vec > 1) {
    B2R_LAUNCH_RBK(V16);
  } else {
    B2R_LAUNCH_RBK(1);
  }
#undef B2R_LAUNCH_RBK
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int64_t elems = nkeys * ncols;
  const int64_t n_thr = elems > nkeys ? elems : nkeys;
  rows_by_key_merge_kernel<SumT><<<unsigned(ceil_div<int64_t>(n_thr, 256)), 256, 0, stream>>>(
    sums, counts, partial_sums, partial_counts, p.n_groups, elems, int(nkeys), reset);
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
