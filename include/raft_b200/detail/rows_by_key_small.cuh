// Keyed row sums of SMALL inputs (up to kSmallMaxRows rows) in ONE launch:
//     sums[keys[i]][:] += w[i] * A[i][:]
//
// The sorted pipeline of rows_by_key_sorted.cuh needs six launches, which is all a few-MB input
// pays for. Here every CTA (one per SM) owns a contiguous range of keys: it reads the whole key
// vector once (a few tens of KB, from L2), counting-sorts the rows of ITS keys into shared memory (integer atomics),
// and then adds those rows up, one warp per (key, slice of its rows), sums per column in registers
// (fp64-carried / compensated) - every matrix row is read once, by exactly one CTA, nothing is
// shared between CTAs, there are no floating-point atomics and no scratch memory.
#pragma once

#include "common.cuh"
#include "launch.cuh"
#include "ops.cuh"

namespace raft_b200 {
namespace detail {

constexpr int kSmallMaxRows = 32768;  // row numbers are staged as 16-bit values and every CTA scans all keys
constexpr int kSmallTpb     = 512;

template <typename DataT, typename KeyT, typename WeightT, typename SumT, int VEC>
__global__ void __launch_bounds__(kSmallTpb) rbk_small_kernel(SumT* __restrict__ sums,
                                                             long long* __restrict__ counts,
                                                             const DataT* __restrict__ A,
                                                             int64_t lda,
                                                             const KeyT* __restrict__ keys,
                                                             const WeightT* __restrict__ weights,
                                                             int nrows,
                                                             int ncols,
                                                             int nkeys,
                                                             int keys_per_cta,
                                                             int G,
                                                             bool reset)
{
  using State = typename sum_state<SumT>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* s_off             = reinterpret_cast<int*>(smem_raw);                         // [keys_per_cta + 1]
  int* s_cur             = s_off + keys_per_cta + 1;                                 // [keys_per_cta]
  unsigned short* s_rows = reinterpret_cast<unsigned short*>(s_cur + keys_per_cta);  // [nrows] rows sorted by key
  unsigned char* tail    = smem_raw + (size_t(2 * keys_per_cta + 1) * 4 + size_t(nrows) * 2 + 15) / 16 * 16;
  unsigned short* s_lk   = reinterpret_cast<unsigned short*>(tail);  // [nrows] key - k0 of every row, 0xffff: not mine
  State* s_part          = reinterpret_cast<State*>(tail);           // [warps][32 * VEC], after the sort is done
  __shared__ int s_warp[kSmallTpb / 32];
  __shared__ int s_total;

  const int tid  = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int k0   = blockIdx.x * keys_per_cta;
  int nk         = nkeys - k0;
  nk             = nk < keys_per_cta ? nk : keys_per_cta;
  if (nk <= 0) return;
  const op::Add add{};

  // 1. counting sort of the rows whose key lies in [k0, k0 + nk)
  for (int k = tid; k < nk; k += kSmallTpb)
    s_cur[k] = 0;
  __syncthreads();
  constexpr int KU = 8;  // independent key loads in flight per thread
  for (int i0 = 0; i0 < nrows; i0 += KU * kSmallTpb) {
    long long kk[KU];
#pragma unroll
    for (int j = 0; j < KU; ++j) {
      const int i = i0 + j * kSmallTpb + tid;
      kk[j]       = i < nrows ? static_cast<long long>(keys[i]) - k0 : -1;
    }
#pragma unroll
    for (int j = 0; j < KU; ++j) {
      const int i = i0 + j * kSmallTpb + tid;
      if (i < nrows) {
        const bool mine = kk[j] >= 0 && kk[j] < nk;
        s_lk[i]         = mine ? static_cast<unsigned short>(kk[j]) : static_cast<unsigned short>(0xffff);
        if (mine) atomicAdd(&s_cur[int(kk[j])], 1);
      }
    }
  }
  __syncthreads();
  int run = 0;
  for (int kb = 0; kb < nk; kb += kSmallTpb) {
    const int k = kb + tid;
    const int t = k < nk ? s_cur[k] : 0;
    int inc     = t;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += a;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int v = lane < kSmallTpb / 32 ? s_warp[lane] : 0;
      int wi      = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += a;
      }
      if (lane < kSmallTpb / 32) s_warp[lane] = wi - v;
      if (lane == 31) s_total = wi;
    }
    __syncthreads();
    const int first = run + s_warp[warp] + inc - t;
    if (k < nk) {
      s_off[k] = first;
      s_cur[k] = first;
    }
    run += s_total;
    __syncthreads();
  }
  if (tid == 0) s_off[nk] = run;
  __syncthreads();
  for (int i = tid; i < nrows; i += kSmallTpb) {
    const unsigned k = s_lk[i];
    if (k != 0xffffu) s_rows[atomicAdd(&s_cur[k], 1)] = static_cast<unsigned short>(i);
  }
  __syncthreads();  // s_lk is dead from here on: s_part takes its place
  if (counts != nullptr) {
    for (int k = tid; k < nk; k += kSmallTpb) {
      const long long n = s_off[k + 1] - s_off[k];
      counts[k0 + k]    = reset ? n : counts[k0 + k] + n;
    }
  }

  // 2. sums: S warps share a key when the CTA has fewer keys than warps
  constexpr int NW = kSmallTpb / 32;
  constexpr int Q  = 8;  // row loads in flight per lane
  const int S      = nk < NW ? NW / nk : 1;
  const int lg     = 31 - __clz(G);
  const int lig    = lane & (G - 1);
  const int grp    = lane >> lg;
  const int gpw    = 32 >> lg;
  const int nvec   = ncols / VEC;  // VEC divides ncols on the vector path
  for (int cv0 = 0; cv0 < nvec; cv0 += G) {
    const int cv      = cv0 + lig;
    const bool col_ok = cv < nvec;
    for (int it0 = 0; it0 < nk * S; it0 += NW) {  // uniform trip count: barriers inside when S > 1
      const int item  = it0 + warp;
      const bool live = item < nk * S;
      const int k     = live ? item / S : 0;
      const int sl    = live ? item - k * S : 0;
      State acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        acc[e].init(SumT(0));
      if (live) {
        const int seg0 = s_off[k], len = s_off[k + 1] - seg0;
        const int j0 = seg0 + int((long long)len * sl / S), j1 = seg0 + int((long long)len * (sl + 1) / S);
        for (int i0 = j0; i0 < j1; i0 += Q * gpw) {
          VecOf<DataT, VEC> v[Q];
          SumT w[Q];
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            int i           = i0 + q * gpw + grp;
            i               = i < j1 ? i : j1 - 1;  // duplicate, masked below
            const int64_t r = s_rows[i];
            v[q]            = load_stream<DataT, VEC>(A + r * lda + int64_t(col_ok ? cv : 0) * VEC);
            w[q]            = weights != nullptr ? SumT(weights[r]) : SumT(1);
          }
#pragma unroll
          for (int q = 0; q < Q; ++q) {
            if (i0 + q * gpw + grp < j1) {
#pragma unroll
              for (int e = 0; e < VEC; ++e) {
                SumT x = SumT(v[q].e[e]);
                if (weights != nullptr) x *= w[q];
                acc[e].push(x, add);
              }
            }
          }
        }
      }
      // fold the row groups of the warp (different rows of the same columns)
      for (int off = G; off < 32; off <<= 1) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          State got = shfl_xor_any(acc[e], off);
          acc[e].merge(got, add);
        }
      }
      if (S > 1) {
        // the S warps of a key meet in shared memory; the first of them adds up in warp order
        if (grp == 0) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            s_part[(warp * 32 + lig) * VEC + e] = acc[e];
        }
        __syncthreads();
        if (live && sl == 0 && grp == 0) {
          for (int s = 1; s < S; ++s) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              acc[e].merge(s_part[((warp + s) * 32 + lig) * VEC + e], add);
          }
        }
        __syncthreads();
      }
      if (live && sl == 0 && grp == 0 && col_ok) {
        SumT* dst = sums + size_t(k0 + k) * ncols + size_t(cv) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          if (!reset) acc[e].push(dst[e], add);
          dst[e] = acc[e].value();
        }
      }
    }
  }
}

// One CTA adds up ALL rows of its keys: fine while that is about a megabyte per CTA (ranges of keys
// go to at most one CTA per SM); beyond that - few keys or long rows - the sorted pipeline spreads
// the rows of a key over many warps and wins although it needs six launches.
inline bool rows_by_key_small_preferred(int64_t nrows, int64_t ncols, int64_t nkeys, size_t elem_size)
{
  const int64_t ctas = nkeys < sm_count() ? nkeys : sm_count();
  return nrows * ncols * int64_t(elem_size) <= ctas * (int64_t(1) << 20);
}

inline bool rows_by_key_small_supported(int64_t nrows, int64_t ncols, int64_t nkeys)
{
  // keys per CTA are staged as 16-bit values too (0xffff = not this CTA's key)
  return nrows > 0 && nrows <= kSmallMaxRows && ncols > 0 && ncols <= int64_t(0x7fffffff) && nkeys > 0 &&
         nkeys <= int64_t(1) << 22;
}

template <typename DataT, typename KeyT, typename WeightT, typename SumT>
cudaError_t launch_rows_by_key_small(SumT* sums,
                                     long long* counts,
                                     const DataT* A,
                                     int64_t lda,
                                     const KeyT* keys,
                                     const WeightT* weights,
                                     int64_t nrows,
                                     int64_t ncols,
                                     int64_t nkeys,
                                     bool reset,
                                     cudaStream_t stream)
{
  constexpr int V16 = vec16<DataT>::value;
  using State       = typename sum_state<SumT>::type;
  const bool vec_ok = V16 > 1 && ncols % V16 == 0 && lda % V16 == 0 && aligned16(A);
  const int vec     = vec_ok ? V16 : 1;
  int64_t ctas      = int64_t(sm_count());  // one wave: every CTA reads the whole key vector
  if (ctas > nkeys) ctas = nkeys;
  const int kpc     = int(ceil_div<int64_t>(nkeys, ctas));
  ctas              = ceil_div<int64_t>(nkeys, kpc);
  const int nvec    = int(ncols / vec);
  const unsigned g  = next_pow2(unsigned(nvec > 0 ? nvec : 1));
  const int G       = int(g > 32u ? 32u : g);
  const size_t head = (size_t(2 * kpc + 1) * 4 + size_t(nrows) * 2 + 15) / 16 * 16;
  const size_t part = size_t(kSmallTpb / 32) * 32 * size_t(vec) * sizeof(State);
  const size_t lk   = size_t(nrows) * 2;
  const size_t smem = head + (part > lk ? part : lk);
  cudaError_t e;
#define B2R_LAUNCH_SMALL(VEC_)                                                                             \
  do {                                                                                                     \
    auto kern = rbk_small_kernel<DataT, KeyT, WeightT, SumT, VEC_>;                                        \
    if (smem + 1024 > (size_t(48) << 10)) {                                                                \
      e = ensure_dynamic_smem(kern, smem);                                                                 \
      if (e != cudaSuccess) return e;                                                                      \
    }                                                                                                      \
    kern<<<unsigned(ctas), kSmallTpb, smem, stream>>>(sums, counts, A, lda, keys, weights, int(nrows),     \
                                                      int(ncols), int(nkeys), kpc, G, reset);              \
  } while (0)
  if (vec > 1) {
    B2R_LAUNCH_SMALL(V16);
  } else {
    B2R_LAUNCH_SMALL(1);
  }
#undef B2R_LAUNCH_SMALL
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
