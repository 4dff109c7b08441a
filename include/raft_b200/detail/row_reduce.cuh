// Reduction along the contiguous axis: out[i] = final(reduce_j main(x[i][j], j)).
//
// Replaces the reference's thin / medium / thick coalesced kernels
// (linalg/detail/coalesced_reduction-inl.cuh:48-227, 329-400, 481-533) with two kernels
// and a shape policy:
//
//  row_reduce_kernel   a sub-warp of G lanes (G = 1..32, chosen from the row length) owns a
//                      row; every lane keeps U independent 16-byte loads in flight.
//                        kRows   mode: the U loads belong to U different rows (short rows);
//                                      the U partials of a group are finished together by
//                                      the transposing sub-warp reduction, which also
//                                      spreads the outputs over lanes for a packed store.
//                        kChunks mode: the U loads are U consecutive chunks of the SAME row
//                                      (rows of a few KB and more, one row per group).
//  row_split_kernel    few but very long rows: a row is cut into S segments, one CTA each;
//                      the S partials per row go to scratch memory and a second, tiny
//                      row_reduce_kernel pass folds them and applies init / inplace / final.
//
// fp32 sums are carried in fp64 (WideSumState), fp64 sums are compensated; every other operator
// runs through GenericState. main_op receives the index along the reduced axis, as in the
// reference. The stored type may differ from the accumulator type (StoreT = what final_op
// returns, e.g. only the key of a key/value pair); such a reduction cannot run in place.
#pragma once

#include "common.cuh"
#include "ops.cuh"

namespace raft_b200 {
namespace detail {

enum RowMode : int { kRows = 0, kChunks = 1 };

template <typename OutT, typename State, bool IsSum>
B2R_DI void init_state(State& st, const OutT& init, bool first_lane)
{
  if constexpr (IsSum) {
    // the initial value enters a sum exactly once
    st.init(first_lane ? init : OutT(0));
  } else {
    // any other operator: init must be its identity (or the op idempotent), as the
    // reference requires, because every lane starts from it
    st.init(init);
  }
}

// state <- reduce_op(state, main_op(x, idx)): the one place an element enters a state.
template <typename OutT, typename IdxT, typename State, typename InT, typename I, typename MainOp, typename ReduceOp>
B2R_DI void push_element(State& st, const InT& x, I idx, MainOp& main_op, ReduceOp& reduce_op)
{
  st.push(OutT(main_op(x, IdxT(idx))), reduce_op);
}

// argmin / argmax of tagged values: the same result as argmin_op(state, {idx, x}) - smaller
// (larger) value wins, equal values keep the lower key - written as one predicate and two
// selects so that no key/value pair is materialised per element.
template <typename OutT, typename IdxT, typename K, typename V, typename I>
B2R_DI void push_element(GenericState<KeyValue<K, V>, op::ArgMin>& st, const V& x, I idx, op::ToKeyValue<K>&, op::ArgMin&)
{
  const K k       = K(idx);
  const bool take = (x < st.v.value) | ((x == st.v.value) & (k < st.v.key));
  st.v.value      = take ? x : st.v.value;
  st.v.key        = take ? k : st.v.key;
}
template <typename OutT, typename IdxT, typename K, typename V, typename I>
B2R_DI void push_element(GenericState<KeyValue<K, V>, op::ArgMax>& st, const V& x, I idx, op::ToKeyValue<K>&, op::ArgMax&)
{
  const K k       = K(idx);
  const bool take = (x > st.v.value) | ((x == st.v.value) & (k < st.v.key));
  st.v.value      = take ? x : st.v.value;
  st.v.key        = take ? k : st.v.key;
}

// Row argmin / argmax of tagged values in the one-pass kernels: a lane walks ITS elements of a row in
// ascending column order, so among them "strictly better" alone keeps the first best one - one compare and two
// selects per element instead of three compares. To stay exactly argmin_op(init, elements) the lanes do not
// start from `init` but from {largest key, init.value}: nothing but a strictly better value replaces that,
// a walk that found none looks once more for elements EQUAL to init.value (they win the tie against the largest
// key, the first of them having the lowest column), the cross-lane merges use the full rule, and the writer
// folds the caller's `init` in last. NaN elements are never taken, as with the full rule.
template <typename State, typename MainOp, typename ReduceOp>
struct kvp_walk : std::false_type {};
template <typename K, typename V>
struct kvp_walk<GenericState<KeyValue<K, V>, op::ArgMin>, op::ToKeyValue<K>, op::ArgMin> : std::true_type {
  static constexpr bool is_min = true;
};
template <typename K, typename V>
struct kvp_walk<GenericState<KeyValue<K, V>, op::ArgMax>, op::ToKeyValue<K>, op::ArgMax> : std::true_type {
  static constexpr bool is_min = false;
};
template <typename K>
B2R_DI constexpr K kvp_largest_key()
{
  return K(~K(0)) > K(0) ? K(~K(0)) : K((unsigned long long)(~0ull) >> (65 - 8 * sizeof(K)));
}

// The U x CPL vectors a lane holds of U rows (chunks lig, lig + G, ... of each), walked in column order.
template <bool IsMin, typename K, typename V, typename InT, int VEC, int U, int CPL>
B2R_DI void kvp_walk_rows(GenericState<KeyValue<K, V>, typename std::conditional<IsMin, op::ArgMin, op::ArgMax>::type> (&st)[U],
                          const VecOf<InT, VEC> (&v)[U][CPL], int first_col, int chunk_stride_cols, V start)
{
  constexpr K kLast = kvp_largest_key<K>();
#pragma unroll
  for (int u = 0; u < U; ++u) {
    V bv = start;
    K bk = kLast;
#pragma unroll
    for (int k = 0; k < CPL; ++k) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const V x       = V(v[u][k].e[e]);
        const bool take = IsMin ? (x < bv) : (x > bv);
        bv              = take ? x : bv;
        bk              = take ? K(first_col + k * chunk_stride_cols + e) : bk;
      }
    }
    if (bk == kLast) {  // nothing beat the start value: elements equal to it still beat the largest key
#pragma unroll
      for (int k = CPL - 1; k >= 0; --k) {
#pragma unroll
        for (int e = VEC - 1; e >= 0; --e) {
          if (V(v[u][k].e[e]) == bv) bk = K(first_col + k * chunk_stride_cols + e);
        }
      }
    }
    st[u].v.key   = bk;
    st[u].v.value = bv;
  }
}

template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          int VEC,
          int U,
          int MODE,
          int TPB,
          int CPL   = 1,
          typename StoreT = OutT>
__global__ void __launch_bounds__(TPB, (sizeof(OutT) <= 8 && U * CPL <= 8 ? 4 : 2)) row_reduce_kernel(StoreT* __restrict__ out,
                                                        const InT* __restrict__ data,
                                                        int64_t n_rows,
                                                        int row_len,
                                                        int64_t ld,
                                                        OutT init,
                                                        bool inplace,
                                                        MainOp main_op,
                                                        ReduceOp reduce_op,
                                                        FinalOp final_op,
                                                        int G,
                                                        int64_t batches_per_cta,
                                                        bool unaligned_rows = false)
{
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  grid_dep_sync();

  const int lane  = threadIdx.x & 31;
  const int lg    = 31 - __clz(G);    // G is a power of two
  const int lig   = lane & (G - 1);   // lane in group
  const int grp   = lane >> lg;       // group in warp
  const int gsh   = 5 - lg;           // log2(groups per warp)
  const int gpw   = 1 << gsh;         // groups per warp
  const int nvec  = row_len / VEC;    // VEC divides row_len on the vector path; VEC==1 otherwise

  // A CTA owns a contiguous range of row batches (so that it streams one contiguous piece of
  // the matrix); its warps interleave inside the range. The launcher gives a CTA one batch per warp by default
  // (many short CTAs), more only in chunk mode or when asked to.
  constexpr int64_t warps_total = TPB / 32;
  const int64_t cta_first       = int64_t(blockIdx.x) * batches_per_cta;
  const int64_t warp_global     = cta_first + (threadIdx.x >> 5);

  if constexpr (MODE == kRows) {
    const int rows_per_batch = U * gpw;
    constexpr int ush        = ilog2_floor(U);
    int64_t n_batches        = (n_rows + rows_per_batch - 1) >> (gsh + ush);
    n_batches                = n_batches < cta_first + batches_per_cta ? n_batches : cta_first + batches_per_cta;
    for (int64_t b = warp_global; b < n_batches; b += warps_total) {
      const int64_t row0 = b * rows_per_batch + grp;  // slot u -> row0 + u*gpw
      // slots of this group that are real rows; the others re-read the last real row (their
      // results are never stored), which keeps the load pattern uniform
      const int64_t left = n_rows - row0;
      const int64_t slots = (left + gpw - 1) >> gsh;
      const int valid     = left <= 0 ? 0 : int(slots < U ? slots : U);
      const InT* base    = data + (valid > 0 ? row0 : n_rows - 1) * ld;
      const int64_t step = valid > 0 ? int64_t(gpw) * ld : 0;
      State st[U];
      constexpr bool kWalk = kvp_walk<State, MainOp, ReduceOp>::value;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if constexpr (kWalk) {
          st[u].v.key   = kvp_largest_key<decltype(st[u].v.key)>();
          st[u].v.value = init.value;
        } else {
          init_state<OutT, State, isSum>(st[u], init, lig == 0);
        }
      }
      // CPL chunks of every row per lane and pass: U * CPL loads are in flight per lane, and the
      // more of a row one lane sums by itself the fewer exchanges the reduction below needs
      // (the pass structure is the same for every lane of the warp - a pass is "full" only if it is for
      // the whole group - so a row length that is no multiple of G * CPL costs one masked pass, not two
      // serialised ones)
      for (int cb = 0; cb < nvec; cb += G * CPL) {
        const int c0 = cb + lig;
        if constexpr (CPL == 1) {
          if (c0 >= nvec) break;  // one chunk per lane and pass: a lane beyond the row's end is simply done
        }
        VecOf<InT, VEC> v[U][CPL];
        if (valid == U && (CPL == 1 || cb + CPL * G <= nvec)) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int k = 0; k < CPL; ++k)
              v[u][k] = load_stream<InT, VEC>(base + u * step + int64_t(c0 + k * G) * VEC);
          }
          if constexpr (kWalk) {
            if (cb == 0) {
              // the row's first (for one-pass rows: only) pass: the lane's own columns in ascending order
              kvp_walk_rows<kvp_walk<State, MainOp, ReduceOp>::is_min>(st, v, c0 * VEC, G * VEC, init.value);
            } else {
#pragma unroll
              for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int k = 0; k < CPL; ++k) {
#pragma unroll
                  for (int e = 0; e < VEC; ++e)
                    push_element<OutT, IdxT>(st[u], v[u][k].e[e], (c0 + k * G) * VEC + e, main_op, reduce_op);
                }
              }
            }
          } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
              for (int k = 0; k < CPL; ++k) {
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                  push_element<OutT, IdxT>(st[u], v[u][k].e[e], (c0 + k * G) * VEC + e, main_op, reduce_op);
              }
            }
          }
        } else {
          // ragged batch (fewer than U real rows) or ragged row end (fewer than CPL chunks left)
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int uu = u < valid ? u : (valid > 0 ? valid - 1 : 0);
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              const int c  = c0 + k * G;
              const int cc = c < nvec ? c : cb;  // re-read a valid chunk, ignored below
              v[u][k]      = load_stream<InT, VEC>(base + uu * step + int64_t(cc) * VEC);
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
              if (c0 + k * G < nvec) {
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                  push_element<OutT, IdxT>(st[u], v[u][k].e[e], (c0 + k * G) * VEC + e, main_op, reduce_op);
              }
            }
          }
        }
      }
      subwarp_transpose_reduce<U>(st, lig, G, reduce_op);
      const SubwarpLayout lay = subwarp_layout<U>(lig, G);
      if (lay.writer) {
#pragma unroll
        for (int i = 0; i < U; ++i) {
          if (i < lay.n_final) {
            const int slot  = lay.prefix * lay.n_final + i;
            const int64_t r = row0 + int64_t(slot) * gpw;
            if (r < n_rows) {
              OutT v = st[i].value();
              if constexpr (kWalk) v = reduce_op(init, v);  // the lanes started from {largest key, init.value}
              if constexpr (std::is_same<StoreT, OutT>::value) {
                if (inplace) v = reduce_op(out[r], v);
              }
              out[r] = final_op(v);
            }
          }
        }
      }
    }
  } else {
    // kChunks: one row per group, U chunks of it in flight per lane.
    int64_t n_batches = (n_rows + gpw - 1) >> gsh;
    n_batches         = n_batches < cta_first + batches_per_cta ? n_batches : cta_first + batches_per_cta;
    for (int64_t b = warp_global; b < n_batches; b += warps_total) {
      const int64_t row = b * gpw + grp;
      const int64_t rc  = row < n_rows ? row : n_rows - 1;
      const InT* rp     = data + rc * ld;
      State st[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        init_state<OutT, State, isSum>(st[u], init, lig == 0 && u == 0);
      // Rows that do not start on a 16-byte boundary (unaligned_rows, vector instantiations only):
      // up to VEC - 1 leading and trailing elements are taken one by one, by the first lanes of
      // the group, and the vectors in between are aligned. `head` shifts the column indices.
      int head = 0, nv = nvec;
      if constexpr (VEC > 1) {
        if (unaligned_rows) {
          const int lead = int(((16u - unsigned(reinterpret_cast<uintptr_t>(rp) & 15u)) & 15u) / sizeof(InT));
          head           = lead < row_len ? lead : row_len;
          nv             = (row_len - head) / VEC;
          const int tail = row_len - head - nv * VEC;
          if (lig < head) push_element<OutT, IdxT>(st[U - 1], rp[lig], lig, main_op, reduce_op);
          if (lig < tail)
            push_element<OutT, IdxT>(st[U - 1], rp[head + nv * VEC + lig], head + nv * VEC + lig, main_op, reduce_op);
          rp += head;
        }
      }
      // full passes for the whole group first (the same count for every lane), then one masked pass
      int c = lig;
      for (int cb = 0; cb + U * G <= nv; cb += U * G, c += U * G) {
        VecOf<InT, VEC> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = load_stream<InT, VEC>(rp + int64_t(c + u * G) * VEC);
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            push_element<OutT, IdxT>(st[u], v[u].e[e], head + (c + u * G) * VEC + e, main_op, reduce_op);
        }
      }
      if (c - lig < nv) {
        // ragged end of the row: the chunks that are left go out together, not one by one
        VecOf<InT, VEC> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = load_stream<InT, VEC>(rp + int64_t(c + u * G < nv ? c + u * G : c - lig) * VEC);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (c + u * G < nv) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              push_element<OutT, IdxT>(st[u], v[u].e[e], head + (c + u * G) * VEC + e, main_op, reduce_op);
          }
        }
      }
#pragma unroll
      for (int u = 1; u < U; ++u)
        st[0].merge(st[u], reduce_op);
      for (int off = G >> 1; off > 0; off >>= 1) {
        State got = shfl_xor_any(st[0], off);
        st[0].merge(got, reduce_op);
      }
      if (lig == 0 && row < n_rows) {
        OutT v = st[0].value();
        if constexpr (std::is_same<StoreT, OutT>::value) {
          if (inplace) v = reduce_op(out[row], v);
        }
        out[row] = final_op(v);
      }
    }
  }
}

// One CTA per (segment, row). Writes either the finished output (n_seg == 1) or the
// partial of its segment to partial[row * n_seg + seg].
template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          int VEC,
          int U,
          int TPB,
          typename StoreT = OutT>
__global__ void __launch_bounds__(TPB) row_split_kernel(StoreT* __restrict__ out,
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
                                                       int64_t seg_vecs)
{
  grid_dep_sync();
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  __shared__ State s_warp[TPB / 32];

  const int n_seg    = gridDim.x;
  const int seg      = blockIdx.x;
  const int64_t nvec = row_len / VEC;
  const int64_t v0   = int64_t(seg) * seg_vecs;
  int64_t v1         = v0 + seg_vecs;
  v1                 = v1 < nvec ? v1 : nvec;
  const bool direct  = n_seg == 1;

  for (int64_t row = blockIdx.y; row < n_rows; row += gridDim.y) {
    const InT* rp = data + row * ld;
    State st[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      init_state<OutT, State, isSum>(st[u], init, direct && threadIdx.x == 0 && u == 0);
    int64_t c = v0 + threadIdx.x;
    for (; c + int64_t(U - 1) * TPB < v1; c += int64_t(U) * TPB) {
      VecOf<InT, VEC> v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        v[u] = load_stream<InT, VEC>(rp + (c + int64_t(u) * TPB) * VEC);
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          st[u].push(OutT(main_op(v[u].e[e], IdxT((c + int64_t(u) * TPB) * VEC + e))), reduce_op);
      }
    }
    for (; c < v1; c += TPB) {
      VecOf<InT, VEC> v = load_stream<InT, VEC>(rp + c * VEC);
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        st[0].push(OutT(main_op(v.e[e], IdxT(c * VEC + e))), reduce_op);
    }
    if constexpr (VEC > 1) {
      // a row length that is no multiple of the vector width: the last segment takes the tail
      if (seg == n_seg - 1) {
        for (int64_t i = nvec * VEC + threadIdx.x; i < row_len; i += TPB)
          st[0].push(OutT(main_op(rp[i], IdxT(i))), reduce_op);
      }
    }
#pragma unroll
    for (int u = 1; u < U; ++u)
      st[0].merge(st[u], reduce_op);
    State r = block_merge(st[0], reduce_op, s_warp);
    if (threadIdx.x == 0) {
      if (direct) {
        OutT v = r.value();
        if constexpr (std::is_same<StoreT, OutT>::value) {
          if (inplace) v = reduce_op(out[row], v);
        }
        out[row] = final_op(v);
      } else {
        partial[row * n_seg + seg] = r.carry();
      }
    }
    __syncthreads();  // s_warp is reused by the next row
  }
}

// Folds the n_seg segment partials of every row (one warp per row, fixed order) and applies
// init, inplace and final_op.
template <typename OutT, typename ReduceOp, typename FinalOp, int TPB, typename StoreT = OutT>
__global__ void __launch_bounds__(TPB) row_finalize_kernel(StoreT* __restrict__ out,
                                                          const typename state_for<OutT, ReduceOp>::type::carry_t* __restrict__ partial,
                                                          int64_t n_rows,
                                                          int n_seg,
                                                          OutT init,
                                                          bool inplace,
                                                          ReduceOp reduce_op,
                                                          FinalOp final_op)
{
  grid_dep_sync();
  using State          = typename state_for<OutT, ReduceOp>::type;
  constexpr bool isSum = is_sum_op<ReduceOp>::value && std::is_floating_point<OutT>::value;
  const int lane       = threadIdx.x & 31;
  const int64_t row    = int64_t(blockIdx.x) * (TPB / 32) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  State st;
  init_state<OutT, State, isSum>(st, init, lane == 0);
  for (int sgm = lane; sgm < n_seg; sgm += 32)
    st.push_carry(partial[row * n_seg + sgm], reduce_op);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    State got = shfl_xor_any(st, off);
    st.merge(got, reduce_op);
  }
  if (lane == 0) {
    OutT v = st.value();
    if constexpr (std::is_same<StoreT, OutT>::value) {
      if (inplace) v = reduce_op(out[row], v);
    }
    out[row] = final_op(v);
  }
}

}  // namespace detail
}  // namespace raft_b200
