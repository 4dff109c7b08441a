// Row normalisation: out[i][:] = in[i][:] / norm_i with norm_i = final(reduce_j main(in[i][j], j)),
// rows whose norm is <= eps are left untouched in `out`
// (raft::linalg::row_normalize, linalg/normalize.cuh:46-107, kernels linalg/detail/normalize.cuh:26-197).
//
// Read-reduce-rescale in ONE pass over HBM: 2 x sizeof(T) bytes per element.
//
//  row_normalize_kernel       rows of up to 512 16-byte vectors (2048 fp32): a sub-warp of G lanes
//                             holds the whole row in registers (CPL vectors per lane), U rows at a
//                             time so that 8 or 16 loads are in flight per lane; butterfly reduction,
//                             then the same registers are divided and stored.
//  row_normalize_cta_kernel   rows of up to 4096 vectors (16384 fp32): one CTA per row, 4 / 8 / 16
//                             vectors per thread in registers, one barrier per row.
//  row_normalize_long_kernel  longer rows: one CTA per row, two sweeps; the second sweep re-reads the
//                             row from L1 / L2 (it was just touched), so DRAM still sees it once.
#pragma once

#include "common.cuh"
#include "launch.cuh"
#include "ops.cuh"
#include "row_normalize_staged.cuh"

namespace raft_b200 {
namespace detail {

template <typename T, int VEC>
B2R_DI void store_vec(T* p, const VecOf<T, VEC>& v)
{
  *reinterpret_cast<VecOf<T, VEC>*>(p) = v;
}

template <typename T, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp, int VEC, int CPL, int U>
__global__ void __launch_bounds__(256) row_normalize_kernel(T* out,
                                                           const T* in,
                                                           int64_t n_rows,
                                                           int64_t n_cols,
                                                           T init,
                                                           T eps,
                                                           MainOp main_op,
                                                           ReduceOp reduce_op,
                                                           FinalOp final_op,
                                                           int G)
{
  grid_dep_sync();
  using State = typename state_for<T, ReduceOp>::type;
  const int lane = threadIdx.x & 31;
  const int lg   = 31 - __clz(G);
  const int lig  = lane & (G - 1);
  const int grp  = lane >> lg;
  const int gpw  = 32 >> lg;              // rows per warp and load
  const int nvec = int(n_cols / VEC);     // VEC divides n_cols on the vector path
  const int64_t rows_per_pass = int64_t(gpw) * U;
  const int64_t warp0         = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps       = int64_t(gridDim.x) * (blockDim.x >> 5);
  bool chunk_ok[CPL];
#pragma unroll
  for (int k = 0; k < CPL; ++k)
    chunk_ok[k] = k * G + lig < nvec;

  for (int64_t r0 = warp0 * rows_per_pass; r0 < n_rows; r0 += n_warps * rows_per_pass) {
    VecOf<T, VEC> v[U][CPL];
    bool row_ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r  = r0 + int64_t(u) * gpw + grp;
      row_ok[u]        = r < n_rows;
      const T* row_ptr = in + (row_ok[u] ? r : r0) * n_cols;
#pragma unroll
      for (int k = 0; k < CPL; ++k)
        v[u][k] = load_stream<T, VEC>(row_ptr + int64_t(chunk_ok[k] ? k * G + lig : 0) * VEC);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      State st;
      st.init(init);
#pragma unroll
      for (int k = 0; k < CPL; ++k) {
        if (chunk_ok[k]) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            st.push(T(main_op(v[u][k].e[e], IdxT((k * G + lig) * VEC + e))), reduce_op);
        }
      }
      for (int off = G >> 1; off > 0; off >>= 1) {
        State got = shfl_xor_any(st, off);
        st.merge(got, reduce_op);
      }
      // every lane of the row divides by the SAME value: the one of the group's first lane
      const T norm = shfl_idx_any(T(final_op(st.value())), lane & ~(G - 1));
      if (row_ok[u] && !(norm <= eps)) {
        T* row_ptr = out + (r0 + int64_t(u) * gpw + grp) * n_cols;
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
          if (chunk_ok[k]) {
            VecOf<T, VEC> o;
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              o.e[e] = v[u][k].e[e] / norm;
            store_vec<T, VEC>(row_ptr + int64_t(k * G + lig) * VEC, o);
          }
        }
      }
    }
  }
}

// One CTA per row, the row held in registers (CPT vectors per thread): rows of up to 256 * CPT vectors.
template <typename T, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp, int VEC, int CPT>
__global__ void __launch_bounds__(256) row_normalize_cta_kernel(T* out,
                                                               const T* in,
                                                               int64_t n_rows,
                                                               int64_t n_cols,
                                                               T init,
                                                               T eps,
                                                               MainOp main_op,
                                                               ReduceOp reduce_op,
                                                               FinalOp final_op)
{
  grid_dep_sync();
  using State = typename state_for<T, ReduceOp>::type;
  __shared__ State s_state[2][8];  // double-buffered: one barrier per row
  const int tid  = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nvec = int(n_cols / VEC);
  bool chunk_ok[CPT];
#pragma unroll
  for (int k = 0; k < CPT; ++k)
    chunk_ok[k] = k * 256 + tid < nvec;
  int phase = 0;
  for (int64_t r = blockIdx.x; r < n_rows; r += gridDim.x, phase ^= 1) {
    const T* src = in + r * n_cols;
    VecOf<T, VEC> v[CPT];
#pragma unroll
    for (int k = 0; k < CPT; ++k)
      v[k] = load_stream<T, VEC>(src + int64_t(chunk_ok[k] ? k * 256 + tid : 0) * VEC);
    State st;
    st.init(init);
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
      if (chunk_ok[k]) {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          st.push(T(main_op(v[k].e[e], IdxT((k * 256 + tid) * VEC + e))), reduce_op);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      State got = shfl_xor_any(st, off);
      st.merge(got, reduce_op);
    }
    if (lane == 0) s_state[phase][warp] = st;
    __syncthreads();
    // every thread folds the eight warp results in the same order: the same norm everywhere
    State tot = s_state[phase][0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
      tot.merge(s_state[phase][w], reduce_op);
    const T norm = T(final_op(tot.value()));
    if (!(norm <= eps)) {
      T* dst = out + r * n_cols;
#pragma unroll
      for (int k = 0; k < CPT; ++k) {
        if (chunk_ok[k]) {
          VecOf<T, VEC> o;
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            o.e[e] = v[k].e[e] / norm;
          store_vec<T, VEC>(dst + int64_t(k * 256 + tid) * VEC, o);
        }
      }
    }
  }
}

template <typename T, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp, int VEC>
__global__ void __launch_bounds__(256) row_normalize_long_kernel(T* out,
                                                                const T* in,
                                                                int64_t n_rows,
                                                                int64_t n_cols,
                                                                T init,
                                                                T eps,
                                                                MainOp main_op,
                                                                ReduceOp reduce_op,
                                                                FinalOp final_op)
{
  grid_dep_sync();
  using State     = typename state_for<T, ReduceOp>::type;
  using Vec       = VecOf<T, VEC>;
  constexpr int Q = 4;  // loads in flight per thread
  __shared__ State s_state[8];
  __shared__ T s_norm;
  const int tid      = threadIdx.x;
  const int64_t nvec = n_cols / VEC;
  for (int64_t r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const T* src = in + r * n_cols;
    State st;
    st.init(init);
    for (int64_t c0 = tid; c0 < nvec; c0 += int64_t(Q) * 256) {
      Vec v[Q];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const int64_t c = c0 + int64_t(q) * 256;
        v[q]            = *reinterpret_cast<const Vec*>(src + (c < nvec ? c : c0) * VEC);  // cached: read again below
      }
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const int64_t c = c0 + int64_t(q) * 256;
        if (c < nvec) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            st.push(T(main_op(v[q].e[e], IdxT(c * VEC + e))), reduce_op);
        }
      }
    }
    st = block_merge(st, reduce_op, s_state);
    if (tid == 0) s_norm = T(final_op(st.value()));
    __syncthreads();
    const T norm = s_norm;
    if (!(norm <= eps)) {
      T* dst = out + r * n_cols;
      for (int64_t c0 = tid; c0 < nvec; c0 += int64_t(Q) * 256) {
        Vec v[Q];
#pragma unroll
        for (int q = 0; q < Q; ++q) {
          const int64_t c = c0 + int64_t(q) * 256;
          v[q]            = *reinterpret_cast<const Vec*>(src + (c < nvec ? c : c0) * VEC);
        }
#pragma unroll
        for (int q = 0; q < Q; ++q) {
          const int64_t c = c0 + int64_t(q) * 256;
          if (c < nvec) {
            Vec o;
#pragma unroll
            for (int e = 0; e < VEC; ++e)
              o.e[e] = v[q].e[e] / norm;
            store_vec<T, VEC>(dst + c * VEC, o);
          }
        }
      }
    }
    __syncthreads();  // s_state / s_norm are rewritten for the next row
  }
}

template <typename T, typename IdxT, typename MainOp, typename ReduceOp, typename FinalOp>
cudaError_t launch_row_normalize(T* out,
                                 const T* in,
                                 int64_t n_rows,
                                 int64_t n_cols,
                                 T init,
                                 T eps,
                                 MainOp main_op,
                                 ReduceOp reduce_op,
                                 FinalOp final_op,
                                 cudaStream_t stream,
                                 int* status = nullptr)
{
  if (n_rows <= 0 || n_cols <= 0) return cudaSuccess;
  constexpr int V16 = vec16<T>::value;
  const bool vec_ok = V16 > 1 && n_cols % V16 == 0 && aligned16(in) && aligned16(out);
  const int vec     = vec_ok ? V16 : 1;
  const int64_t nvec = n_cols / vec;
  const int sms      = sm_count();

  // Rows staged through shared memory in both directions (row_normalize_staged.cuh): rows that do not
  // start on 16-byte boundaries, and aligned rows whose vector count is no power of two (the lane groups
  // of the kernels below are), large matrices only.
  if constexpr (V16 > 1 && sizeof(T) >= 2) {
    const size_t row_bytes = size_t(n_cols) * sizeof(T);
    bool staged            = tuning().row_staged == 1 && aligned16(in) && aligned16(out) &&
                  n_cols <= tuning().row_staged_max &&
                  // measured with a cold L2: 64 MB for rows off the boundaries and short aligned rows, 256 MB
                  // for longer aligned rows (the direct kernels are better there to begin with)
                  size_t(n_rows) * row_bytes >= 2 * (size_t(vec_ok && n_cols > 64 ? tuning().row_staged_wide_min_kb
                                                                                   : tuning().row_staged_min_kb)
                                                     << 10);
    if (staged && vec_ok) {
      // measured: the direct kernels hold their own for powers of two and for 3 x 2^k vectors from 48 on
      const int mode       = tuning().row_staged_aligned;  // 1: by rule, 2: always, 3: never
      const bool pow2      = (nvec & (nvec - 1)) == 0;
      const bool three_2k  = nvec >= 48 && nvec % 3 == 0 && ((nvec / 3) & (nvec / 3 - 1)) == 0;
      staged = mode == 2 || (mode == 1 && !pow2 && !three_2k && n_cols <= tuning().row_staged_aligned_max);
    } else if (staged) {
      staged = row_bytes >= 12;  // one or two elements per row: nothing to gain
    }
    if (staged) {
      const StagedPlan sp = plan_staged_rows(n_rows, row_bytes, int(nvec), vec_ok);
      const size_t smem   = sp.smem + size_t(sp.stages) * size_t((sp.tile_rows + 31) / 32) * sizeof(unsigned);
      if (sp.ok && smem <= (size_t(108) << 10)) {
#define B2R_NORMALIZE_STAGED(VEC_)                                                                            \
  do {                                                                                                        \
    auto kern      = row_normalize_staged_kernel<T, IdxT, MainOp, ReduceOp, FinalOp, VEC_>;                   \
    cudaError_t ea = ensure_dynamic_smem(kern, smem);                                                         \
    if (ea != cudaSuccess) return ea;                                                                         \
    (void)launch_dep(kern, dim3(unsigned(sp.ctas)), dim3(kTmaThreads), smem, stream,                                  \
                     out, in, sp.n_main, int(n_cols), init, eps, main_op,                                             \
                                                          reduce_op, final_op, sp.G, sp.rot, int(sp.tile_rows), \
                                                          sp.rows_per_cta, sp.stages, ring_ctl(status));      \
  } while (0)
        if (vec_ok) {
          B2R_NORMALIZE_STAGED(V16);
        } else {
          B2R_NORMALIZE_STAGED(1);
        }
#undef B2R_NORMALIZE_STAGED
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess || sp.n_main == n_rows) return e;
        // the rows behind the last 16-byte boundary: the direct kernels
        return launch_row_normalize<T, IdxT, MainOp, ReduceOp, FinalOp>(out + sp.n_main * n_cols, in + sp.n_main * n_cols,
                                                                        n_rows - sp.n_main, n_cols, init, eps, main_op,
                                                                        reduce_op, final_op, stream, status);
      }
    }
  }

#define B2R_NORMALIZE_REG(VEC_, CPL_)                                                                     \
  do {                                                                                                    \
    constexpr int U_ = CPL_ >= 8 ? 1 : 8 / CPL_;                                                         \
    auto kern        = row_normalize_kernel<T, IdxT, MainOp, ReduceOp, FinalOp, VEC_, CPL_, U_>;          \
    static int occ   = resident_ctas(kern, 256, 0);                                                       \
    const unsigned g = next_pow2(unsigned(ceil_div<int64_t>(nvec, CPL_)));                                \
    const int G      = int(g > 32u ? 32u : g);                                                            \
    const int64_t rows_per_cta = int64_t(32 / G) * U_ * 8;                                                \
    int64_t ctas               = ceil_div<int64_t>(n_rows, rows_per_cta);                                 \
    (void)occ;                                                                                            \
    const int64_t cap = int64_t(sms) * (tuning().normalize_ctas_per_sm > 0 ? tuning().normalize_ctas_per_sm : 256); \
    if (ctas > cap) ctas = cap;                                                                           \
    (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(256), 0, stream,                                                \
                     out, in, n_rows, n_cols, init, eps, main_op, reduce_op,                                          \
                                             final_op, G);                                                \
  } while (0)
#define B2R_NORMALIZE_CTA(VEC_, CPT_)                                                                     \
  do {                                                                                                    \
    auto kern      = row_normalize_cta_kernel<T, IdxT, MainOp, ReduceOp, FinalOp, VEC_, CPT_>;            \
    static int occ = resident_ctas(kern, 256, 0);                                                         \
    int64_t ctas   = n_rows;                                                                              \
    (void)occ;                                                                                            \
    {                                                                                                     \
      const int64_t cap = int64_t(sms) * (tuning().normalize_ctas_per_sm > 0 ? tuning().normalize_ctas_per_sm : 256); \
      if (ctas > cap) ctas = cap;                                                                         \
    }                                                                                                     \
    (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(256), 0, stream,                                                \
                     out, in, n_rows, n_cols, init, eps, main_op, reduce_op,                                          \
                                             final_op);                                                   \
  } while (0)
#define B2R_NORMALIZE_ANY(VEC_)                                                                           \
  do {                                                                                                    \
    if (nvec > 4096) {                                                                                    \
      auto kern      = row_normalize_long_kernel<T, IdxT, MainOp, ReduceOp, FinalOp, VEC_>;               \
      static int occ = resident_ctas(kern, 256, 0);                                                       \
      int64_t ctas   = n_rows;                                                                            \
      if (ctas > int64_t(sms) * occ) ctas = int64_t(sms) * occ;                                           \
      (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(256), 0, stream,                                              \
                       out, in, n_rows, n_cols, init, eps, main_op, reduce_op,                                        \
                                               final_op);                                                 \
    } else if (nvec > 2048) {                                                                             \
      B2R_NORMALIZE_CTA(VEC_, 16);                                                                        \
    } else if (nvec > 1024) {                                                                             \
      B2R_NORMALIZE_CTA(VEC_, 8);                                                                         \
    } else if (nvec > 512) {                                                                              \
      B2R_NORMALIZE_CTA(VEC_, 4);                                                                         \
    } else if (nvec > 256) {                                                                              \
      B2R_NORMALIZE_REG(VEC_, 16);                                                                        \
    } else if (nvec > 128) {                                                                              \
      B2R_NORMALIZE_REG(VEC_, 8);                                                                         \
    } else if (nvec >= 32) {                                                                              \
      B2R_NORMALIZE_REG(VEC_, 4);                                                                         \
    } else if (nvec >= 8) {                                                                               \
      B2R_NORMALIZE_REG(VEC_, 2);                                                                         \
    } else {                                                                                              \
      B2R_NORMALIZE_REG(VEC_, 1);                                                                         \
    }                                                                                                     \
  } while (0)
  if (vec > 1) {
    B2R_NORMALIZE_ANY(V16);
  } else {
    B2R_NORMALIZE_ANY(1);
  }
#undef B2R_NORMALIZE_ANY
#undef B2R_NORMALIZE_CTA
#undef B2R_NORMALIZE_REG
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
