// Bridge between the raft::linalg function templates and the B200 kernels.
//
//  * functor types an enum can name (raft::identity_op, sq_op, abs_op, nz_op; add_op, min_op,
//    max_op; identity_op, sqrt_op, abs_op, mul_const_op, div_const_op) with an (input, output) type
//    pair the shared library was built for  ->  one call into the C ABI (include/raft_b200.h),
//    i.e. the precompiled sm_100a kernels;
//  * anything else (device lambdas, user structs, key/value taggers)  ->  the same kernel
//    templates of raft_b200/detail, instantiated in the caller's translation unit.
// Status codes come back as the reference's exception types.
#pragma once

#include <raft/core/error.hpp>
#include <raft/core/kvp.hpp>
#include <raft/core/operators.hpp>

#include <raft_b200.h>
#include <raft_b200/detail/cols_by_key.cuh>
#include <raft_b200/detail/launch.cuh>
#include <raft_b200/detail/rows_by_key.cuh>

#include <type_traits>

namespace raft_b200 {
namespace detail {
// raft::add_op reductions on floating-point outputs take the wide / compensated sum states
template <>
struct is_sum_op<raft::add_op> : std::true_type {};
}  // namespace detail
}  // namespace raft_b200

namespace raft {
namespace linalg {
namespace b200 {

inline void check(int status, const char* what)
{
  if (status == B2R_OK) return;
  if (status == B2R_ERR_BAD_ARG) throw raft::logic_error(std::string(what) + ": " + b2r_status_string(status));
  if (status == B2R_ERR_CUDA) {
    const cudaError_t e = static_cast<cudaError_t>(b2r_last_cuda_error());
    throw raft::cuda_error(std::string(what) + ": CUDA error " + cudaGetErrorName(e) + " " + cudaGetErrorString(e));
  }
  throw raft::exception(std::string(what) + ": " + b2r_status_string(status));
}

inline void check_cuda(cudaError_t e, const char* what)
{
  if (e == cudaSuccess) return;
  (void)cudaGetLastError();
  throw raft::cuda_error(std::string(what) + ": CUDA error " + cudaGetErrorName(e) + " " + cudaGetErrorString(e));
}

// ---- type -> enum tables ---------------------------------------------------------------------
template <typename T>
struct dtype_of : std::integral_constant<int, -1> {};
template <>
struct dtype_of<float> : std::integral_constant<int, B2R_F32> {};
template <>
struct dtype_of<double> : std::integral_constant<int, B2R_F64> {};
template <>
struct dtype_of<__half> : std::integral_constant<int, B2R_F16> {};
template <>
struct dtype_of<int> : std::integral_constant<int, B2R_I32> {};
template <>
struct dtype_of<unsigned> : std::integral_constant<int, B2R_U32> {};
template <>
struct dtype_of<long long> : std::integral_constant<int, B2R_I64> {};
template <>
struct dtype_of<long> : std::integral_constant<int, sizeof(long) == 8 ? B2R_I64 : B2R_I32> {};

template <typename In, typename Out>
struct abi_pair
  : std::integral_constant<bool,
                           (std::is_same<In, float>::value && std::is_same<Out, float>::value) ||
                             (std::is_same<In, double>::value && std::is_same<Out, double>::value) ||
                             (std::is_same<In, float>::value && std::is_same<Out, double>::value) ||
                             (std::is_same<In, __half>::value && std::is_same<Out, float>::value) ||
                             (std::is_same<In, int>::value && std::is_same<Out, int>::value)> {};

template <typename F>
struct main_enum : std::integral_constant<int, -1> {};
template <>
struct main_enum<raft::identity_op> : std::integral_constant<int, B2R_MAIN_IDENTITY> {};
template <>
struct main_enum<raft::sq_op> : std::integral_constant<int, B2R_MAIN_SQ> {};
template <>
struct main_enum<raft::abs_op> : std::integral_constant<int, B2R_MAIN_ABS> {};
template <>
struct main_enum<raft::nz_op> : std::integral_constant<int, B2R_MAIN_NZ> {};

template <typename F>
struct reduce_enum : std::integral_constant<int, -1> {};
template <>
struct reduce_enum<raft::add_op> : std::integral_constant<int, B2R_REDUCE_ADD> {};
template <>
struct reduce_enum<raft::min_op> : std::integral_constant<int, B2R_REDUCE_MIN> {};
template <>
struct reduce_enum<raft::max_op> : std::integral_constant<int, B2R_REDUCE_MAX> {};

template <typename F>
struct final_enum : std::integral_constant<int, -1> {
  static double scalar(const F&) { return 1.0; }
};
template <>
struct final_enum<raft::identity_op> : std::integral_constant<int, B2R_FINAL_IDENTITY> {
  static double scalar(const raft::identity_op&) { return 1.0; }
};
template <>
struct final_enum<raft::sqrt_op> : std::integral_constant<int, B2R_FINAL_SQRT> {
  static double scalar(const raft::sqrt_op&) { return 1.0; }
};
template <>
struct final_enum<raft::abs_op> : std::integral_constant<int, B2R_FINAL_ABS> {
  static double scalar(const raft::abs_op&) { return 1.0; }
};
template <typename T>
struct final_enum<raft::plug_const_op<T, raft::mul_op>> : std::integral_constant<int, B2R_FINAL_MUL_CONST> {
  static double scalar(const raft::plug_const_op<T, raft::mul_op>& f) { return double(f.c); }
};
template <typename T>
struct final_enum<raft::plug_const_op<T, raft::div_op>> : std::integral_constant<int, B2R_FINAL_DIV_CONST> {
  static double scalar(const raft::plug_const_op<T, raft::div_op>& f) { return double(f.c); }
};

// the min/max combinations the library carries (main_op identity or abs)
template <int MainE, int ReduceE>
struct combo_built
  : std::integral_constant<bool,
                           (ReduceE == B2R_REDUCE_ADD && MainE >= 0) ||
                             ((ReduceE == B2R_REDUCE_MIN || ReduceE == B2R_REDUCE_MAX) &&
                              (MainE == B2R_MAIN_IDENTITY || MainE == B2R_MAIN_ABS))> {};

// ---- reduce ----------------------------------------------------------------------------------
// D = number of columns, N = number of rows (the convention of raft::linalg::reduce).
template <bool rowMajor,
          bool alongRows,
          typename InType,
          typename OutType,
          typename IdxType,
          typename MainLambda,
          typename ReduceLambda,
          typename FinalLambda>
void reduce(OutType* dots,
            const InType* data,
            IdxType D,
            IdxType N,
            OutType init,
            cudaStream_t stream,
            bool inplace,
            MainLambda main_op,
            ReduceLambda reduce_op,
            FinalLambda final_op)
{
  constexpr int mainE  = main_enum<MainLambda>::value;
  constexpr int redE   = reduce_enum<ReduceLambda>::value;
  constexpr int finE   = final_enum<FinalLambda>::value;
  constexpr bool named = mainE >= 0 && redE >= 0 && finE >= 0 && combo_built<mainE, redE>::value &&
                         abi_pair<InType, OutType>::value &&
                         !(finE == B2R_FINAL_SQRT && !std::is_floating_point<OutType>::value);
  const int64_t n_out = alongRows ? int64_t(N) : int64_t(D);
  const int64_t n_red = alongRows ? int64_t(D) : int64_t(N);
  if constexpr (named) {
    b2r_reduce_desc d = {};
    d.in_dtype        = dtype_of<InType>::value;
    d.out_dtype       = dtype_of<OutType>::value;
    d.layout          = rowMajor ? B2R_ROW_MAJOR : B2R_COL_MAJOR;
    d.apply           = alongRows ? B2R_ALONG_ROWS : B2R_ALONG_COLUMNS;
    d.n_rows          = int64_t(N);
    d.n_cols          = int64_t(D);
    d.main_op         = mainE;
    d.reduce_op       = redE;
    d.final_op        = finE;
    d.inplace         = inplace ? 1 : 0;
    d.init            = double(init);
    d.init_i          = std::is_integral<OutType>::value ? static_cast<long long>(init) : 0;
    d.final_scalar    = final_enum<FinalLambda>::scalar(final_op);
    check(b2r_reduce(&d, dots, data, nullptr, 0, reinterpret_cast<b2r_stream_t>(stream)), "raft::linalg::reduce");
  } else {
    constexpr bool contiguous = rowMajor == alongRows;
    if constexpr (contiguous) {
      check_cuda(raft_b200::detail::launch_row_reduce<InType, OutType, IdxType>(
                   dots, data, n_out, n_red, n_red, init, inplace, main_op, reduce_op, final_op, stream),
                 "raft::linalg::reduce");
    } else {
      check_cuda(raft_b200::detail::launch_col_reduce<InType, OutType, IdxType>(
                   dots, data, n_red, n_out, n_out, init, inplace, main_op, reduce_op, final_op, stream),
                 "raft::linalg::reduce");
    }
  }
}

// ---- by key ----------------------------------------------------------------------------------
template <typename DataT, typename KeyT, typename WeightT, typename SumsT, typename IdxT>
void reduce_rows_by_key(const DataT* d_A,
                        IdxT lda,
                        const KeyT* d_keys,
                        const WeightT* d_weights,
                        IdxT nrows,
                        IdxT ncols,
                        IdxT nkeys,
                        SumsT* d_sums,
                        cudaStream_t stream,
                        bool reset_sums)
{
  check_cuda(raft_b200::detail::launch_rows_by_key<DataT, KeyT, WeightT, SumsT>(
               d_sums, nullptr, d_A, int64_t(lda), d_keys, d_weights, int64_t(nrows), int64_t(ncols), int64_t(nkeys),
               reset_sums, stream),
             "raft::linalg::reduce_rows_by_key");
}

template <typename T, typename KeyT, typename IdxT>
void reduce_cols_by_key(
  const T* data, const KeyT* keys, T* out, IdxT nrows, IdxT ncols, IdxT nkeys, cudaStream_t stream, bool reset_sums)
{
  check_cuda(raft_b200::detail::launch_cols_by_key<T, KeyT>(
               out, data, keys, int64_t(nrows), int64_t(ncols), int64_t(nkeys), reset_sums, stream),
             "raft::linalg::reduce_cols_by_key");
}

}  // namespace b200
}  // namespace linalg
}  // namespace raft
