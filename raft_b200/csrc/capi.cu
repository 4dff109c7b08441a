// C ABI entry points: argument validation, dtype dispatch, status reporting, and the two
// small elementwise kernels of the boundary (deferred final_op, synthetic data generator).
#include "capi_internal.cuh"

#include <raft_b200/detail/cols_by_key.cuh>
#include <raft_b200/detail/rows_by_key.cuh>
#include <raft_b200/detail/synth.cuh>

#include <mutex>

namespace raft_b200 {
namespace capi {

static thread_local int g_last_cuda_error = 0;

// One status word per device (a __device__ variable exists once on every device that loads the library).
// In host code its name is only a handle: the address the kernels get comes from cudaGetSymbolAddress.
static __device__ int g_kernel_status;
static std::mutex g_status_mutex;
static int* g_status_ptr[64]    = {};
static bool g_status_tried[64]  = {};

int* kernel_status_word()
{
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_tried[dev]) {
    g_status_tried[dev] = true;
    void* p             = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_status) == cudaSuccess) {
      g_status_ptr[dev] = static_cast<int*>(p);
    } else {
      (void)cudaGetLastError();
    }
  }
  return g_status_ptr[dev];
}

int set_cuda_error(cudaError_t e)
{
  if (e == cudaSuccess) return B2R_OK;
  g_last_cuda_error = int(e);
  (void)cudaGetLastError();  // clear the sticky launch error, as the reference's RAFT_CUDA_TRY does
  return B2R_ERR_CUDA;
}

static bool is_kvp(int32_t dt) { return dt >= B2R_KVP_I32_F32 && dt <= B2R_KVP_I32_I32; }

static int check_desc(const b2r_reduce_desc* d, const void* out, const void* in)
{
  if (d == nullptr) return B2R_ERR_BAD_ARG;
  if (d->n_rows < 0 || d->n_cols < 0) return B2R_ERR_BAD_ARG;
  if (d->layout != B2R_ROW_MAJOR && d->layout != B2R_COL_MAJOR) return B2R_ERR_BAD_ARG;
  if (d->apply != B2R_ALONG_ROWS && d->apply != B2R_ALONG_COLUMNS) return B2R_ERR_BAD_ARG;
  const ReduceGeometry g = geometry(*d);
  if (g.n_out > 0 && out == nullptr) return B2R_ERR_BAD_ARG;
  if (g.n_out > 0 && g.n_red > 0 && in == nullptr) return B2R_ERR_BAD_ARG;
  return B2R_OK;
}

template <typename T>
__global__ void apply_final_kernel(T* v, int64_t n, op::RuntimeFinal<T> fin)
{
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) v[i] = fin(v[i]);
}

template <typename T>
static int apply_final_typed(void* v, int64_t n, int32_t final_op, double scalar, cudaStream_t s)
{
  if (final_op == B2R_FINAL_IDENTITY || n == 0) return B2R_OK;
  op::RuntimeFinal<T> fin{final_op, T(scalar)};
  apply_final_kernel<T><<<unsigned((n + 255) / 256), 256, 0, s>>>(static_cast<T*>(v), n, fin);
  return set_cuda_error(cudaGetLastError());
}

template <typename DataT, typename KeyT>
static int rows_by_key_typed(void* sums, int64_t* counts, const void* A, int64_t lda, const void* keys,
                             const void* weights, int64_t nrows, int64_t ncols, int64_t nkeys, bool reset,
                             detail::Workspace ws, cudaStream_t s)
{
  return set_cuda_error(detail::launch_rows_by_key<DataT, KeyT, DataT, DataT>(
    static_cast<DataT*>(sums), reinterpret_cast<long long*>(counts), static_cast<const DataT*>(A), lda,
    static_cast<const KeyT*>(keys), static_cast<const DataT*>(weights), nrows, ncols, nkeys, reset, s, ws));
}

template <typename T, typename KeyT>
static int cols_by_key_typed(void* out, const void* data, const void* keys, int64_t nrows, int64_t ncols,
                             int64_t nkeys, bool reset, detail::Workspace ws, cudaStream_t s)
{
  return set_cuda_error(detail::launch_cols_by_key<T, KeyT>(
    static_cast<T*>(out), static_cast<const T*>(data), static_cast<const KeyT*>(keys), nrows, ncols, nkeys,
    reset, s, ws));
}

}  // namespace capi
}  // namespace raft_b200

using namespace raft_b200;
using namespace raft_b200::capi;

extern "C" {

int b2r_reduce(const b2r_reduce_desc* desc, void* out, const void* in, void* workspace,
               size_t workspace_bytes, b2r_stream_t stream)
{
  const int chk = check_desc(desc, out, in);
  if (chk != B2R_OK) return chk;
  const b2r_reduce_desc& d = *desc;
  const detail::Workspace ws = make_workspace(workspace, workspace_bytes);
  cudaStream_t s   = to_stream(stream);
  if (is_kvp(d.out_dtype)) return reduce_kvp_any(d, out, in, ws, s);
  if (d.main_op == B2R_MAIN_TO_KVP || d.reduce_op == B2R_REDUCE_ARGMIN || d.reduce_op == B2R_REDUCE_ARGMAX)
    return B2R_ERR_UNSUPPORTED;
  if (d.in_dtype == B2R_F32 && d.out_dtype == B2R_F32) return reduce_f32_f32(d, out, in, ws, s);
  if (d.in_dtype == B2R_F64 && d.out_dtype == B2R_F64) return reduce_f64_f64(d, out, in, ws, s);
  if (d.in_dtype == B2R_F32 && d.out_dtype == B2R_F64) return reduce_f32_f64(d, out, in, ws, s);
  if (d.in_dtype == B2R_F16 && d.out_dtype == B2R_F32) return reduce_f16_f32(d, out, in, ws, s);
  if (d.in_dtype == B2R_I32 && d.out_dtype == B2R_I32) return reduce_i32_i32(d, out, in, ws, s);
  return B2R_ERR_UNSUPPORTED;
}

size_t b2r_reduce_workspace_bytes(const b2r_reduce_desc* desc, const void* in)
{
  if (desc == nullptr || desc->n_rows < 0 || desc->n_cols < 0) return 0;
  const b2r_reduce_desc& d = *desc;
  if (is_kvp(d.out_dtype)) return ws_kvp_any(d, in);
  if (d.in_dtype == B2R_F32 && d.out_dtype == B2R_F32) return ws_f32_f32(d, in);
  if (d.in_dtype == B2R_F64 && d.out_dtype == B2R_F64) return ws_f64_f64(d, in);
  if (d.in_dtype == B2R_F32 && d.out_dtype == B2R_F64) return ws_f32_f64(d, in);
  if (d.in_dtype == B2R_F16 && d.out_dtype == B2R_F32) return ws_f16_f32(d, in);
  if (d.in_dtype == B2R_I32 && d.out_dtype == B2R_I32) return ws_i32_i32(d, in);
  return 0;
}

int b2r_norm(int32_t norm_type, int32_t apply, int32_t layout, int32_t in_dtype, int32_t out_dtype,
             int64_t n_rows, int64_t n_cols, int32_t final_op, double final_scalar, void* out, const void* in,
             void* workspace, size_t workspace_bytes, b2r_stream_t stream)
{
  b2r_reduce_desc d = {};
  d.in_dtype        = in_dtype;
  d.out_dtype       = out_dtype;
  d.layout          = layout;
  d.apply           = apply;
  d.n_rows          = n_rows;
  d.n_cols          = n_cols;
  d.final_op        = final_op;
  d.final_scalar    = final_scalar;
  d.inplace         = 0;
  d.init            = 0.0;
  d.init_i          = 0;
  switch (norm_type) {
    case B2R_NORM_L1:
      d.main_op   = B2R_MAIN_ABS;
      d.reduce_op = B2R_REDUCE_ADD;
      break;
    case B2R_NORM_L2:
      d.main_op   = B2R_MAIN_SQ;
      d.reduce_op = B2R_REDUCE_ADD;
      break;
    case B2R_NORM_LINF:
      d.main_op   = B2R_MAIN_ABS;
      d.reduce_op = B2R_REDUCE_MAX;
      break;
    default: return B2R_ERR_UNSUPPORTED;  // L0: the reference throws (linalg/detail/norm.cuh:36,59)
  }
  return b2r_reduce(&d, out, in, workspace, workspace_bytes, stream);
}

int b2r_reduce_rows_by_key(void* sums, int64_t* counts, const void* A, int64_t lda, const void* keys,
                           const void* weights, int32_t data_dtype, int32_t key_dtype, int64_t nrows,
                           int64_t ncols, int64_t nkeys, int32_t reset, void* workspace,
                           size_t workspace_bytes, b2r_stream_t stream)
{
  if (nrows < 0 || ncols < 0 || nkeys < 0 || lda < ncols) return B2R_ERR_BAD_ARG;
  if (ncols > 0 && nkeys > 0 && sums == nullptr) return B2R_ERR_BAD_ARG;
  if (nrows > 0 && ncols > 0 && (A == nullptr || keys == nullptr)) return B2R_ERR_BAD_ARG;
  const detail::Workspace ws = make_workspace(workspace, workspace_bytes);
  cudaStream_t s = to_stream(stream);
  const bool rs  = reset != 0;
#define B2R_RBK(DT, KT) \
  return rows_by_key_typed<DT, KT>(sums, counts, A, lda, keys, weights, nrows, ncols, nkeys, rs, ws, s)
  if (data_dtype == B2R_F32) {
    if (key_dtype == B2R_I32) B2R_RBK(float, int);
    if (key_dtype == B2R_U32) B2R_RBK(float, unsigned);
    if (key_dtype == B2R_I64) B2R_RBK(float, long long);
  } else if (data_dtype == B2R_F64) {
    if (key_dtype == B2R_I32) B2R_RBK(double, int);
    if (key_dtype == B2R_U32) B2R_RBK(double, unsigned);
    if (key_dtype == B2R_I64) B2R_RBK(double, long long);
  }
#undef B2R_RBK
  return B2R_ERR_UNSUPPORTED;
}

size_t b2r_reduce_rows_by_key_workspace_bytes(const void* A, int64_t lda, int32_t data_dtype, int64_t nrows,
                                              int64_t ncols, int64_t nkeys)
{
  if (data_dtype == B2R_F32)
    return detail::rows_by_key_scratch_bytes<float, float>(static_cast<const float*>(A), lda, nrows, ncols, nkeys);
  if (data_dtype == B2R_F64)
    return detail::rows_by_key_scratch_bytes<double, double>(static_cast<const double*>(A), lda, nrows, ncols, nkeys);
  return 0;
}

int b2r_reduce_cols_by_key(void* out, const void* data, const void* keys, int32_t dtype, int32_t key_dtype,
                           int64_t nrows, int64_t ncols, int64_t nkeys, int32_t reset, void* workspace,
                           size_t workspace_bytes, b2r_stream_t stream)
{
  if (nrows < 0 || ncols < 0 || nkeys < 0) return B2R_ERR_BAD_ARG;
  if (nrows > 0 && nkeys > 0 && out == nullptr) return B2R_ERR_BAD_ARG;
  if (nrows > 0 && ncols > 0 && (data == nullptr || keys == nullptr)) return B2R_ERR_BAD_ARG;
  const detail::Workspace ws = make_workspace(workspace, workspace_bytes);
  cudaStream_t s = to_stream(stream);
  const bool rs  = reset != 0;
#define B2R_CBK(DT, KT) return cols_by_key_typed<DT, KT>(out, data, keys, nrows, ncols, nkeys, rs, ws, s)
  if (dtype == B2R_F32) {
    if (key_dtype == B2R_I32) B2R_CBK(float, int);
    if (key_dtype == B2R_U32) B2R_CBK(float, unsigned);
    if (key_dtype == B2R_I64) B2R_CBK(float, long long);
  } else if (dtype == B2R_F64) {
    if (key_dtype == B2R_I32) B2R_CBK(double, int);
    if (key_dtype == B2R_U32) B2R_CBK(double, unsigned);
    if (key_dtype == B2R_I64) B2R_CBK(double, long long);
  }
#undef B2R_CBK
  return B2R_ERR_UNSUPPORTED;
}

size_t b2r_reduce_cols_by_key_workspace_bytes(const void* data, int32_t dtype, int64_t nrows, int64_t ncols,
                                              int64_t nkeys)
{
  if (nrows <= 0 || ncols <= 0 || nkeys <= 0) return 0;
  if (dtype == B2R_F32) return detail::cols_by_key_scratch_bytes<float>(static_cast<const float*>(data), nrows, ncols, nkeys);
  if (dtype == B2R_F64) return detail::cols_by_key_scratch_bytes<double>(static_cast<const double*>(data), nrows, ncols, nkeys);
  return 0;
}

int b2r_last_kernel_status(int32_t* status_out, int32_t clear)
{
  if (status_out == nullptr) return B2R_ERR_BAD_ARG;
  int* word = kernel_status_word();
  if (word == nullptr) return set_cuda_error(cudaErrorInvalidSymbol);
  int v         = 0;
  cudaError_t e = cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && clear != 0 && v != 0) e = cudaMemset(word, 0, sizeof(int));
  if (e != cudaSuccess) return set_cuda_error(e);
  *status_out = v != 0 ? B2R_ERR_TIMEOUT : B2R_OK;
  return B2R_OK;
}

int b2r_set_wait_limit_ms(uint32_t ms)
{
  detail::wait_limit_override_ms().store(ms, std::memory_order_relaxed);  // 0: back to the knob / default
  return B2R_OK;
}

int b2r_apply_final(void* v, int32_t dtype, int64_t n, int32_t final_op, double final_scalar, b2r_stream_t stream)
{
  if (n < 0 || (n > 0 && v == nullptr)) return B2R_ERR_BAD_ARG;
  if (final_op < B2R_FINAL_IDENTITY || final_op > B2R_FINAL_ABS) return B2R_ERR_BAD_ARG;
  cudaStream_t s = to_stream(stream);
  switch (dtype) {
    case B2R_F32: return apply_final_typed<float>(v, n, final_op, final_scalar, s);
    case B2R_F64: return apply_final_typed<double>(v, n, final_op, final_scalar, s);
    case B2R_I32:
      if (final_op == B2R_FINAL_SQRT) return B2R_ERR_UNSUPPORTED;
      return apply_final_typed<int>(v, n, final_op, final_scalar, s);
    default: return B2R_ERR_UNSUPPORTED;
  }
}

int b2r_synth_fill(void* dst, int32_t dtype, int64_t n, int64_t first_index, uint64_t seed, int32_t kind,
                   double lo, double hi, b2r_stream_t stream)
{
  if (n < 0 || (n > 0 && dst == nullptr) || kind < 0 || kind > 2) return B2R_ERR_BAD_ARG;
  if (n == 0) return B2R_OK;
  cudaStream_t s = to_stream(stream);
  cudaError_t e;
  switch (dtype) {
    case B2R_F32: e = synth::launch_fill<float>(static_cast<float*>(dst), n, first_index, seed, kind, lo, hi, s); break;
    case B2R_F64: e = synth::launch_fill<double>(static_cast<double*>(dst), n, first_index, seed, kind, lo, hi, s); break;
    case B2R_F16:
      if (kind == 2) return B2R_ERR_UNSUPPORTED;
      e = synth::launch_fill<__half>(static_cast<__half*>(dst), n, first_index, seed, kind, lo, hi, s);
      break;
    case B2R_I32:
      if (kind != 2) return B2R_ERR_UNSUPPORTED;
      e = synth::launch_fill<int>(static_cast<int*>(dst), n, first_index, seed, kind, lo, hi, s);
      break;
    case B2R_U32:
      if (kind != 2) return B2R_ERR_UNSUPPORTED;
      e = synth::launch_fill<unsigned>(static_cast<unsigned*>(dst), n, first_index, seed, kind, lo, hi, s);
      break;
    case B2R_I64:
      if (kind != 2) return B2R_ERR_UNSUPPORTED;
      e = synth::launch_fill<long long>(static_cast<long long*>(dst), n, first_index, seed, kind, lo, hi, s);
      break;
    case B2R_I16:
      if (kind != 2) return B2R_ERR_UNSUPPORTED;
      e = synth::launch_fill<short>(static_cast<short*>(dst), n, first_index, seed, kind, lo, hi, s);
      break;
    default: return B2R_ERR_UNSUPPORTED;
  }
  return set_cuda_error(e);
}

int b2r_trim_scratch_pool(void)
{
  cudaMemPool_t pool = detail::scratch_pool();
  if (pool == nullptr) return B2R_OK;
  return set_cuda_error(cudaMemPoolTrimTo(pool, 0));
}

int b2r_reload_tuning(void)
{
  detail::reload_tuning();
  return B2R_OK;
}

const char* b2r_status_string(int status)
{
  switch (status) {
    case B2R_OK: return "ok";
    case B2R_ERR_BAD_ARG: return "bad argument";
    case B2R_ERR_UNSUPPORTED: return "unsupported dtype / operator combination";
    case B2R_ERR_CUDA: return "CUDA runtime error (see b2r_last_cuda_error)";
    case B2R_ERR_TOO_LARGE: return "size beyond the limit of this entry point";
    case B2R_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out";
    default: return "unknown status";
  }
}

int b2r_last_cuda_error(void) { return g_last_cuda_error; }

const char* b2r_version(void) { return "raft_b200 0.1 (sm_100a)"; }

}  // extern "C"
