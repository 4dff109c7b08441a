// Internal glue of the C ABI: status bookkeeping and the typed dispatcher that maps a
// b2r_reduce_desc onto the kernel templates. Each capi_reduce_*.cu instantiates the
// dispatcher for one (input, output) type pair so the pairs compile in parallel.
#pragma once

#include <raft_b200.h>
#include <raft_b200/detail/launch.cuh>

namespace raft_b200 {
namespace capi {

int set_cuda_error(cudaError_t e);  // records e for b2r_last_cuda_error, returns B2R_ERR_CUDA / B2R_OK

// Device address of the library's kernel-status word on the CURRENT device (looked up once per device), or
// null if the lookup failed: ring kernels whose bounded wait ran out set it, b2r_last_kernel_status reads it.
int* kernel_status_word();

// A caller's workspace plus the status word, as the launchers take them.
inline detail::Workspace make_workspace(void* workspace, size_t workspace_bytes)
{
  detail::Workspace ws;
  ws.ptr    = workspace;
  ws.bytes  = workspace != nullptr ? workspace_bytes : 0;
  ws.status = kernel_status_word();
  return ws;
}

inline cudaStream_t to_stream(b2r_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Geometry of a reduce call once layout and apply are folded together
// (the same folding as the reference's linalg/detail/reduce.cuh:36-47).
struct ReduceGeometry {
  bool contiguous;   // reduce along the contiguous axis (row kernel) or the strided one
  int64_t n_out;     // number of outputs
  int64_t n_red;     // length of the reduced axis
};

inline ReduceGeometry geometry(const b2r_reduce_desc& d)
{
  const bool row_major  = d.layout == B2R_ROW_MAJOR;
  const bool along_rows = d.apply == B2R_ALONG_ROWS;
  ReduceGeometry g;
  g.contiguous = row_major == along_rows;
  g.n_out      = along_rows ? d.n_rows : d.n_cols;
  g.n_red      = along_rows ? d.n_cols : d.n_rows;
  return g;
}

template <typename InT, typename OutT, typename MainOp, typename ReduceOp, typename FinalOp>
int run_reduce(const b2r_reduce_desc& d,
               OutT* out,
               const InT* in,
               OutT init,
               MainOp main_op,
               ReduceOp reduce_op,
               FinalOp final_op,
               detail::Workspace ws,
               cudaStream_t stream)
{
  const ReduceGeometry g = geometry(d);
  cudaError_t e;
  if (g.contiguous) {
    e = detail::launch_row_reduce<InT, OutT, int64_t>(
      out, in, g.n_out, g.n_red, g.n_red, init, d.inplace != 0, main_op, reduce_op, final_op, stream, ws);
  } else {
    e = detail::launch_col_reduce<InT, OutT, int64_t>(
      out, in, g.n_red, g.n_out, g.n_out, init, d.inplace != 0, main_op, reduce_op, final_op, stream, ws);
  }
  return set_cuda_error(e);
}

template <typename InT, typename OutT, typename ReduceOp>
size_t reduce_workspace(const b2r_reduce_desc& d, const InT* in)
{
  const ReduceGeometry g = geometry(d);
  if (g.n_out <= 0) return 0;
  if (g.contiguous) {
    using CarryT = typename detail::state_for<OutT, ReduceOp>::type::carry_t;
    return detail::row_reduce_scratch_bytes<CarryT>(g.n_out, g.n_red, sizeof(InT), nullptr);
  }
  return detail::col_reduce_scratch_bytes<InT, OutT, ReduceOp>(in, g.n_red, g.n_out, g.n_out);
}

// Scalar (non key/value) outputs: main in {identity, sq, abs, nz} x reduce in {add, min, max}.
template <typename InT, typename OutT>
int reduce_scalar(const b2r_reduce_desc& d, void* out_v, const void* in_v, detail::Workspace ws, cudaStream_t stream)
{
  OutT* out      = static_cast<OutT*>(out_v);
  const InT* in  = static_cast<const InT*>(in_v);
  OutT init      = std::is_floating_point<OutT>::value ? OutT(d.init) : OutT(d.init_i);
  op::RuntimeFinal<OutT> fin{d.final_op, OutT(d.final_scalar)};
  if (d.final_op < B2R_FINAL_IDENTITY || d.final_op > B2R_FINAL_ABS) return B2R_ERR_BAD_ARG;
  if (d.final_op == B2R_FINAL_SQRT && !std::is_floating_point<OutT>::value) return B2R_ERR_UNSUPPORTED;
#define B2R_CASE(MAIN_ENUM, MAIN_T, RED_T) \
  case MAIN_ENUM: return run_reduce<InT, OutT>(d, out, in, init, MAIN_T{}, RED_T{}, fin, ws, stream)
  switch (d.reduce_op) {
    case B2R_REDUCE_ADD:
      switch (d.main_op) {
        B2R_CASE(B2R_MAIN_IDENTITY, op::Identity, op::Add);
        B2R_CASE(B2R_MAIN_SQ, op::Square, op::Add);
        B2R_CASE(B2R_MAIN_ABS, op::Abs, op::Add);
        B2R_CASE(B2R_MAIN_NZ, op::NonZero, op::Add);
        default: return B2R_ERR_UNSUPPORTED;
      }
    case B2R_REDUCE_MIN:
      switch (d.main_op) {
        B2R_CASE(B2R_MAIN_IDENTITY, op::Identity, op::Min);
        B2R_CASE(B2R_MAIN_ABS, op::Abs, op::Min);
        default: return B2R_ERR_UNSUPPORTED;
      }
    case B2R_REDUCE_MAX:
      switch (d.main_op) {
        B2R_CASE(B2R_MAIN_IDENTITY, op::Identity, op::Max);
        B2R_CASE(B2R_MAIN_ABS, op::Abs, op::Max);
        default: return B2R_ERR_UNSUPPORTED;
      }
    default: return B2R_ERR_UNSUPPORTED;
  }
#undef B2R_CASE
}

template <typename InT, typename OutT>
size_t reduce_scalar_workspace(const b2r_reduce_desc& d, const void* in)
{
  if (d.reduce_op == B2R_REDUCE_ADD)
    return reduce_workspace<InT, OutT, op::Add>(d, static_cast<const InT*>(in));
  return reduce_workspace<InT, OutT, op::Min>(d, static_cast<const InT*>(in));
}

// Key/value outputs: main = to_kvp, reduce in {argmin, argmax}, contiguous axis only.
template <typename InT>
int reduce_kvp(const b2r_reduce_desc& d, void* out_v, const void* in_v, detail::Workspace ws, cudaStream_t stream)
{
  using KV = KeyValue<int, InT>;
  static_assert(sizeof(KV) == sizeof(int) + sizeof(InT) || sizeof(KV) == 2 * sizeof(int) ||
                  sizeof(KV) == 16,
                "unexpected key/value layout");
  if (d.main_op != B2R_MAIN_TO_KVP) return B2R_ERR_UNSUPPORTED;
  if (d.final_op != B2R_FINAL_IDENTITY) return B2R_ERR_UNSUPPORTED;
  if (!geometry(d).contiguous) return B2R_ERR_UNSUPPORTED;  // as linalg/strided_reduction.cuh:70-77
  KV init;
  init.key   = int(d.init_key);
  init.value = std::is_floating_point<InT>::value ? InT(d.init) : InT(d.init_i);
  KV* out       = static_cast<KV*>(out_v);
  const InT* in = static_cast<const InT*>(in_v);
  switch (d.reduce_op) {
    case B2R_REDUCE_ARGMIN:
      return run_reduce<InT, KV>(d, out, in, init, op::ToKeyValue<int>{}, op::ArgMin{}, op::Identity{}, ws, stream);
    case B2R_REDUCE_ARGMAX:
      return run_reduce<InT, KV>(d, out, in, init, op::ToKeyValue<int>{}, op::ArgMax{}, op::Identity{}, ws, stream);
    default: return B2R_ERR_UNSUPPORTED;
  }
}

template <typename InT>
size_t reduce_kvp_workspace(const b2r_reduce_desc& d, const void* in)
{
  return reduce_workspace<InT, KeyValue<int, InT>, op::ArgMin>(d, static_cast<const InT*>(in));
}

// one translation unit per type pair
int reduce_f32_f32(const b2r_reduce_desc&, void*, const void*, detail::Workspace, cudaStream_t);
int reduce_f64_f64(const b2r_reduce_desc&, void*, const void*, detail::Workspace, cudaStream_t);
int reduce_f32_f64(const b2r_reduce_desc&, void*, const void*, detail::Workspace, cudaStream_t);
int reduce_f16_f32(const b2r_reduce_desc&, void*, const void*, detail::Workspace, cudaStream_t);
int reduce_i32_i32(const b2r_reduce_desc&, void*, const void*, detail::Workspace, cudaStream_t);
int reduce_kvp_any(const b2r_reduce_desc&, void*, const void*, detail::Workspace, cudaStream_t);
size_t ws_f32_f32(const b2r_reduce_desc&, const void*);
size_t ws_f64_f64(const b2r_reduce_desc&, const void*);
size_t ws_f32_f64(const b2r_reduce_desc&, const void*);
size_t ws_f16_f32(const b2r_reduce_desc&, const void*);
size_t ws_i32_i32(const b2r_reduce_desc&, const void*);
size_t ws_kvp_any(const b2r_reduce_desc&, const void*);

}  // namespace capi
}  // namespace raft_b200
