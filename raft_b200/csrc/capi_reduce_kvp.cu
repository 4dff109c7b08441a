// C-ABI reduce instantiations for key/value (argmin / argmax) outputs.
#include "capi_internal.cuh"

namespace raft_b200 {
namespace capi {

int reduce_kvp_any(const b2r_reduce_desc& d, void* out, const void* in, detail::Workspace ws, cudaStream_t s)
{
  if (d.in_dtype == B2R_F32 && d.out_dtype == B2R_KVP_I32_F32) return reduce_kvp<float>(d, out, in, ws, s);
  if (d.in_dtype == B2R_F64 && d.out_dtype == B2R_KVP_I32_F64) return reduce_kvp<double>(d, out, in, ws, s);
  if (d.in_dtype == B2R_I16 && d.out_dtype == B2R_KVP_I32_I16) return reduce_kvp<short>(d, out, in, ws, s);
  if (d.in_dtype == B2R_I32 && d.out_dtype == B2R_KVP_I32_I32) return reduce_kvp<int>(d, out, in, ws, s);
  return B2R_ERR_UNSUPPORTED;
}

size_t ws_kvp_any(const b2r_reduce_desc& d, const void* in)
{
  if (d.in_dtype == B2R_F32) return reduce_kvp_workspace<float>(d, in);
  if (d.in_dtype == B2R_F64) return reduce_kvp_workspace<double>(d, in);
  if (d.in_dtype == B2R_I16) return reduce_kvp_workspace<short>(d, in);
  if (d.in_dtype == B2R_I32) return reduce_kvp_workspace<int>(d, in);
  return 0;
}

}  // namespace capi
}  // namespace raft_b200
