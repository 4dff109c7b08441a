// C-ABI reduce instantiations for __half input -> float output.
#include "capi_internal.cuh"

namespace raft_b200 {
namespace capi {

int reduce_f16_f32(const b2r_reduce_desc& d, void* out, const void* in, detail::Workspace ws, cudaStream_t s)
{
  return reduce_scalar<__half, float>(d, out, in, ws, s);
}

size_t ws_f16_f32(const b2r_reduce_desc& d, const void* in) { return reduce_scalar_workspace<__half, float>(d, in); }

}  // namespace capi
}  // namespace raft_b200
