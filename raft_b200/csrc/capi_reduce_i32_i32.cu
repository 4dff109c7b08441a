// C-ABI reduce instantiations for int input -> int output.
#include "capi_internal.cuh"

namespace raft_b200 {
namespace capi {

int reduce_i32_i32(const b2r_reduce_desc& d, void* out, const void* in, detail::Workspace ws, cudaStream_t s)
{
  return reduce_scalar<int, int>(d, out, in, ws, s);
}

size_t ws_i32_i32(const b2r_reduce_desc& d, const void* in) { return reduce_scalar_workspace<int, int>(d, in); }

}  // namespace capi
}  // namespace raft_b200
