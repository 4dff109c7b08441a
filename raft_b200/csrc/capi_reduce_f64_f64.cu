// C-ABI reduce instantiations for double input -> double output.
#include "capi_internal.cuh"

namespace raft_b200 {
namespace capi {

int reduce_f64_f64(const b2r_reduce_desc& d, void* out, const void* in, detail::Workspace ws, cudaStream_t s)
{
  return reduce_scalar<double, double>(d, out, in, ws, s);
}

size_t ws_f64_f64(const b2r_reduce_desc& d, const void* in) { return reduce_scalar_workspace<double, double>(d, in); }

}  // namespace capi
}  // namespace raft_b200
