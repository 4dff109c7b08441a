// Measurement aids of the C ABI: the two floors a benchmark compares a small reduction with.
//   b2r_probe_empty_launch   one empty kernel on the stream: what an event pair around ANY launch costs
//   b2r_probe_stream_read    reads a buffer once with every SM streaming 16-byte loads (sixteen in flight
//                            per lane, four CTAs per SM) and nothing else: the fastest a kernel of this
//                            library could possibly consume that many bytes
// Neither has a counterpart in the reference; its benchmarks (cpp/bench/prims/common/benchmark.hpp)
// report times without a floor.
#include "capi_internal.cuh"

namespace raft_b200 {
namespace capi {

__global__ void probe_empty_kernel() {}

template <int U>
__global__ void __launch_bounds__(256) probe_read_kernel(float* sink, const float* data, int64_t nvec, int64_t vec_per_cta)
{
  using detail::VecOf;
  const int64_t v0 = int64_t(blockIdx.x) * vec_per_cta;
  int64_t v1       = v0 + vec_per_cta;
  v1               = v1 < nvec ? v1 : nvec;
  float s          = 0.f;
  int64_t c        = v0 + threadIdx.x;
  for (; c + int64_t(U - 1) * 256 < v1; c += int64_t(U) * 256) {
    VecOf<float, 4> v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      v[u] = detail::load_stream<float, 4>(data + (c + int64_t(u) * 256) * 4);
#pragma unroll
    for (int u = 0; u < U; ++u)
      s += (v[u].e[0] + v[u].e[1]) + (v[u].e[2] + v[u].e[3]);
  }
  for (; c < v1; c += 256) {
    const VecOf<float, 4> v = detail::load_stream<float, 4>(data + c * 4);
    s += (v.e[0] + v.e[1]) + (v.e[2] + v.e[3]);
  }
  // the sum only keeps the loads alive; it is stored for one value nobody will ever see
  if (sink != nullptr && s == 1.2345678e38f) sink[0] = s;
}

}  // namespace capi
}  // namespace raft_b200

using namespace raft_b200;
using namespace raft_b200::capi;

extern "C" int b2r_probe_empty_launch(b2r_stream_t stream)
{
  probe_empty_kernel<<<1, 32, 0, to_stream(stream)>>>();
  return set_cuda_error(cudaGetLastError());
}

extern "C" int b2r_probe_stream_read(const void* data, size_t bytes, float* sink, b2r_stream_t stream)
{
  if (bytes > 0 && data == nullptr) return B2R_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(data) & 15u) != 0) return B2R_ERR_BAD_ARG;
  const int64_t nvec = int64_t(bytes / 16);
  if (nvec == 0) return B2R_OK;
  const int64_t ctas = int64_t(detail::sm_count()) * 4;
  int64_t vpc        = detail::ceil_div<int64_t>(nvec, ctas);
  vpc                = detail::ceil_div<int64_t>(vpc, 256) * 256;
  const unsigned grid = unsigned(detail::ceil_div<int64_t>(nvec, vpc));
  probe_read_kernel<16><<<grid, 256, 0, to_stream(stream)>>>(sink, static_cast<const float*>(data), nvec, vpc);
  return set_cuda_error(cudaGetLastError());
}
