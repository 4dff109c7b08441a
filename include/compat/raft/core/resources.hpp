// Minimal raft::resources for the stand-alone build: the reduction headers only ever ask a
// handle for its CUDA stream (reference: core/resources.hpp:47-139,
// core/resource/cuda_stream.hpp:61-79; the default is the per-thread stream, :23).
#pragma once
#include <cuda_runtime_api.h>

namespace raft {

class resources {
 public:
  resources() = default;
  explicit resources(cudaStream_t s) : stream_(s) {}
  cudaStream_t stream_ = cudaStreamPerThread;
};

using device_resources = resources;

namespace resource {
inline cudaStream_t get_cuda_stream(resources const& res) { return res.stream_; }
inline void set_cuda_stream(resources& res, cudaStream_t s) { res.stream_ = s; }
inline void sync_stream(resources const& res) { cudaStreamSynchronize(res.stream_); }
}  // namespace resource

}  // namespace raft
