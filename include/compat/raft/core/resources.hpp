// Minimal raft::resources for the stand-alone build: the reduction headers ask a handle for its CUDA
// stream (reference: core/resources.hpp:47-139, core/resource/cuda_stream.hpp:61-79; the default is the
// per-thread stream, :23), and the sharded forms ask it for the device it was made on, for the handles of its
// multi-GPU world and for their NCCL communicators (core/resource/{device_id,multi_gpu,nccl_comm}.hpp).
// Like the reference's, a handle is a bag of lazily made resources behind a const interface.
#pragma once
#include <cuda_runtime_api.h>

#include <memory>
#include <vector>

namespace raft {

class resources {
 public:
  resources() { cudaGetDevice(&device_id_); }
  explicit resources(cudaStream_t s) : stream_(s) { cudaGetDevice(&device_id_); }
  cudaStream_t stream_ = cudaStreamPerThread;
  int device_id_       = 0;
  int root_rank_       = 0;

  // the per-device handles of a multi-GPU handle, made on first use
  std::vector<resources>& world() const
  {
    if (!world_) world_ = std::make_shared<std::vector<resources>>();
    return *world_;
  }
  bool has_world() const { return bool(world_); }
  mutable std::shared_ptr<void> extra_;  // the NCCL clique of raft/core/resource/nccl_comm.hpp

 private:
  mutable std::shared_ptr<std::vector<resources>> world_;
};

using device_resources = resources;

namespace resource {
inline cudaStream_t get_cuda_stream(resources const& res) { return res.stream_; }
inline void set_cuda_stream(resources& res, cudaStream_t s) { res.stream_ = s; }
inline void sync_stream(resources const& res) { cudaStreamSynchronize(res.stream_); }
}  // namespace resource

}  // namespace raft
