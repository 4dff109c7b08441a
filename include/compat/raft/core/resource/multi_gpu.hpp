// Stand-alone counterpart of raft/core/resource/multi_gpu.hpp:64-129: the per-device handles of a
// single-process multi-GPU handle ("world"), the root rank, and the device switches.
#pragma once
#include <raft/core/resource/device_id.hpp>
#include <raft/core/resources.hpp>

#include <cuda_runtime_api.h>

#include <vector>

namespace raft {
namespace resource {
inline std::vector<raft::resources>& get_multi_gpu_resource(resources const& res) { return res.world(); }
inline bool is_multi_gpu(resources const& res) { return res.has_world(); }
inline int get_num_ranks(resources const& res) { return int(res.world().size()); }
inline const raft::resources& get_device_resources_for_rank(resources const& res, int rank) { return res.world()[rank]; }
inline const raft::resources& set_current_device_to_rank(resources const& res, int rank)
{
  const raft::resources& dev_res = res.world()[rank];
  cudaSetDevice(get_device_id(dev_res));
  return dev_res;
}
inline int get_root_rank(resources const& res) { return res.root_rank_; }
inline void set_root_rank(resources& res, int root_rank) { res.root_rank_ = root_rank; }
inline const raft::resources& set_current_device_to_root_rank(resources const& res)
{
  return set_current_device_to_rank(res, res.root_rank_);
}
}  // namespace resource
}  // namespace raft
