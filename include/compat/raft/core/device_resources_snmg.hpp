// Stand-alone counterpart of raft/core/device_resources_snmg.hpp:36-150: a handle that one process uses to
// drive several GPUs - a device handle for the GPU it was made on plus one handle per device of its world.
// (Memory pools, which the reference's class also manages, have no counterpart here: the stand-alone build
// has no rmm.)
#pragma once
#include <raft/core/resource/multi_gpu.hpp>
#include <raft/core/resources.hpp>

#include <cuda_runtime_api.h>

#include <vector>

namespace raft {

class device_resources_snmg : public resources {
 public:
  /** every visible GPU */
  device_resources_snmg() : resources()
  {
    int n = 0;
    cudaGetDeviceCount(&n);
    std::vector<int> ids(n > 0 ? n : 0);
    for (int i = 0; i < n; ++i)
      ids[i] = i;
    init_world(ids);
  }
  /** a subset of the GPUs */
  explicit device_resources_snmg(const std::vector<int>& device_ids) : resources() { init_world(device_ids); }

 private:
  void init_world(const std::vector<int>& device_ids)
  {
    int main_gpu = 0;
    cudaGetDevice(&main_gpu);
    resource::set_root_rank(*this, 0);
    auto& world = resource::get_multi_gpu_resource(*this);
    for (int id : device_ids) {
      cudaSetDevice(id);
      world.emplace_back();  // a handle made with that device current
    }
    cudaSetDevice(main_gpu);
  }
};

}  // namespace raft
