// Stand-alone counterpart of raft/core/resource/nccl_comm.hpp:22-95: one NCCL communicator per device
// of the world, created on first use with ncclCommInitAll and destroyed with the handle.
#pragma once
#include <raft/core/error.hpp>
#include <raft/core/resource/multi_gpu.hpp>

#include <nccl.h>

#include <memory>
#include <vector>

namespace raft {
namespace resource {
namespace detail {
struct nccl_clique {
  std::vector<ncclComm_t> comms;
  ~nccl_clique()
  {
    for (ncclComm_t c : comms)
      if (c != nullptr) ncclCommDestroy(c);
  }
};
}  // namespace detail

inline std::vector<ncclComm_t>& get_nccl_comms(resources const& res)
{
  if (!res.extra_) {
    auto clique        = std::make_shared<detail::nccl_clique>();
    const auto& world  = res.world();
    std::vector<int> device_ids(world.size());
    for (size_t i = 0; i < world.size(); ++i)
      device_ids[i] = get_device_id(world[i]);
    clique->comms.resize(world.size(), nullptr);
    RAFT_EXPECTS(ncclCommInitAll(clique->comms.data(), int(device_ids.size()), device_ids.data()) == ncclSuccess,
                 "ncclCommInitAll failed");
    res.extra_ = clique;
  }
  return static_cast<detail::nccl_clique*>(res.extra_.get())->comms;
}
inline ncclComm_t& get_nccl_comm_for_rank(resources const& res, int rank) { return get_nccl_comms(res)[rank]; }
}  // namespace resource
}  // namespace raft
