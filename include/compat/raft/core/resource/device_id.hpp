// Stand-alone counterpart of raft/core/resource/device_id.hpp:46-53: the device a handle was made on.
#pragma once
#include <raft/core/resources.hpp>

namespace raft {
namespace resource {
inline int get_device_id(resources const& res) { return res.device_id_; }
}  // namespace resource
}  // namespace raft
