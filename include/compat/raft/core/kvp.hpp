// Stand-alone raft::KeyValuePair (reference: core/kvp.hpp:20-62): a {key, value} aggregate with
// the member order and layout reductions such as argmin / argmax write to memory.
#pragma once
#include <cuda_runtime.h>

namespace raft {

template <typename K, typename V>
struct KeyValuePair {
  using Key   = K;
  using Value = V;
  Key key;
  Value value;

  KeyValuePair() = default;
  __host__ __device__ KeyValuePair(Key const& k, Value const& v) : key(k), value(v) {}

  __host__ __device__ bool operator!=(const KeyValuePair& o) const { return value != o.value || key != o.key; }
  __host__ __device__ bool operator==(const KeyValuePair& o) const { return value == o.value && key == o.key; }
  __host__ __device__ bool operator<(const KeyValuePair& o) const
  {
    return key < o.key || (key == o.key && value < o.value);
  }
  __host__ __device__ bool operator>(const KeyValuePair& o) const
  {
    return key > o.key || (key == o.key && value > o.value);
  }
};

}  // namespace raft
