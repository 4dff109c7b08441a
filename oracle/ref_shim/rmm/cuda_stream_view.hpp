// Stand-in for rmm/cuda_stream_view.hpp, only for compiling the untouched reference headers
// offline into oracle/_ref (test infrastructure). A value wrapper around cudaStream_t.
#pragma once
#include <cuda_runtime_api.h>

namespace rmm {
class cuda_stream_view {
 public:
  constexpr cuda_stream_view() = default;
  constexpr cuda_stream_view(cudaStream_t s) noexcept : stream_(s) {}
  constexpr cudaStream_t value() const noexcept { return stream_; }
  constexpr operator cudaStream_t() const noexcept { return stream_; }
  bool is_per_thread_default() const noexcept { return stream_ == cudaStreamPerThread; }
  bool is_default() const noexcept { return stream_ == cudaStreamLegacy || stream_ == nullptr; }
  void synchronize() const { cudaStreamSynchronize(stream_); }
  void synchronize_no_throw() const noexcept { cudaStreamSynchronize(stream_); }

 private:
  cudaStream_t stream_{};
};
inline bool operator==(cuda_stream_view a, cuda_stream_view b) { return a.value() == b.value(); }
inline bool operator!=(cuda_stream_view a, cuda_stream_view b) { return !(a == b); }
static const cuda_stream_view cuda_stream_default{};
static const cuda_stream_view cuda_stream_legacy{cudaStreamLegacy};
static const cuda_stream_view cuda_stream_per_thread{cudaStreamPerThread};
}  // namespace rmm
