// Stand-in for rmm/device_uvector.hpp (oracle/_ref build only): stream-ordered device array.
#pragma once
#include <rmm/cuda_stream_view.hpp>

#include <cstddef>

namespace rmm {
template <typename T>
class device_uvector {
 public:
  device_uvector(std::size_t n, cuda_stream_view s) : n_(n), s_(s)
  {
    if (n_ > 0) cudaMallocAsync(reinterpret_cast<void**>(&p_), n_ * sizeof(T), s_.value());
  }
  ~device_uvector()
  {
    if (p_ != nullptr) cudaFreeAsync(p_, s_.value());
  }
  device_uvector(const device_uvector&)            = delete;
  device_uvector& operator=(const device_uvector&) = delete;
  T* data() noexcept { return p_; }
  const T* data() const noexcept { return p_; }
  std::size_t size() const noexcept { return n_; }

 private:
  T* p_ = nullptr;
  std::size_t n_;
  cuda_stream_view s_;
};
}  // namespace rmm
