// Stand-alone replacement for the parts of raft/core/error.hpp the reduction headers use:
// the exception types and the RAFT_EXPECTS / RAFT_FAIL / THROW / RAFT_CUDA_TRY macros
// (reference: core/error.hpp:276-348, util/cuda_rt_essentials.hpp:25-67). Used when no full
// RAFT installation provides <raft/core/error.hpp>.
#pragma once
#include <cuda_runtime_api.h>

#include <cstdio>
#include <stdexcept>
#include <string>

namespace raft {

class exception : public std::exception {
 public:
  explicit exception(std::string msg) : msg_(std::move(msg)) {}
  const char* what() const noexcept override { return msg_.c_str(); }

 private:
  std::string msg_;
};

class logic_error : public exception {
 public:
  using exception::exception;
};

class cuda_error : public exception {
 public:
  using exception::exception;
};

namespace detail {
template <typename... A>
inline std::string format_msg(const char* file, int line, const char* fmt, A... args)
{
  char buf[1024];
  if constexpr (sizeof...(A) == 0) {
    std::snprintf(buf, sizeof(buf), "%s", fmt);
  } else {
    std::snprintf(buf, sizeof(buf), fmt, args...);
  }
  return std::string(buf) + " (" + file + ":" + std::to_string(line) + ")";
}
}  // namespace detail
}  // namespace raft

#define RAFT_EXPECTS(cond, ...)                                                                       \
  do {                                                                                                \
    if (!(cond)) throw raft::logic_error(raft::detail::format_msg(__FILE__, __LINE__, __VA_ARGS__));  \
  } while (0)

#define RAFT_FAIL(...) throw raft::logic_error(raft::detail::format_msg(__FILE__, __LINE__, __VA_ARGS__))

#define THROW(...) throw raft::exception(raft::detail::format_msg(__FILE__, __LINE__, __VA_ARGS__))

#define RAFT_CUDA_TRY(call)                                                                     \
  do {                                                                                          \
    const cudaError_t raft_status_ = (call);                                                    \
    if (raft_status_ != cudaSuccess) {                                                          \
      (void)cudaGetLastError();                                                                 \
      throw raft::cuda_error(raft::detail::format_msg(__FILE__, __LINE__, "CUDA error: %s %s",  \
                                                      cudaGetErrorName(raft_status_),           \
                                                      cudaGetErrorString(raft_status_)));       \
    }                                                                                           \
  } while (0)
