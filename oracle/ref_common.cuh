// Shared by the oracle/_ref translation units: wraps calls into the UNMODIFIED reference
// headers (included from the read-only reference checkout at build time) behind a small C ABI
// that takes the same descriptor as the product library. Test infrastructure only.
#pragma once
#include <raft_b200.h>

#include <raft/core/kvp.hpp>
#include <raft/core/operators.hpp>
#include <raft/linalg/reduce.cuh>

#include <cstdio>
#include <exception>

#define REF_EXPORT extern "C" __attribute__((visibility("default")))

namespace refwrap {

template <typename F>
int guarded(F&& f)
{
  try {
    f();
  } catch (const std::exception& e) {
    std::fprintf(stderr, "reference threw: %s\n", e.what());
    return B2R_ERR_CUDA;
  }
  return B2R_OK;
}

// value, index -> {index, value}: the functor the reference's tests define locally
// (cpp/tests/linalg/reduce.cu:346-349); the reference ships none.
template <typename T, typename IdxT>
struct ValueToKVP {
  __host__ __device__ raft::KeyValuePair<IdxT, T> operator()(T value, IdxT idx) { return {idx, value}; }
};

template <bool RowMajor, bool AlongRows, typename In, typename Out, typename Main, typename Red, typename Fin>
int run(const b2r_reduce_desc& d, void* out, const void* in, Out init, Main m, Red r, Fin f, cudaStream_t s)
{
  return guarded([&] {
    raft::linalg::reduce<RowMajor, AlongRows, In, Out, int>(static_cast<Out*>(out), static_cast<const In*>(in),
                                                           int(d.n_cols), int(d.n_rows), init, s, d.inplace != 0, m,
                                                           r, f);
  });
}

}  // namespace refwrap
