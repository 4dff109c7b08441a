// Counter-based synthetic data: element i depends only on (seed, i). The arithmetic is
// integer hashing followed by at most one int->double conversion, one double multiply and
// one double add, each correctly rounded, so a host implementation of the same formulas
// (oracle/oracle.c: synth_*) produces identical bits.
#pragma once

#include "common.cuh"

namespace raft_b200 {
namespace synth {

B2R_HDI uint64_t mix64(uint64_t x)
{
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

B2R_HDI uint64_t hash_at(uint64_t seed_mixed, uint64_t index) { return mix64(seed_mixed ^ mix64(index)); }

// kind 0: uniform [lo, hi) with a 24-bit (float / half) or 53-bit (double) mantissa draw
// kind 1: sum of eight 16-bit uniforms, centred and scaled to unit variance
// kind 2: lo + (32 random bits) mod (hi - lo), an integer
template <typename T>
B2R_DI T value_at(uint64_t seed_mixed, uint64_t index, int kind, double lo, double hi)
{
  const uint64_t h = hash_at(seed_mixed, index);
  if (kind == 2) {
    const long long ilo  = static_cast<long long>(lo);
    const long long span = static_cast<long long>(hi) - ilo;
    const long long v    = ilo + static_cast<long long>((h >> 32) % static_cast<uint64_t>(span > 0 ? span : 1));
    if constexpr (std::is_same<T, __half>::value) {
      return __float2half(float(v));
    } else {
      return T(v);
    }
  }
  double r;
  if (kind == 1) {
    const uint64_t h2 = mix64(h);
    long long s       = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      s += static_cast<long long>((h >> (16 * k)) & 0xffffull);
      s += static_cast<long long>((h2 >> (16 * k)) & 0xffffull);
    }
    s -= 4ll * 65535ll;  // centre: 8 * 65535 / 2
    // standard deviation of the sum: sqrt(8 * (65536^2 - 1) / 12)
    r = __dmul_rn(static_cast<double>(s), 1.0 / 53509.91992145008);
  } else {
    double u;
    if constexpr (std::is_same<T, double>::value) {
      u = __dmul_rn(static_cast<double>(h >> 11), 1.0 / 9007199254740992.0);
    } else {
      u = __dmul_rn(static_cast<double>(h >> 40), 1.0 / 16777216.0);
    }
    r = __dadd_rn(lo, __dmul_rn(hi - lo, u));
  }
  if constexpr (std::is_same<T, __half>::value) {
    return __float2half(__double2float_rn(r));
  } else if constexpr (std::is_same<T, float>::value) {
    return __double2float_rn(r);
  } else {
    return T(r);
  }
}

template <typename T>
__global__ void fill_kernel(T* dst, int64_t n, int64_t first, uint64_t seed_mixed, int kind, double lo, double hi)
{
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    dst[i] = value_at<T>(seed_mixed, uint64_t(first + i), kind, lo, hi);
}

template <typename T>
cudaError_t launch_fill(T* dst, int64_t n, int64_t first, uint64_t seed, int kind, double lo, double hi, cudaStream_t s)
{
  int64_t ctas = (n + 255) / 256;
  if (ctas > 148 * 64) ctas = 148 * 64;
  fill_kernel<T><<<unsigned(ctas), 256, 0, s>>>(dst, n, first, mix64(seed), kind, lo, hi);
  return cudaGetLastError();
}

}  // namespace synth
}  // namespace raft_b200
