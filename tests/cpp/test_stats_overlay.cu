// Overlay check of the "next" callers: the REFERENCE's own, unmodified raft::stats::{sum, mean,
// stddev, vars, weighted_mean} headers compiled on top of this repository's raft/linalg headers
// (which come first on the include path), i.e. what a RAFT user gets by dropping the headers in.
// Cases follow the reference's tests: constant matrices and the error-compensation pattern of
// cpp/tests/stats/sum.cu:50-129, and mean / stddev / weighted mean of random data against host
// loops (cpp/tests/stats/{mean,stddev,weighted_mean}.cu).
#include <raft/core/device_mdspan.hpp>
#include <raft/core/resources.hpp>
#include <raft/stats/mean.cuh>
#include <raft/stats/stddev.cuh>
#include <raft/stats/sum.cuh>
#include <raft/stats/weighted_mean.cuh>

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

static int g_fail = 0;
#define CHECK(cond, name)                                 \
  do {                                                    \
    const bool ok_ = (cond);                              \
    std::printf("%s %s\n", ok_ ? "ok  " : "FAIL", name);  \
    if (!ok_) ++g_fail;                                   \
  } while (0)

template <typename T>
struct DevBuf {
  T* p = nullptr;
  size_t n;
  explicit DevBuf(size_t n_) : n(n_) { cudaMalloc(&p, (n ? n : 1) * sizeof(T)); }
  DevBuf(const std::vector<T>& h) : n(h.size())
  {
    cudaMalloc(&p, (n ? n : 1) * sizeof(T));
    cudaMemcpy(p, h.data(), n * sizeof(T), cudaMemcpyHostToDevice);
  }
  ~DevBuf() { cudaFree(p); }
  std::vector<T> host() const
  {
    std::vector<T> h(n);
    cudaDeviceSynchronize();
    cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost);
    return h;
  }
};

static bool approx(double a, double b, double eps)
{
  const double d = std::fabs(a - b), m = std::fmax(std::fabs(a), std::fabs(b));
  return (d > eps ? d / m : d) <= eps;
}

template <typename T>
static void sum_case(int rows, int cols, bool row_major, T value, double tol, bool compensation)
{
  raft::resources handle;
  std::vector<T> h(size_t(rows) * cols, value);
  const double large = std::is_same<T, double>::value ? 1e12 : 1e7;
  if (compensation) {
    for (int i = 0; i < rows * cols; ++i) {
      const int row = row_major ? i / cols : i % rows;
      if (row % 3 == 2) {
        h[i]                                  = T(double(value) * large);
        h[row_major ? (i - cols) : (i - 1)]   = T(-double(value) * large);
        h[row_major ? (i - 2 * cols) : (i - 2)] = T(3.0 * double(value));
      }
    }
  }
  DevBuf<T> d(h), out(cols);
  if (row_major) {
    raft::stats::sum(handle, raft::make_device_matrix_view<const T, int, raft::row_major>(d.p, rows, cols),
                     raft::make_device_vector_view<T, int>(out.p, cols));
  } else {
    raft::stats::sum(handle, raft::make_device_matrix_view<const T, int, raft::col_major>(d.p, rows, cols),
                     raft::make_device_vector_view<T, int>(out.p, cols));
  }
  auto got = out.host();
  bool ok  = true;
  for (int c = 0; c < cols; ++c)
    ok = ok && approx(double(rows) * double(value), double(got[c]), tol);
  char name[160];
  std::snprintf(name, sizeof(name), "stats::sum %s %dx%d %s%s", std::is_same<T, double>::value ? "f64" : "f32", rows,
                cols, row_major ? "row-major" : "col-major", compensation ? " (cancelling 1e7 / 1e12 pairs)" : "");
  CHECK(ok, name);
}

static void mean_stddev_case(int rows, int cols, bool row_major)
{
  raft::resources handle;
  cudaStream_t stream = raft::resource::get_cuda_stream(handle);
  std::mt19937 gen(42);
  std::normal_distribution<float> dist(1.0f, 2.0f);
  std::vector<float> h(size_t(rows) * cols);
  for (auto& x : h)
    x = dist(gen);
  auto at = [&](int r, int c) { return double(h[row_major ? size_t(r) * cols + c : size_t(c) * rows + r]); };
  std::vector<double> mu(cols, 0), sd(cols, 0);
  for (int c = 0; c < cols; ++c) {
    for (int r = 0; r < rows; ++r)
      mu[c] += at(r, c);
    mu[c] /= rows;
    for (int r = 0; r < rows; ++r)
      sd[c] += (at(r, c) - mu[c]) * (at(r, c) - mu[c]);
    sd[c] = std::sqrt(sd[c] / (rows - 1));
  }
  DevBuf<float> d(h), dmu(cols), dsd(cols), dvar(cols);
  if (row_major) {
    raft::stats::mean<true>(dmu.p, d.p, cols, rows, stream);
    raft::stats::stddev<true>(dsd.p, d.p, dmu.p, cols, rows, true, stream);
    raft::stats::vars<true>(dvar.p, d.p, dmu.p, cols, rows, true, stream);
  } else {
    raft::stats::mean<false>(dmu.p, d.p, cols, rows, stream);
    raft::stats::stddev<false>(dsd.p, d.p, dmu.p, cols, rows, true, stream);
    raft::stats::vars<false>(dvar.p, d.p, dmu.p, cols, rows, true, stream);
  }
  auto gmu = dmu.host(), gsd = dsd.host(), gvar = dvar.host();
  bool ok_mu = true, ok_sd = true, ok_var = true;
  for (int c = 0; c < cols; ++c) {
    ok_mu  = ok_mu && approx(mu[c], gmu[c], 1e-5);
    ok_sd  = ok_sd && approx(sd[c], gsd[c], 1e-4);
    ok_var = ok_var && approx(sd[c] * sd[c], gvar[c], 1e-4);
  }
  char name[128];
  std::snprintf(name, sizeof(name), "stats::mean %dx%d %s", rows, cols, row_major ? "row-major" : "col-major");
  CHECK(ok_mu, name);
  CHECK(ok_sd, "  ... stats::stddev (sample)");
  CHECK(ok_var, "  ... stats::vars (sample)");
}

static void weighted_mean_case(int rows, int cols)
{
  raft::resources handle;
  cudaStream_t stream = raft::resource::get_cuda_stream(handle);
  std::mt19937 gen(7);
  std::uniform_real_distribution<float> dist(-1.f, 1.f), wd(0.1f, 1.f);
  std::vector<float> h(size_t(rows) * cols), w(cols);
  for (auto& x : h)
    x = dist(gen);
  for (auto& x : w)
    x = wd(gen);
  double ws = 0;
  for (auto x : w)
    ws += x;
  std::vector<double> e(rows, 0);
  for (int r = 0; r < rows; ++r) {
    for (int c = 0; c < cols; ++c)
      e[r] += double(h[size_t(r) * cols + c]) * w[c];
    e[r] /= ws;
  }
  DevBuf<float> d(h), dw(w), out(rows);
  raft::stats::rowWeightedMean(out.p, d.p, dw.p, cols, rows, stream);
  auto got = out.host();
  bool ok  = true;
  for (int r = 0; r < rows; ++r)
    ok = ok && approx(e[r], got[r], 1e-5);
  CHECK(ok, "stats::rowWeightedMean 1000x77");
}

int main()
{
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return 2;
  for (bool rm : {true, false}) {
    sum_case<float>(4, 5, rm, 1.f, 1e-4, false);
    sum_case<float>(1024, 32, rm, 1.f, 1e-4, false);
    sum_case<float>(1024, 256, rm, 1.f, 1e-4, false);
    sum_case<float>(10000000, 1, rm, 0.001f, 1e-4, false);
    sum_case<float>(1 << 22, 2, rm, 0.1f, 1e-4, false);
    sum_case<float>(17, 5, rm, 0.001f, 1e-4, false);
    sum_case<float>(3, 97, rm, 0.001f, 1e-4, false);
    sum_case<double>(1024, 256, rm, 1.0, 1e-6, false);
    sum_case<double>(10000000, 1, rm, 0.001, 1e-6, false);
    // the reference checks these with 100 x tolerance; the wide / compensated sums here hold the plain one
    sum_case<float>(1023, 32, rm, 1.f, 1e-4, true);
    sum_case<float>(3 * 7001, 5, rm, 0.001f, 1e-4, true);
    sum_case<double>(1023, 32, rm, 1.0, 1e-6, true);
    mean_stddev_case(4000, 70, rm);
    mean_stddev_case(333, 513, rm);
  }
  weighted_mean_case(1000, 77);
  cudaDeviceSynchronize();
  if (cudaGetLastError() != cudaSuccess || g_fail) {
    std::printf("%d CHECKS FAILED\n", g_fail);
    return 1;
  }
  std::printf("ALL PASSED\n");
  return 0;
}
