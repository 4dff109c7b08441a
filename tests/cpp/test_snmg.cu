// The row-sharded raft::linalg overloads that take the reference's single-process multi-GPU handle
// (include/raft/linalg/sharded_reduce.cuh), on every visible device: column mean, row L2 norms and keyed
// row sums of a matrix cut into unequal row blocks, against the same reductions of the whole matrix on
// device 0. Built twice: stand-alone (raft::device_resources_snmg of include/compat) and, with
// -DB2R_TEST_OVERLAY, on the reference's own raft/core headers, where the handle is a raft::resources whose
// multi-GPU world is filled exactly as device_resources_snmg's constructor fills it
// (core/device_resources_snmg.hpp:137-150; that header itself needs rmm's memory resources).
#include <raft/linalg/reduce.cuh>
#include <raft/linalg/reduce_rows_by_key.cuh>
#include <raft/linalg/sharded_reduce.cuh>
#ifndef B2R_TEST_OVERLAY
#include <raft/core/device_resources_snmg.hpp>
#endif

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CK(x)                                                                            \
  do {                                                                                   \
    cudaError_t e_ = (x);                                                                \
    if (e_ != cudaSuccess) {                                                             \
      std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__);       \
      std::exit(1);                                                                      \
    }                                                                                    \
  } while (0)

static int g_fail = 0;
static void expect(bool ok, const char* what)
{
  std::printf("%s %s\n", ok ? "ok  " : "FAIL", what);
  if (!ok) ++g_fail;
}

int main()
{
  int n_dev = 0;
  CK(cudaGetDeviceCount(&n_dev));
  if (n_dev > 8) n_dev = 8;
  const int n_rows = 100003, n_cols = 64, n_keys = 37;
  std::vector<float> h(size_t(n_rows) * n_cols);
  std::vector<int> hk(n_rows);
  unsigned s = 12345u;
  for (auto& v : h) {
    s = s * 1664525u + 1013904223u;
    v = float(s >> 8) * (2.0f / 16777216.0f) - 1.0f;
  }
  for (int i = 0; i < n_rows; ++i) {
    s     = s * 1664525u + 1013904223u;
    hk[i] = int((s >> 10) % unsigned(n_keys));
  }
#ifdef B2R_TEST_OVERLAY
  raft::resources handle;
  {
    auto& world = raft::resource::get_multi_gpu_resource(handle);
    for (int d = 0; d < n_dev; ++d) {
      CK(cudaSetDevice(d));
      world.emplace_back();
      raft::resource::get_device_id(world.back());
    }
    CK(cudaSetDevice(0));
  }
#else
  std::vector<int> ids(n_dev);
  for (int d = 0; d < n_dev; ++d)
    ids[d] = d;
  raft::device_resources_snmg handle(ids);
#endif
  expect(raft::resource::get_num_ranks(handle) == n_dev, "world size");

  // unequal row blocks: the first device gets the remainder and a little more
  std::vector<int> r0(n_dev + 1, 0);
  for (int d = 0; d < n_dev; ++d)
    r0[d + 1] = d + 1 == n_dev ? n_rows : r0[d] + (n_rows / n_dev) + (d == 0 ? 17 : -17 / (n_dev > 1 ? n_dev - 1 : 1));
  std::vector<float*> A(n_dev), norms(n_dev), mean(n_dev), sums(n_dev);
  std::vector<int*> keys(n_dev);
  for (int d = 0; d < n_dev; ++d) {
    const size_t rows = size_t(r0[d + 1] - r0[d]);
    CK(cudaSetDevice(d));
    CK(cudaMalloc(&A[d], rows * n_cols * 4 + 16));
    CK(cudaMalloc(&keys[d], rows * 4 + 16));
    CK(cudaMalloc(&norms[d], rows * 4 + 16));
    CK(cudaMalloc(&mean[d], n_cols * 4));
    CK(cudaMalloc(&sums[d], size_t(n_keys) * n_cols * 4));
    CK(cudaMemcpy(A[d], h.data() + size_t(r0[d]) * n_cols, rows * n_cols * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(keys[d], hk.data() + r0[d], rows * 4, cudaMemcpyHostToDevice));
  }
  using mview = raft::device_matrix_view<const float, int, raft::row_major>;
  std::vector<mview> shards;
  std::vector<raft::device_vector_view<float, int>> v_norms, v_mean;
  std::vector<raft::device_vector_view<const int, int>> v_keys;
  std::vector<raft::device_matrix_view<float, int, raft::row_major>> v_sums;
  for (int d = 0; d < n_dev; ++d) {
    const int rows = r0[d + 1] - r0[d];
    shards.push_back(raft::make_device_matrix_view<const float, int, raft::row_major>(A[d], rows, n_cols));
    v_norms.push_back(raft::make_device_vector_view<float, int>(norms[d], rows));
    v_mean.push_back(raft::make_device_vector_view<float, int>(mean[d], n_cols));
    v_keys.push_back(raft::make_device_vector_view<const int, int>(keys[d], rows));
    v_sums.push_back(raft::make_device_matrix_view<float, int, raft::row_major>(sums[d], n_keys, n_cols));
  }
  raft::linalg::reduce(handle, shards, v_norms, 0.0f, raft::Apply::ALONG_ROWS, raft::sq_op(), raft::add_op(), raft::sqrt_op());
  raft::linalg::reduce(handle, shards, v_mean, 0.0f, raft::Apply::ALONG_COLUMNS, raft::identity_op(), raft::add_op(),
                       raft::div_const_op<float>(float(n_rows)));
  raft::linalg::reduce_rows_by_key(handle, shards, v_keys, v_sums, n_keys);
  for (int d = 0; d < n_dev; ++d) {
    CK(cudaSetDevice(d));
    CK(cudaDeviceSynchronize());
  }

  // the same on the whole matrix, device 0
  CK(cudaSetDevice(0));
  float *fA, *f_norms, *f_mean, *f_sums;
  int* f_keys;
  CK(cudaMalloc(&fA, h.size() * 4));
  CK(cudaMalloc(&f_keys, size_t(n_rows) * 4));
  CK(cudaMalloc(&f_norms, size_t(n_rows) * 4));
  CK(cudaMalloc(&f_mean, n_cols * 4));
  CK(cudaMalloc(&f_sums, size_t(n_keys) * n_cols * 4));
  CK(cudaMemcpy(fA, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(f_keys, hk.data(), size_t(n_rows) * 4, cudaMemcpyHostToDevice));
  cudaStream_t st = nullptr;
  raft::linalg::reduce<true, true>(f_norms, fA, n_cols, n_rows, 0.0f, st, false, raft::sq_op(), raft::add_op(), raft::sqrt_op());
  raft::linalg::reduce<true, false>(f_mean, fA, n_cols, n_rows, 0.0f, st, false, raft::identity_op(), raft::add_op(),
                                    raft::div_const_op<float>(float(n_rows)));
  raft::linalg::reduce_rows_by_key(fA, n_cols, f_keys, static_cast<char*>(nullptr), n_rows, n_cols, n_keys, f_sums, st);
  CK(cudaDeviceSynchronize());
  std::vector<float> e_norms(n_rows), e_mean(n_cols), e_sums(size_t(n_keys) * n_cols);
  CK(cudaMemcpy(e_norms.data(), f_norms, e_norms.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(e_mean.data(), f_mean, e_mean.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(e_sums.data(), f_sums, e_sums.size() * 4, cudaMemcpyDeviceToHost));

  auto close = [](float a, float b) { return std::fabs(a - b) <= 1e-5f || std::fabs(a - b) <= 1e-5f * std::fmax(std::fabs(a), std::fabs(b)); };
  bool ok_norm = true, ok_mean = true, ok_sums = true;
  for (int d = 0; d < n_dev; ++d) {
    const int rows = r0[d + 1] - r0[d];
    std::vector<float> g(rows), gm(n_cols), gs(size_t(n_keys) * n_cols);
    CK(cudaSetDevice(d));
    CK(cudaMemcpy(g.data(), norms[d], size_t(rows) * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(gm.data(), mean[d], gm.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(gs.data(), sums[d], gs.size() * 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < rows; ++i)
      ok_norm = ok_norm && g[i] == e_norms[r0[d] + i];  // the same kernel on the same rows: the same bits
    for (int j = 0; j < n_cols; ++j)
      ok_mean = ok_mean && close(gm[j], e_mean[j]);
    for (size_t j = 0; j < gs.size(); ++j)
      ok_sums = ok_sums && close(gs[j], e_sums[j]);
  }
  expect(ok_norm, "row L2 norms: disjoint slices, bit-identical to the single-device call");
  expect(ok_mean, "column mean: every device holds the mean of the whole matrix");
  expect(ok_sums, "keyed row sums: every device holds the sums over all shards");
  std::printf(g_fail == 0 ? "SNMG ALL PASSED (%d device%s)\n" : "SNMG FAILED (%d device%s)\n", n_dev, n_dev == 1 ? "" : "s");
  return g_fail == 0 ? 0 : 1;
}
