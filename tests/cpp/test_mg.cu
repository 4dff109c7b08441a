// Single-process multi-device layer (include/raft_b200_mg.h) on every visible device (1..8): a host
// matrix is cut into unequal contiguous row blocks (one of them empty when there are 3 or more
// devices), one per device, and the sharded results are compared with sequential host loops:
//   - column sum with a div_const final (mean), column max of |x|: all-reduced, every device holds it
//   - row L2 norms: disjoint output slices, no exchange
//   - keyed row sums and counts, then a second call that accumulates (reset = 0)
//   - communicators created by the library and adopted from the caller (ncclCommInitAll)
//   - argument errors
// Prints one line per check and "ALL PASSED" / exits non-zero.
#include <raft_b200_mg.h>

#include <cuda_runtime.h>
#include <nccl.h>

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

static int g_fail = 0;
#define CHECK(cond, name)                                \
  do {                                                   \
    const bool ok_ = (cond);                             \
    std::printf("%s %s\n", ok_ ? "ok  " : "FAIL", name); \
    if (!ok_) ++g_fail;                                  \
  } while (0)

static bool approx(double a, double b, double eps)
{
  const double d = std::fabs(a - b);
  const double m = std::fmax(std::fabs(a), std::fabs(b));
  return (d > eps ? d / m : d) <= eps;
}

template <typename T>
static T* to_device(int dev, const T* h, size_t n)
{
  T* p = nullptr;
  cudaSetDevice(dev);
  cudaMalloc(&p, (n ? n : 1) * sizeof(T));
  if (n) cudaMemcpy(p, h, n * sizeof(T), cudaMemcpyHostToDevice);
  return p;
}
template <typename T>
static std::vector<T> to_host(int dev, const T* p, size_t n)
{
  std::vector<T> h(n);
  cudaSetDevice(dev);
  cudaDeviceSynchronize();
  if (n) cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost);
  return h;
}

static void run_all(b2r_mg_comm* comm, const std::vector<int>& devs, const char* tag)
{
  const int n      = int(devs.size());
  const int64_t R  = 100003, C = 64, K = 37;
  std::mt19937 gen(99);
  std::uniform_real_distribution<float> dist(-1.f, 1.f);
  std::vector<float> h(size_t(R) * C);
  for (auto& x : h)
    x = dist(gen);
  std::vector<int> hk(R);
  for (auto& k : hk)
    k = int(gen() % K);
  // unequal blocks; with 3 or more devices the second one is empty
  std::vector<int64_t> rows(n), first(n);
  int64_t at = 0;
  for (int d = 0; d < n; ++d) {
    int64_t want = (d == n - 1) ? R - at : (R / n) + 17 * (d % 2 ? -1 : 1);
    if (n >= 3 && d == 1) want = 0;
    rows[d]  = want;
    first[d] = at;
    at += want;
  }
  std::vector<const void*> ins(n), keys(n);
  std::vector<void*> col(n), rown(n), sums(n);
  std::vector<int64_t*> cnts(n);
  for (int d = 0; d < n; ++d) {
    ins[d]  = to_device(devs[d], h.data() + first[d] * C, size_t(rows[d] * C));
    keys[d] = to_device(devs[d], hk.data() + first[d], size_t(rows[d]));
    col[d]  = to_device<float>(devs[d], nullptr, 0);
    cudaFree(col[d]);
    cudaMalloc(&col[d], C * sizeof(float));
    cudaMalloc(&rown[d], size_t(rows[d] ? rows[d] : 1) * sizeof(float));
    cudaMalloc(&sums[d], size_t(K * C) * sizeof(float));
    cudaMalloc(reinterpret_cast<void**>(&cnts[d]), K * sizeof(int64_t));
  }
  char name[128];
  // host answers
  std::vector<double> mean(C, 0), amax(C, 0), l2(R, 0), ksum(size_t(K) * C, 0);
  std::vector<long long> kcnt(K, 0);
  for (int64_t r = 0; r < R; ++r) {
    ++kcnt[hk[r]];
    for (int64_t c = 0; c < C; ++c) {
      const double x = h[r * C + c];
      mean[c] += x;
      amax[c] = std::fmax(amax[c], std::fabs(x));
      l2[r] += double(float(x) * float(x));
      ksum[size_t(hk[r]) * C + c] += x;
    }
  }
  for (auto& m : mean)
    m /= double(R);

  b2r_reduce_desc d = {};
  d.in_dtype = d.out_dtype = B2R_F32;
  d.layout                 = B2R_ROW_MAJOR;
  d.apply                  = B2R_ALONG_COLUMNS;
  d.n_cols                 = C;
  d.main_op                = B2R_MAIN_IDENTITY;
  d.reduce_op              = B2R_REDUCE_ADD;
  d.final_op               = B2R_FINAL_DIV_CONST;
  d.final_scalar           = double(R);
  int st = b2r_mg_reduce(comm, &d, col.data(), ins.data(), rows.data(), nullptr);
  b2r_mg_sync(comm);
  bool ok = st == B2R_OK;
  for (int dv = 0; dv < n && ok; ++dv) {
    auto got = to_host(devs[dv], static_cast<float*>(col[dv]), C);
    for (int64_t c = 0; c < C; ++c)
      ok = ok && approx(mean[c], got[c], 1e-5);
  }
  std::snprintf(name, sizeof(name), "%s column mean on %d device(s), every device holds it", tag, n);
  CHECK(ok, name);

  d.main_op  = B2R_MAIN_ABS;
  d.reduce_op = B2R_REDUCE_MAX;
  d.final_op = B2R_FINAL_IDENTITY;
  st         = b2r_mg_reduce(comm, &d, col.data(), ins.data(), rows.data(), nullptr);
  b2r_mg_sync(comm);
  ok = st == B2R_OK;
  for (int dv = 0; dv < n && ok; ++dv) {
    auto got = to_host(devs[dv], static_cast<float*>(col[dv]), C);
    for (int64_t c = 0; c < C; ++c)
      ok = ok && double(got[c]) == amax[c];
  }
  CHECK(ok, "  ... column max |x| (exact)");

  d.apply     = B2R_ALONG_ROWS;
  d.main_op   = B2R_MAIN_SQ;
  d.reduce_op = B2R_REDUCE_ADD;
  st          = b2r_mg_reduce(comm, &d, rown.data(), ins.data(), rows.data(), nullptr);
  b2r_mg_sync(comm);
  ok = st == B2R_OK;
  for (int dv = 0; dv < n && ok; ++dv) {
    auto got = to_host(devs[dv], static_cast<float*>(rown[dv]), size_t(rows[dv]));
    for (int64_t r = 0; r < rows[dv]; ++r)
      ok = ok && approx(l2[first[dv] + r], got[r], 1e-5);
  }
  CHECK(ok, "  ... squared row norms, disjoint slices");

  for (int pass = 0; pass < 2; ++pass) {
    st = b2r_mg_reduce_rows_by_key(comm, sums.data(), cnts.data(), ins.data(), C, keys.data(), nullptr, B2R_F32,
                                   B2R_I32, rows.data(), C, K, pass == 0 ? 1 : 0, nullptr);
    b2r_mg_sync(comm);
    ok = st == B2R_OK;
    for (int dv = 0; dv < n && ok; ++dv) {
      auto gs = to_host(devs[dv], static_cast<float*>(sums[dv]), size_t(K * C));
      auto gc = to_host(devs[dv], cnts[dv], size_t(K));
      for (size_t i = 0; i < gs.size(); ++i)
        ok = ok && approx((pass + 1) * ksum[i], gs[i], 1e-5);
      for (int64_t k = 0; k < K; ++k)
        ok = ok && gc[k] == (pass + 1) * kcnt[k];
    }
    CHECK(ok, pass == 0 ? "  ... keyed row sums and counts" : "  ... accumulated a second time (reset = 0)");
  }

  d.apply   = B2R_ALONG_COLUMNS;
  d.inplace = 1;
  CHECK(b2r_mg_reduce(comm, &d, col.data(), ins.data(), rows.data(), nullptr) == B2R_ERR_UNSUPPORTED,
        "  ... inplace column reduction is refused");
  for (int dv = 0; dv < n; ++dv) {
    cudaSetDevice(devs[dv]);
    cudaFree(const_cast<void*>(ins[dv]));
    cudaFree(const_cast<void*>(keys[dv]));
    cudaFree(col[dv]);
    cudaFree(rown[dv]);
    cudaFree(sums[dv]);
    cudaFree(cnts[dv]);
  }
}

int main()
{
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    std::printf("no CUDA device\n");
    return 2;
  }
  if (ndev > 8) ndev = 8;
  std::vector<int> devs(ndev);
  for (int i = 0; i < ndev; ++i)
    devs[i] = i;
  b2r_mg_comm* comm = nullptr;
  CHECK(b2r_mg_comm_create(&comm, devs.data(), ndev) == B2R_OK && b2r_mg_comm_size(comm) == ndev, "comm create");
  if (comm != nullptr) run_all(comm, devs, "own communicators:");
  b2r_mg_comm_destroy(comm);

  std::vector<ncclComm_t> nccl(ndev);
  if (ncclCommInitAll(nccl.data(), ndev, devs.data()) == ncclSuccess) {
    std::vector<void*> handles(nccl.begin(), nccl.end());
    b2r_mg_comm* adopted = nullptr;
    CHECK(b2r_mg_comm_adopt(&adopted, devs.data(), ndev, handles.data()) == B2R_OK, "comm adopt");
    if (adopted != nullptr) run_all(adopted, devs, "adopted communicators:");
    b2r_mg_comm_destroy(adopted);
    for (auto& c : nccl)
      ncclCommDestroy(c);
  } else {
    CHECK(false, "ncclCommInitAll");
  }

  const int twice[2] = {0, 0};
  b2r_mg_comm* bad   = nullptr;
  CHECK(b2r_mg_comm_create(&bad, twice, 2) == B2R_ERR_BAD_ARG, "a device listed twice is refused");
  const int beyond[1] = {ndev + 100};
  CHECK(b2r_mg_comm_create(&bad, beyond, 1) == B2R_ERR_BAD_ARG, "a device ordinal beyond the visible ones is refused");
  if (g_fail) {
    std::printf("%d CHECKS FAILED\n", g_fail);
    return 1;
  }
  std::printf("ALL PASSED\n");
  return 0;
}
