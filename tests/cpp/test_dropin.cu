// Exercises the drop-in raft::linalg headers (include/raft/linalg/*.cuh, stand-alone core under
// include/compat) the way the reference's own gtests do, against sequential host loops:
//   - the 3x4 known-answer max reduce, both layouts, both axes (cpp/tests/linalg/reduce.cu:106-178)
//   - sq / add / sqrt reduce with inplace second pass (reduce.cu:191-241)
//   - key/value reduce with a test-local tagger and ArgMax functor (reduce.cu:346-411)
//   - row / column norms through the mdspan API (cpp/tests/linalg/norm.cu)
//   - device lambdas as main / final op (the way stats::stddev and weighted_mean call reduce)
//   - reduce_rows_by_key incl. the (ncols, nrows) mdspan convention (reduce_rows_by_key.cu:134-147)
//   - reduce_cols_by_key incl. nkeys inferred from the output view
//   - row_normalize: the three norm types, a user functor triple, rows below eps left untouched
//     (cpp/tests/linalg/normalize.cu:38-98)
//   - mapThenSumReduce / map_reduce: sum against a host loop, a two-array map (squared difference,
//     as linalg/detail/mean_squared_error.cuh calls it), and the min = 1 / max = 5 known answers of
//     cpp/tests/linalg/map_then_reduce.cu:133-171
//   - shape errors -> raft::logic_error, unsupported strided output type -> raft::exception
// Prints one line per check and "ALL PASSED" / exits non-zero.
#include <raft/linalg/coalesced_reduction.cuh>
#include <raft/linalg/map_reduce.cuh>
#include <raft/linalg/map_then_reduce.cuh>
#include <raft/linalg/norm.cuh>
#include <raft/linalg/normalize.cuh>
#include <raft/linalg/reduce.cuh>
#include <raft/linalg/reduce_cols_by_key.cuh>
#include <raft/linalg/reduce_rows_by_key.cuh>
#include <raft/linalg/strided_reduction.cuh>
#include <raft/matrix/argmax.cuh>
#include <raft/matrix/argmin.cuh>

#include <cmath>
#include <limits>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

static int g_fail = 0;
#define CHECK(cond, name)                         \
  do {                                            \
    const bool ok_ = (cond);                      \
    std::printf("%s %s\n", ok_ ? "ok  " : "FAIL", name); \
    if (!ok_) ++g_fail;                           \
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

// the reference's hybrid rule (cpp/tests/test_utils.h:31-45)
static bool approx(double a, double b, double eps)
{
  const double d = std::fabs(a - b);
  const double m = std::fmax(std::fabs(a), std::fabs(b));
  return (d > eps ? d / m : d) <= eps;
}
template <typename T>
static bool all_approx(const std::vector<double>& e, const std::vector<T>& a, double eps)
{
  if (e.size() != a.size()) return false;
  for (size_t i = 0; i < e.size(); ++i)
    if (!approx(e[i], double(a[i]), eps)) {
      std::printf("   mismatch at %zu: expect %.9g got %.9g\n", i, e[i], double(a[i]));
      return false;
    }
  return true;
}

template <typename T, typename IdxT = int>
struct ValueToKVP {
  __host__ __device__ raft::KeyValuePair<IdxT, T> operator()(T value, IdxT idx) { return {idx, value}; }
};
template <typename K, typename V>
struct ArgMaxOp {
  __host__ __device__ raft::KeyValuePair<K, V> operator()(raft::KeyValuePair<K, V> a, raft::KeyValuePair<K, V> b)
  {
    return (a.value > b.value || (a.value == b.value && a.key <= b.key)) ? a : b;
  }
};

static std::vector<float> random_matrix(int rows, int cols, unsigned seed)
{
  std::mt19937 gen(seed);
  std::uniform_real_distribution<float> dist(-1.f, 1.f);
  std::vector<float> h(size_t(rows) * cols);
  for (auto& x : h)
    x = dist(gen);
  return h;
}

static void test_simple_max()
{
  raft::resources handle;
  std::vector<float> h = {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12};
  DevBuf<float> d(h);
  {
    auto m = raft::make_device_matrix_view<const float, int, raft::row_major>(d.p, 3, 4);
    DevBuf<float> o(3), oc(4);
    raft::linalg::reduce<raft::Apply::ALONG_ROWS>(handle, m, raft::make_device_vector_view<float, int>(o.p, 3), 0.0f,
                                                  false, raft::identity_op(), raft::max_op(), raft::identity_op());
    raft::linalg::reduce<raft::Apply::ALONG_COLUMNS>(handle, m, raft::make_device_vector_view<float, int>(oc.p, 4),
                                                     0.0f, false, raft::identity_op(), raft::max_op(),
                                                     raft::identity_op());
    CHECK((o.host() == std::vector<float>{4, 8, 12}), "simple max, row-major, along rows");
    CHECK((oc.host() == std::vector<float>{9, 10, 11, 12}), "simple max, row-major, along columns");
  }
  {
    auto m = raft::make_device_matrix_view<const float, int, raft::col_major>(d.p, 3, 4);
    DevBuf<float> o(3), oc(4);
    raft::linalg::reduce<raft::Apply::ALONG_ROWS>(handle, m, raft::make_device_vector_view<float, int>(o.p, 3), 0.0f,
                                                  false, raft::identity_op(), raft::max_op(), raft::identity_op());
    raft::linalg::reduce<raft::Apply::ALONG_COLUMNS>(handle, m, raft::make_device_vector_view<float, int>(oc.p, 4),
                                                     0.0f, false, raft::identity_op(), raft::max_op(),
                                                     raft::identity_op());
    CHECK((o.host() == std::vector<float>{10, 11, 12}), "simple max, col-major, along rows");
    CHECK((oc.host() == std::vector<float>{3, 6, 9, 12}), "simple max, col-major, along columns");
  }
}

template <bool rowMajor, bool alongRows>
static void test_reduce_sq_sqrt(int rows, int cols)
{
  auto h = random_matrix(rows, cols, 1234);
  DevBuf<float> d(h);
  const int n_out = alongRows ? rows : cols;
  const int n_red = alongRows ? cols : rows;
  std::vector<double> e(n_out, 0.0);
  for (int o = 0; o < n_out; ++o) {
    for (int j = 0; j < n_red; ++j) {
      const int r = alongRows ? o : j, c = alongRows ? j : o;
      const float x = h[rowMajor ? size_t(r) * cols + c : size_t(c) * rows + r];
      e[o] += double(x * x);
    }
  }
  DevBuf<float> out(n_out);
  cudaStream_t s;
  cudaStreamCreate(&s);
  raft::linalg::reduce<rowMajor, alongRows>(out.p, d.p, cols, rows, 0.0f, s, false, raft::sq_op(), raft::add_op(),
                                            raft::sqrt_op());
  cudaStreamSynchronize(s);
  std::vector<double> e1(n_out);
  for (int o = 0; o < n_out; ++o)
    e1[o] = std::sqrt(e[o]);
  char name[128];
  std::snprintf(name, sizeof(name), "reduce sq/add/sqrt %dx%d rowMajor=%d alongRows=%d", rows, cols, rowMajor, alongRows);
  auto got = out.host();
  CHECK(all_approx(e1, got, 2e-6), name);
  raft::linalg::reduce<rowMajor, alongRows>(out.p, d.p, cols, rows, 0.0f, s, true, raft::sq_op(), raft::add_op(),
                                            raft::sqrt_op());
  cudaStreamSynchronize(s);
  std::vector<double> e2(n_out);
  for (int o = 0; o < n_out; ++o)
    e2[o] = std::sqrt(double(got[o]) + e[o]);
  std::snprintf(name, sizeof(name), "  ... inplace second pass");
  CHECK(all_approx(e2, out.host(), 2e-6), name);
  cudaStreamDestroy(s);
}

static void test_kvp(int rows, int cols)
{
  auto h = random_matrix(rows, cols, 99);
  for (size_t i = 0; i < h.size(); i += 3)
    h[i] = 0.5f;  // ties
  DevBuf<float> d(h);
  using KV = raft::KeyValuePair<int, float>;
  DevBuf<KV> out(rows);
  raft::linalg::reduce<true, true, float, KV, int>(out.p, d.p, cols, rows, KV{0, 0.0f}, nullptr, false,
                                                   ValueToKVP<float, int>(), ArgMaxOp<int, float>(),
                                                   raft::identity_op());
  auto got = out.host();
  bool ok  = true;
  for (int r = 0; r < rows && ok; ++r) {
    KV best{0, 0.0f};
    for (int c = 0; c < cols; ++c) {
      const float v = h[size_t(r) * cols + c];
      if (v > best.value || (v == best.value && c < best.key)) best = KV{c, v};
    }
    ok = got[r].key == best.key && got[r].value == best.value;
    if (!ok) std::printf("   row %d expect {%d,%g} got {%d,%g}\n", r, best.key, best.value, got[r].key, got[r].value);
  }
  char name[96];
  std::snprintf(name, sizeof(name), "key/value argmax with user functors %dx%d (bit exact)", rows, cols);
  CHECK(ok, name);
  // raft::argmin_op with +inf start
  raft::linalg::coalescedReduction<float, KV, int>(out.p, d.p, cols, rows, KV{0, INFINITY}, nullptr, false,
                                                   ValueToKVP<float, int>(), raft::argmin_op(), raft::identity_op());
  got = out.host();
  ok  = true;
  for (int r = 0; r < rows && ok; ++r) {
    int bk   = 0;
    float bv = h[size_t(r) * cols];
    for (int c = 1; c < cols; ++c)
      if (h[size_t(r) * cols + c] < bv) {
        bv = h[size_t(r) * cols + c];
        bk = c;
      }
    ok = got[r].key == bk && got[r].value == bv;
  }
  CHECK(ok, "  ... coalescedReduction with raft::argmin_op (ties -> lowest index)");
}

static void test_norms(int rows, int cols)
{
  raft::resources handle;
  auto h = random_matrix(rows, cols, 7);
  DevBuf<float> d(h);
  auto m = raft::make_device_matrix_view<const float, int, raft::row_major>(d.p, rows, cols);
  DevBuf<float> r1(rows), r2(rows), c2(cols), cinf(cols);
  raft::linalg::norm<raft::linalg::L1Norm, raft::Apply::ALONG_ROWS>(handle, m,
                                                                    raft::make_device_vector_view<float, int>(r1.p, rows));
  raft::linalg::norm<raft::linalg::L2Norm, raft::Apply::ALONG_ROWS>(
    handle, m, raft::make_device_vector_view<float, int>(r2.p, rows), raft::sqrt_op());
  raft::linalg::norm<raft::linalg::L2Norm, raft::Apply::ALONG_COLUMNS>(
    handle, m, raft::make_device_vector_view<float, int>(c2.p, cols));
  raft::linalg::norm<raft::linalg::LinfNorm, raft::Apply::ALONG_COLUMNS>(
    handle, m, raft::make_device_vector_view<float, int>(cinf.p, cols));
  std::vector<double> e1(rows, 0), e2(rows, 0), ec(cols, 0), ei(cols, 0);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const float x = h[size_t(r) * cols + c];
      e1[r] += std::fabs(x);
      e2[r] += double(x * x);
      ec[c] += double(x * x);
      ei[c] = std::fmax(ei[c], std::fabs(x));
    }
  for (auto& v : e2)
    v = std::sqrt(v);
  char name[96];
  std::snprintf(name, sizeof(name), "norm L1 rows %dx%d", rows, cols);
  CHECK(all_approx(e1, r1.host(), 1e-5), name);
  CHECK(all_approx(e2, r2.host(), 1e-5), "  ... L2 rows with sqrt_op");
  CHECK(all_approx(ec, c2.host(), 1e-5), "  ... L2 columns (squared)");
  CHECK(all_approx(ei, cinf.host(), 0.0), "  ... Linf columns (exact)");
  bool threw = false;
  try {
    raft::linalg::norm<raft::linalg::L0PseudoNorm, raft::Apply::ALONG_ROWS>(
      handle, m, raft::make_device_vector_view<float, int>(r1.p, rows));
  } catch (const raft::exception&) {
    threw = true;
  }
  CHECK(threw, "  ... L0 pseudo-norm throws");
}

static void test_lambdas(int rows, int cols)
{
  auto h = random_matrix(rows, cols, 21);
  DevBuf<float> d(h);
  std::vector<float> mu(cols), w(cols);
  for (int c = 0; c < cols; ++c) {
    mu[c] = 0.01f * c;
    w[c]  = 1.0f + 0.001f * c;
  }
  DevBuf<float> dmu(mu), dw(w);

  const float* w_p  = dw.p;
  // row-wise weighted sum: main_op uses the column index (as stats::weighted_mean does)
  DevBuf<float> o1(rows);
  raft::linalg::reduce<true, true>(
    o1.p, d.p, cols, rows, 0.0f, nullptr, false, [w_p] __device__(float x, int j) { return x * w_p[j]; },
    raft::add_op(), [cols] __device__(float s) { return s / float(cols); });
  std::vector<double> e1(rows, 0);
  for (int r = 0; r < rows; ++r) {
    for (int c = 0; c < cols; ++c)
      e1[r] += double(h[size_t(r) * cols + c] * w[c]);
    e1[r] = double(float(e1[r]) / float(cols));
  }
  CHECK(all_approx(e1, o1.host(), 1e-5), "device lambdas: weighted row mean (index-dependent main_op)");
  // column-wise centred sum of squares: main_op uses the ROW index on the strided path
  std::vector<float> rowshift(rows);
  for (int r = 0; r < rows; ++r)
    rowshift[r] = 0.001f * (r % 17);
  DevBuf<float> drs(rowshift);
  const float* rs_p = drs.p;
  DevBuf<float> o2(cols);
  raft::linalg::reduce<true, false>(
    o2.p, d.p, cols, rows, 0.0f, nullptr, false,
    [rs_p] __device__(float x, int i) {
      const float t = x - rs_p[i];
      return t * t;
    },
    raft::add_op(), raft::sqrt_op());
  std::vector<double> e2(cols, 0);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const float t = h[size_t(r) * cols + c] - rowshift[r];
      e2[c] += double(t * t);
    }
  for (auto& v : e2)
    v = std::sqrt(v);
  CHECK(all_approx(e2, o2.host(), 1e-5), "device lambdas: column reduce with row-index-dependent main_op");

}

static void test_rows_by_key(int nobs, int cols, int nkeys, bool weighted)
{
  raft::resources handle;
  auto h = random_matrix(nobs, cols, 5);
  std::mt19937 gen(11);
  std::vector<uint32_t> keys(nobs);
  for (auto& k : keys)
    k = gen() % nkeys;
  std::vector<float> w(nobs);
  for (auto& x : w)
    x = 0.5f + (gen() % 100) * 0.01f;
  DevBuf<float> dA(h), dw(w), sums(size_t(nkeys) * cols);
  DevBuf<uint32_t> dk(keys);
  DevBuf<char> scratch(nobs);
  std::vector<double> e(size_t(nkeys) * cols, 0.0);
  for (int i = 0; i < nobs; ++i)
    for (int c = 0; c < cols; ++c) {
      float v = h[size_t(i) * cols + c];
      if (weighted) v *= w[i];
      e[size_t(keys[i]) * cols + c] += v;
    }
  // the reference's mdspan convention: (cols, nobs) view over [nobs][cols] memory (tests :134-147)
  auto A_view    = raft::make_device_matrix_view<const float, int, raft::row_major>(dA.p, cols, nobs);
  auto keys_view = raft::make_device_vector_view<const uint32_t, int>(dk.p, nobs);
  auto sums_view = raft::make_device_matrix_view<float, int, raft::row_major>(sums.p, cols, nkeys);
  auto char_view = raft::make_device_vector_view<char, int>(scratch.p, nobs);
  if (weighted) {
    raft::linalg::reduce_rows_by_key(handle, A_view, keys_view, sums_view, nkeys, char_view,
                                     std::make_optional(raft::make_device_vector_view<const float, int>(dw.p, nobs)),
                                     true);
  } else {
    raft::linalg::reduce_rows_by_key<float, uint32_t, float, int>(handle, A_view, keys_view, sums_view, nkeys,
                                                                  char_view);
  }
  char name[96];
  std::snprintf(name, sizeof(name), "reduce_rows_by_key %dx%d, %d keys%s", nobs, cols, nkeys, weighted ? ", weighted" : "");
  CHECK(all_approx(e, sums.host(), 1e-5), name);
  // raw-pointer overload, accumulate on top
  raft::linalg::reduce_rows_by_key(dA.p, cols, dk.p, weighted ? dw.p : static_cast<float*>(nullptr), scratch.p, nobs,
                                   cols, nkeys, sums.p, nullptr, false);
  for (auto& v : e)
    v *= 2;
  CHECK(all_approx(e, sums.host(), 2e-5), "  ... raw-pointer overload, reset_sums = false");
}

static void test_cols_by_key(int rows, int cols, int nkeys)
{
  raft::resources handle;
  auto h = random_matrix(rows, cols, 8);
  std::mt19937 gen(3);
  std::vector<int> keys(cols);
  for (auto& k : keys)
    k = gen() % nkeys;
  DevBuf<float> d(h), out(size_t(rows) * nkeys);
  DevBuf<int> dk(keys);
  std::vector<double> e(size_t(rows) * nkeys, 0.0);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c)
      e[size_t(r) * nkeys + keys[c]] += h[size_t(r) * cols + c];
  auto dv = raft::make_device_matrix_view<const float, int, raft::row_major>(d.p, rows, cols);
  auto kv = raft::make_device_vector_view<const int, int>(dk.p, cols);
  auto ov = raft::make_device_matrix_view<float, int, raft::row_major>(out.p, rows, nkeys);
  raft::linalg::reduce_cols_by_key(handle, dv, kv, ov);  // nkeys inferred from the output view
  char name[96];
  std::snprintf(name, sizeof(name), "reduce_cols_by_key %dx%d, %d keys (nkeys inferred)", rows, cols, nkeys);
  CHECK(all_approx(e, out.host(), 1e-3), name);
}

static void test_matrix_arg()
{
  // cpp/tests/matrix/argmin.cu:71-75 and argmax.cu:71-72: the same 3x4 matrix -> {0,3,3} / {3,0,2}
  raft::resources handle;
  std::vector<float> h = {0.1f, 0.2f, 0.3f, 0.4f, 0.4f, 0.3f, 0.2f, 0.1f, 0.2f, 0.3f, 0.5f, 0.0f};
  DevBuf<float> d(h);
  DevBuf<int> o(3);
  auto in = raft::make_device_matrix_view<const float, std::uint32_t, raft::row_major>(d.p, 3u, 4u);
  raft::matrix::argmin(handle, in, raft::make_device_vector_view<int, std::uint32_t>(o.p, 3u));
  CHECK((o.host() == std::vector<int>{0, 3, 3}), "matrix::argmin known answer {0,3,3}");
  raft::matrix::argmax(handle, in, raft::make_device_vector_view<int, std::uint32_t>(o.p, 3u));
  CHECK((o.host() == std::vector<int>{3, 0, 2}), "matrix::argmax known answer {3,0,2}");
  std::vector<double> hd(h.begin(), h.end());
  DevBuf<double> dd(hd);
  DevBuf<short> os(3);  // an index type the C ABI does not name: header-only kernels
  auto ind = raft::make_device_matrix_view<const double, std::uint32_t, raft::row_major>(dd.p, 3u, 4u);
  raft::matrix::argmin(handle, ind, raft::make_device_vector_view<short, std::uint32_t>(os.p, 3u));
  CHECK((os.host() == std::vector<short>{0, 3, 3}), "matrix::argmin double -> short index");
  const int rows = 5000, cols = 200;
  auto big = random_matrix(rows, cols, 77);
  for (size_t i = 0; i < big.size(); i += 5)
    big[i] = -0.25f;  // ties
  DevBuf<float> db(big);
  DevBuf<int> ob(rows);
  raft::matrix::argmin(handle, raft::make_device_matrix_view<const float, int, raft::row_major>(db.p, rows, cols),
                       raft::make_device_vector_view<int, int>(ob.p, rows));
  auto got = ob.host();
  bool ok  = true;
  for (int r = 0; r < rows && ok; ++r) {
    int bk = 0;
    for (int c = 1; c < cols; ++c)
      if (big[size_t(r) * cols + c] < big[size_t(r) * cols + bk]) bk = c;
    ok = got[r] == bk;
  }
  CHECK(ok, "matrix::argmin 5000x200 with ties (lowest index)");
}

// L3 norm through user functors: |x|^3 summed, cube root at the end
struct CubeAbs {
  __host__ __device__ float operator()(float x, int) const { return fabsf(x) * x * x; }
};
struct CubeRoot {
  __host__ __device__ float operator()(float x) const { return cbrtf(x); }
};

static void test_row_normalize(int rows, int cols)
{
  raft::resources handle;
  auto h = random_matrix(rows, cols, 21);
  for (int c = 0; c < cols; ++c)
    h[size_t(rows / 2) * cols + c] = 0.f;  // a zero row: must not be written
  DevBuf<float> d(h);
  auto in = raft::make_device_matrix_view<const float, int, raft::row_major>(d.p, rows, cols);
  char name[96];
  for (int t = 0; t < 4; ++t) {
    std::vector<float> sentinel(size_t(rows) * cols, 7.f);
    DevBuf<float> o(sentinel);
    auto out = raft::make_device_matrix_view<float, int, raft::row_major>(o.p, rows, cols);
    if (t == 0) raft::linalg::row_normalize<raft::linalg::L1Norm>(handle, in, out);
    if (t == 1) raft::linalg::row_normalize<raft::linalg::L2Norm>(handle, in, out);
    if (t == 2) raft::linalg::row_normalize<raft::linalg::LinfNorm>(handle, in, out);
    if (t == 3) raft::linalg::row_normalize(handle, in, out, 0.f, CubeAbs{}, raft::add_op{}, CubeRoot{});
    std::vector<double> e(size_t(rows) * cols);
    for (int r = 0; r < rows; ++r) {
      double acc = 0;
      for (int c = 0; c < cols; ++c) {
        const double x = std::fabs(double(h[size_t(r) * cols + c]));
        acc            = t == 0 ? acc + x : t == 1 ? acc + x * x : t == 2 ? std::fmax(acc, x) : acc + x * x * x;
      }
      const double nrm = t == 1 ? std::sqrt(acc) : t == 3 ? std::cbrt(acc) : acc;
      for (int c = 0; c < cols; ++c)
        e[size_t(r) * cols + c] = nrm <= 1e-8 ? 7.0 : double(h[size_t(r) * cols + c]) / nrm;
    }
    static const char* what[] = {"L1", "L2", "Linf", "user functors (L3)"};
    std::snprintf(name, sizeof(name), "row_normalize %s %dx%d", what[t], rows, cols);
    CHECK(all_approx(e, o.host(), 1e-5), name);
  }
  bool threw = false;
  try {
    DevBuf<float> o(size_t(rows) * cols);
    raft::linalg::row_normalize<raft::linalg::L2Norm>(
      handle, in, raft::make_device_matrix_view<float, int, raft::row_major>(o.p, rows, cols - 1));
  } catch (const raft::logic_error&) {
    threw = true;
  }
  CHECK(threw, "  ... column mismatch throws logic_error");
}

struct SqDiff {
  __host__ __device__ float operator()(float a, float b) const { return (a - b) * (a - b); }
};
struct MinOf {
  template <typename T>
  __host__ __device__ T operator()(T a, T b) const { return a < b ? a : b; }
};
struct MaxOf {
  template <typename T>
  __host__ __device__ T operator()(T a, T b) const { return a > b ? a : b; }
};

static void test_map_reduce()
{
  raft::resources handle;
  cudaStream_t stream = raft::resource::get_cuda_stream(handle);
  char name[96];
  for (size_t len : {size_t(1), size_t(1237), size_t(1024 * 1024), size_t(1024 * 1024 + 1), size_t(3 * 1000 * 1000 + 2)}) {
    std::mt19937 gen(1234);
    std::uniform_real_distribution<float> dist(-1.f, 1.f);
    std::vector<float> a(len), b(len);
    double sum = 0, sq = 0;
    for (size_t i = 0; i < len; ++i) {
      a[i] = dist(gen);
      b[i] = dist(gen);
      sum += a[i];
      sq += double((a[i] - b[i]) * (a[i] - b[i]));
    }
    DevBuf<float> da(a), db(b), of(1);
    DevBuf<double> od(1);
    raft::linalg::mapThenSumReduce(of.p, len, raft::identity_op{}, stream, da.p);
    std::snprintf(name, sizeof(name), "mapThenSumReduce identity float len %zu", len);
    CHECK(approx(sum, of.host()[0], 1e-3), name);
    raft::linalg::mapThenSumReduce(od.p, len, raft::identity_op{}, stream, da.p);
    CHECK(approx(sum, od.host()[0], 1e-6 * std::sqrt(double(len))), "  ... float -> double");
    raft::linalg::mapThenSumReduce<float, SqDiff, size_t, 256, const float*>(of.p, len, SqDiff{}, stream, da.p,
                                                                              (const float*)db.p);
    CHECK(approx(sq, of.host()[0], 1e-5), "  ... two arrays (squared difference)");
  }
  {  // known answers: values in [2, 3), one 1 and one 5 planted (map_then_reduce.cu:133-171)
    const int n = 1237;
    std::mt19937 gen(137);
    std::uniform_real_distribution<float> dist(2.f, 3.f);
    std::vector<float> h(n);
    for (auto& x : h)
      x = dist(gen);
    h[42]  = 1.f;
    h[337] = 5.f;
    DevBuf<float> d(h), o(1);
    DevBuf<double> o2(1);
    auto in = raft::make_device_vector_view<const float>(d.p, static_cast<std::uint32_t>(n));
    raft::linalg::map_reduce(handle, in, raft::make_device_scalar_view(o.p), std::numeric_limits<float>::max(),
                             raft::identity_op{}, MinOf{});
    CHECK(o.host()[0] == 1.f, "map_reduce min known answer 1");
    raft::linalg::map_reduce(handle, in, raft::make_device_scalar_view(o.p), std::numeric_limits<float>::min(),
                             raft::identity_op{}, MaxOf{});
    CHECK(o.host()[0] == 5.f, "map_reduce max known answer 5");
    raft::linalg::map_reduce(handle, in, raft::make_device_scalar_view(o2.p), double(std::numeric_limits<float>::min()),
                             raft::identity_op{}, raft::max_op{});
    CHECK(o2.host()[0] == 5.0, "  ... float -> double with raft::max_op (library path)");
  }
}

static void test_errors()
{
  raft::resources handle;
  DevBuf<float> d(12), o(5);
  auto m    = raft::make_device_matrix_view<const float, int, raft::row_major>(d.p, 3, 4);
  bool threw = false;
  try {
    raft::linalg::reduce<raft::Apply::ALONG_ROWS>(handle, m, raft::make_device_vector_view<float, int>(o.p, 5), 0.0f);
  } catch (const raft::logic_error&) {
    threw = true;
  }
  CHECK(threw, "wrong output length -> raft::logic_error");
  threw = false;
  try {
    using KV = raft::KeyValuePair<int, float>;
    DevBuf<KV> ko(4);
    raft::linalg::stridedReduction<float, KV, int>(ko.p, d.p, 4, 3, KV{0, 0.f}, nullptr, false, ValueToKVP<float, int>(),
                                                   raft::argmin_op(), raft::identity_op());
  } catch (const raft::exception&) {
    threw = true;
  }
  CHECK(threw, "key/value output on the strided path -> raft::exception");
  threw = false;
  try {
    DevBuf<float> out(8);
    DevBuf<int> k(3);
    auto ov = raft::make_device_matrix_view<float, int, raft::row_major>(out.p, 2, 4);
    raft::linalg::reduce_cols_by_key(handle, m, raft::make_device_vector_view<const int, int>(k.p, 3), ov);
  } catch (const raft::logic_error&) {
    threw = true;
  }
  CHECK(threw, "reduce_cols_by_key shape mismatch -> raft::logic_error");
}

int main()
{
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    std::printf("no CUDA device\n");
    return 2;
  }
  test_simple_max();
  for (int rows : {11, 1234})
    for (int cols : {7, 33, 128, 500}) {
      test_reduce_sq_sqrt<true, true>(rows, cols);
      test_reduce_sq_sqrt<true, false>(rows, cols);
      test_reduce_sq_sqrt<false, true>(rows, cols);
      test_reduce_sq_sqrt<false, false>(rows, cols);
      test_kvp(rows, cols);
    }
  test_reduce_sq_sqrt<true, true>(3, 100000);
  test_norms(1234, 33);
  test_norms(11, 500);
  test_lambdas(777, 65);
  test_rows_by_key(128, 32, 6, false);
  test_rows_by_key(128, 32, 3, true);
  test_rows_by_key(100000, 37, 32, false);
  test_rows_by_key(100000, 37, 2048, true);
  test_cols_by_key(9, 9999, 42);
  test_cols_by_key(1024, 1234, 127);
  test_matrix_arg();
  for (int cols : {3, 33, 128, 500, 1500, 5000, 20000})
    test_row_normalize(257, cols);
  test_map_reduce();
  test_errors();
  cudaDeviceSynchronize();
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    std::printf("FAIL pending CUDA error %s\n", cudaGetErrorString(e));
    return 1;
  }
  if (g_fail) {
    std::printf("%d CHECKS FAILED\n", g_fail);
    return 1;
  }
  std::printf("ALL PASSED\n");
  return 0;
}
