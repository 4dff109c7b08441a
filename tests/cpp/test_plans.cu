// Host-side checks of the launch planners (no kernel is launched, no GPU is needed: without a device the
// planners take 148 SMs). Invariants every plan must keep, whatever the shape:
//   column reduction    row ranges cover the rows; column blocks x row ranges are whole waves of the resident
//                       CTAs; the scratch the plan asks for is what col_reduce_scratch_bytes reports and stays
//                       under a caller's bound (the entry point that allocates nothing relies on it);
//   split rows          few long segments below 400 MB, more and at least 128 KB long above;
//   keyed row sums      windows cover the rows and fit 16-bit offsets; work units of 128..384 rows; the scratch
//                       regions do not overlap;
//   keyed column sums   the table form's shared memory fits one CTA, it has at least two stages, eight consumer
//                       warps up to 136 keys, a cell sees at most 128 additions between two flushes, and the
//                       three forms are chosen by key count and type as documented.
#include <raft_b200/detail/cols_by_key.cuh>
#include <raft_b200/detail/launch.cuh>
#include <raft_b200/detail/rows_by_key_sorted.cuh>

#include <cstdio>
#include <cstdlib>

using namespace raft_b200::detail;

static int g_fail = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      ++g_fail;                                            \
      std::printf("FAIL %s:%d: %s | ", __FILE__, __LINE__, #cond); \
      std::printf(__VA_ARGS__);                            \
      std::printf("\n");                                   \
    }                                                      \
  } while (0)

static const float* fake_ptr() { return reinterpret_cast<const float*>(uintptr_t(1) << 20); }  // 16-byte aligned, never read

static void col_plans()
{
  using State = typename state_for<float, raft_b200::op::Add>::type;
  const int sms = sm_count();
  const int64_t shapes[][2] = {{4096, 4096},   {8192, 8192},    {32768, 32768}, {1024, 32768}, {100000, 2048},
                               {16777216, 64}, {1000000, 512},  {3, 100000},    {20000, 1000}, {300, 70000},
                               {100000, 1024}, {65536, 4096},   {7, 9},         {40000, 8192}, {1, 1 << 20}};
  for (auto& sh : shapes) {
    const int64_t r = sh[0], c = sh[1];
    for (size_t cap : {size_t(0), size_t(1) << 20}) {
      const ColPlan p = plan_col_reduce<float, float, State>(fake_ptr(), r, c, c, cap);
      const int64_t ctas = int64_t(p.grid_x) * p.grid_y;
      const int64_t ranges = p.tma ? p.grid_x : p.grid_y;
      CHECK(p.rows_per_cta * ranges >= r, "%lld x %lld: %lld rows per range x %lld ranges", (long long)r, (long long)c,
            (long long)p.rows_per_cta, (long long)ranges);
      if (!p.tma && !p.tma2d && p.grid_y > 1)
        CHECK(ctas <= int64_t(sms) * 4, "%lld x %lld: %lld CTAs are more than one resident wave", (long long)r, (long long)c,
              (long long)ctas);
      const size_t need = col_reduce_scratch_bytes<float, float, raft_b200::op::Add>(fake_ptr(), r, c, c, cap);
      CHECK(need == p.scratch, "%lld x %lld: scratch %zu vs %zu", (long long)r, (long long)c, need, p.scratch);
      if (cap > 0) CHECK(p.scratch <= cap, "%lld x %lld: %zu bytes over the bound", (long long)r, (long long)c, p.scratch);
      if (p.tma2d) CHECK(size_t(c) * 4 <= (size_t(16) << 10), "%lld x %lld: tiled TMA on rows of %lld bytes", (long long)r,
                         (long long)c, (long long)c * 4);
    }
  }
}

static void split_rows()
{
  int seg = 0;
  row_reduce_scratch_bytes<double>(16, 4000000, 4, &seg);  // 256 MB: few long segments
  CHECK(seg >= 2 && seg <= 148 * 4 / 16 + 1, "16 x 4M: %d segments", seg);
  row_reduce_scratch_bytes<double>(2000, 200000, 4, &seg);  // 1.6 GB: more, at least 128 KB each
  CHECK(seg >= 2 && int64_t(200000) * 4 / seg >= (128 << 10), "2000 x 200000: %d segments", seg);
  row_reduce_scratch_bytes<double>(1000000, 128, 4, &seg);  // plenty of rows: a warp per row
  CHECK(seg == 0, "1M x 128: %d segments", seg);
  const size_t b = row_reduce_scratch_bytes<double>(1, int64_t(1) << 30, 4, &seg);
  CHECK(seg >= 148 && b >= size_t(seg) * sizeof(double), "1 x 2^30: %d segments, %zu bytes", seg, b);
}

static void keyed_rows()
{
  const int64_t shapes[][3] = {{10000000, 128, 1024}, {10000000, 128, 16}, {10000000, 128, 16384}, {100000, 37, 2048},
                               {70001, 48, 200},      {1 << 30, 4, 3},     {40000, 4096, 16},      {300000, 16, 16384}};
  for (auto& sh : shapes) {
    const int64_t n = sh[0], c = sh[1], k = sh[2];
    const SortedPlan p = plan_rows_by_key_sorted<float>(fake_ptr(), c, n, c, k, sizeof(double));
    CHECK(p.window_rows >= 1024 && p.window_rows <= 65536 && p.window_rows % 1024 == 0, "window %d", p.window_rows);
    CHECK(int64_t(p.n_windows) * p.window_rows >= n, "windows do not cover %lld rows", (long long)n);
    CHECK(p.group >= 1 && p.group <= kMaxGroup && int64_t(p.n_groups) * p.group >= p.n_windows, "groups");
    const int t = rbk_unit_target(n);
    CHECK(t >= 128 && t <= 384 && rbk_unit_cap(n) == t * 3 / 2, "unit target %d", t);
    const size_t offs[] = {p.off_perm, p.off_offs,   p.off_gcnt, p.off_uoffs,   p.off_ukey,
                           p.off_ufirst, p.off_ulen, p.off_fold, p.off_counter, p.off_part, p.total};
    for (int i = 0; i + 1 < 11; ++i)
      CHECK(offs[i] < offs[i + 1] && offs[i] % 256 == 0, "scratch region %d", i);
    CHECK(p.off_offs - p.off_perm >= size_t(n) * 4, "sorted offsets of %lld rows", (long long)n);
  }
}

static void keyed_cols()
{
  for (int k : {1, 33, 64, 100, 128, 136, 137, 200, 255}) {
    const CbkTablePlan p = plan_cols_by_key_table<float>(fake_ptr(), 2000, 200000, k);
    CHECK(p.ok, "%d keys: no plan", k);
    if (!p.ok) continue;
    CHECK(p.smem + 1024 <= (size_t(227) << 10), "%d keys: %zu bytes of shared memory", k, p.smem);
    CHECK(p.stages >= 2 && p.stages <= kCbkTableMaxStages, "%d keys: %d stages", k, p.stages);
    CHECK(p.warps == (k <= 136 ? 8 : 4), "%d keys: %d consumer warps", k, p.warps);
    // the narrow box where it makes room for a fourth stage beside eight tables: up to 128 keys
    CHECK(p.cols == (k <= 128 ? kCbkTableColsNarrow : kCbkTableCols), "%d keys: %d columns per box", k, p.cols);
    if (p.cols == kCbkTableColsNarrow) CHECK(p.stages >= 4, "%d keys: %d stages of the narrow box", k, p.stages);
    CHECK(int64_t(p.chunks_per_cta) * p.cols <= int64_t(kCbkTableMaxAdds) * p.warps * k + p.cols,
          "%d keys: %d boxes between two flushes", k, p.chunks_per_cta);
    CHECK(int64_t(p.y_split) * p.chunks_per_cta >= p.n_chunks, "%d keys: the boxes are not covered", k);
    CHECK(p.row_tiles_per_cta * ceil_div<int64_t>(p.n_row_tiles, p.row_tiles_per_cta) >= p.n_row_tiles, "row tiles");
  }
  CHECK(!plan_cols_by_key_table<float>(fake_ptr(), 2000, 200000, 256).ok, "256 keys do not fit a byte");
  CHECK(!plan_cols_by_key_table<float>(fake_ptr(), 2000, 200002, 100).ok, "rows off 16-byte boundaries");
  CHECK(!plan_cols_by_key_table<double>(reinterpret_cast<const double*>(fake_ptr()), 2000, 200000, 100).ok, "fp64");
  // which form takes what (large input; without a device the tensor-map entry point is missing and the table
  // form is not offered, so only the split between the two sorted forms can be checked here)
  Cbk32Plan p32;
  CHECK(cols_by_key_sorted_form<float>(fake_ptr(), 2000, 200000, 8, &p32) == 2, "8 keys: the walk form");
  CHECK(cols_by_key_sorted_form<double>(reinterpret_cast<const double*>(fake_ptr()), 2000, 200000, 64, &p32) == 2,
        "fp64, 64 keys: the walk form");
  CHECK(cols_by_key_sorted_form<float>(fake_ptr(), 2000, 200000, 1000, &p32) == 1, "1000 keys: a lane per segment");
  CHECK(cols_by_key_sorted_form<float>(fake_ptr(), 100, 100, 8, &p32) == 0, "small input: shared-memory atomics");
}

int main()
{
  col_plans();
  split_rows();
  keyed_rows();
  keyed_cols();
  if (g_fail == 0) std::printf("ALL PASSED\n");
  return g_fail == 0 ? 0 : 1;
}
