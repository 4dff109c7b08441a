// Host-side shape policies and launchers for the reduction kernels. Header-only templates:
// the shared library instantiates them for the operator set of the C ABI, the drop-in
// raft::linalg headers instantiate them for caller-supplied functors.
//
// All launchers are asynchronous on the given stream and return a cudaError_t; none of
// them synchronises. Kernels that need scratch memory (row partials, column partials) take
// it from the caller's workspace when one is passed and large enough, otherwise from a
// library-owned stream-ordered pool (allocation and free ordered on the same stream), as the
// reference does through rmm for its only scratch user (coalesced_reduction-inl.cuh:560).
#pragma once

#include "col_reduce.cuh"
#include "col_reduce_tma.cuh"
#include "col_reduce_tma2d.cuh"
#include "row_reduce.cuh"
#include "row_reduce_staged.cuh"
#include "row_reduce_tma.cuh"

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace raft_b200 {
namespace detail {

struct Workspace {
  void* ptr    = nullptr;
  size_t bytes = 0;
  int* status  = nullptr;  // device word that a ring kernel whose bounded wait ran out sets to 1 (null: none)
};

// Library-owned stream-ordered memory pool, one per device, created on first use. The device's
// default pool gives freed memory back to the driver at the next synchronisation, so a caller
// that synchronises between calls would pay a fresh physical allocation (milliseconds) on every
// call; this pool keeps what it has (release threshold = unlimited). b2r_trim_scratch_pool()
// returns the cached memory. Falls back to the default pool if a pool cannot be created.
inline cudaMemPool_t scratch_pool()
{
  static cudaMemPool_t pools[64] = {};
  static bool tried[64]          = {};
  static std::mutex lock;
  int dev                        = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> g(lock);  // first use on a device from several host threads at once
  if (!tried[dev]) {
    tried[dev]            = true;
    cudaMemPoolProps prop = {};
    prop.allocType        = cudaMemAllocationTypePinned;
    prop.handleTypes      = cudaMemHandleTypeNone;
    prop.location.type    = cudaMemLocationTypeDevice;
    prop.location.id      = dev;
    cudaMemPool_t pool    = nullptr;
    if (cudaMemPoolCreate(&pool, &prop) == cudaSuccess) {
      unsigned long long keep = ~0ull;
      if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) == cudaSuccess) {
        pools[dev] = pool;
      } else {
        cudaMemPoolDestroy(pool);
      }
    }
    (void)cudaGetLastError();
  }
  return pools[dev];
}

// Stream-ordered scratch with a caller-provided fast path.
class Scratch {
 public:
  Scratch(const Workspace& ws, size_t need, cudaStream_t stream) : stream_(stream)
  {
    if (need == 0) return;
    if (ws.ptr != nullptr && ws.bytes >= need) {
      ptr_ = ws.ptr;
    } else {
      cudaMemPool_t pool = scratch_pool();
      err_   = pool != nullptr ? cudaMallocFromPoolAsync(&ptr_, need, pool, stream) : cudaMallocAsync(&ptr_, need, stream);
      owned_ = err_ == cudaSuccess;
    }
  }
  ~Scratch()
  {
    if (owned_) cudaFreeAsync(ptr_, stream_);
  }
  Scratch(const Scratch&)            = delete;
  Scratch& operator=(const Scratch&) = delete;
  void* get() const { return ptr_; }
  cudaError_t error() const { return err_; }

 private:
  cudaStream_t stream_;
  void* ptr_       = nullptr;
  bool owned_      = false;
  cudaError_t err_ = cudaSuccess;
};

inline int sm_count()
{
  static std::atomic<int> cached[64];  // zero-initialised; a racing first use stores the same value twice
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Launch-shape knobs. The defaults are the measured best on B200; the environment
// variables exist so that a benchmark can sweep them without rebuilding.
struct Tuning {
  int row_ctas_per_sm      = 0;   // B2R_ROW_CPS   row-kernel CTAs per SM at most (0: 256, i.e. one batch per warp; 8 = two resident waves of long-lived CTAs)
  int row_chunk_threshold  = 4;   // B2R_ROW_CHUNK rows with >= this many passes per lane use kChunks
  int row_cpl              = 0;   // B2R_ROW_CPL   chunks of a row per lane and pass: 1, 2, 4 (0: by row length)
  int col_ctas_per_sm      = 4;   // B2R_COL_CPS   column-partial CTAs per SM (one resident wave)
  int col_gy_round         = 1;   // B2R_COL_GY_ROUND row ranges of the column-partial plan 1: rounded down to whole waves, 2: up
  int split_min_kb         = 0;   // B2R_SPLIT_MIN_KB shortest segment of a split row, KiB (0: 32, 128 for inputs of 400 MB and more)
  int split_ctas_per_sm    = 0;   // B2R_SPLIT_CPS split-row CTAs per SM aimed for (0: 4, 16 for inputs of 400 MB and more)
  int key_block_rows       = 8192;  // B2R_KEY_BLOCK  rows per sorted block (rows-by-key, table algorithm)
  int key_window_rows      = 0;     // B2R_KEY_WINDOW rows per sort window (rows-by-key, sorted algorithm; 0: auto)
  int key_unit_rows        = 0;     // B2R_KEY_UNIT_ROWS rows of one key a warp sums into one partial row (0: by size, 128..384)
  int key_algo             = 0;     // B2R_KEY_ALGO   0: by size, 1: shared-memory table, 2: sort then stream, 3: one-launch kernel (<= 32768 rows)
  int colkey_algo          = 0;     // B2R_COLKEY_ALGO 0: auto, 1: shared-memory atomics, 2: sorted tiles, a lane per segment, 3: sorted tiles, a warp walking its keys, 4: table cells (fp32, up to 255 keys)
  int colkey32_ch          = 0;     // B2R_COLKEY32_CH columns per chunk of the walk form of the keyed column sums (0: the longest that fits)
  int colkey32_rt          = 16;    // B2R_COLKEY32_RT rows per tile of that form: 8, 16 or 32
  int colkey_walk_max_keys = 32;    // B2R_COLKEY_WALK_MAX most keys for which that form is chosen by itself (fp32: the table form takes over)
  int colkey_table_cols    = 0;     // B2R_COLKEY_TABLE_COLS columns of a box of the table form: 228, 188 (0: the narrow one when it makes room for a fourth stage)
  int colkey_table_w8_max  = 136;   // B2R_COLKEY_TABLE_W8 most keys with eight consumer warps (their tables leave room for fewer stages)
  int colkey_table_y       = 0;     // B2R_COLKEY_TABLE_Y column splits of the table form (0: planned)
  int colkey_table_max_keys = 255;  // B2R_COLKEY_TABLE_MAX_KEYS most keys for the table form of the keyed column sums (fp32)
  int colkey_tma           = 1;     // B2R_COLKEY_TMA 1: TMA-staged ring for the sorted column tiles, 2: off
  int col_tma              = 1;     // B2R_COL_TMA    1: TMA-staged tiles for narrow contiguous column reductions, 2: off
  int col_tma_tile_kb      = 32;    // B2R_COL_TMA_KB tile size of the TMA ring, KiB
  int col_tma2d_min_mb     = 256;   // B2R_COL_TMA2D_MB smallest matrix (MiB) for the tiled-TMA kernel of wide matrices
  int col_tma2d_max_row_kb = 16;    // B2R_COL_TMA2D_ROW_KB longest row (KiB) for it: beyond, whole waves of the register-staged kernel are faster
  int tma_stages           = 4;     // B2R_TMA_STAGES stages of the TMA ring (2..8)
  int row_tma              = 0;     // B2R_ROW_TMA    ring kernel for short contiguous rows: unset = by shape, 1: wherever it fits, 2: never
  int row_ring_min_vec     = 8;     // B2R_ROW_RING_MINVEC shortest row (16-byte vectors) that takes the ring kernel by itself
  int row_ring_max_vec     = 128;   // B2R_ROW_RING_MAXVEC longest such row
  int row_ring_min_mb      = 1024;  // B2R_ROW_RING_MIN_MB smallest matrix (MiB) that takes it by itself
  int row_shifted_min      = 48;    // B2R_ROW_SHIFTED_MIN shortest row off 16-byte boundaries that takes aligned vector loads
  int row_tma_tile_kb      = 32;    // B2R_ROW_TMA_KB tile size of the row kernel's ring, KiB
  int row_tma_stages       = 4;     // B2R_ROW_TMA_STAGES
  int row_bpc_mode         = 1;     // B2R_ROW_BPC row batches per CTA 1: a multiple of 8 only when that costs under 7 %, 2: always a multiple of 8, 3: odd
  int row_staged           = 1;     // B2R_ROW_STAGED  1: shared-memory staging for contiguous rows off 16-byte boundaries, 2: off
  int row_staged_aligned   = 1;     // B2R_ROW_STAGED_ALIGNED aligned rows staged 1: when the direct kernel would leave a tenth of its load slots empty, 2: always, 3: never
  int row_staged_aligned_max = 800;  // B2R_ROW_STAGED_ALIGNED_MAX longest aligned row (elements) staged by rule 1
  int row_staged_max       = 1024;   // B2R_ROW_STAGED_MAX longest such row (elements) that is staged
  int row_staged_min_kb    = 32768;  // B2R_ROW_STAGED_MIN_KB smallest matrix (KiB) that is staged: aligned rows up to 64 elements; twice that off the boundaries
  int row_staged_wide_min_kb = 131072;  // B2R_ROW_STAGED_WIDE_MIN_KB the same for longer rows off the boundaries; twice that on them
  int row_staged_tile_kb   = 48;    // B2R_ROW_STAGED_KB tile size of that ring, KiB
  int row_staged_ring_kb   = 100;   // B2R_ROW_STAGED_RING_KB shared memory of one CTA's ring, KiB (100: two CTAs per SM)
  int row_split_ring       = 1;     // B2R_ROW_SPLIT_RING 1: ring of bulk copies for a handful of very long rows, 2: off
  int row_split_ring_min_mb = 64;   // B2R_ROW_SPLIT_RING_MB shortest row (MiB) that takes it
  int dep_launch           = 1;     // B2R_DEP_LAUNCH 1: kernels that begin with grid_dep_sync() are launched with programmatic stream serialization, 2: ordinary launches
  int normalize_ctas_per_sm = 0;    // B2R_NORMALIZE_CPS row_normalize CTAs per SM at most (0: 256, short-lived CTAs; 8: two resident waves)
  int wait_limit_ms        = 1000;  // B2R_WAIT_LIMIT_MS bound of every mbarrier wait inside the ring kernels, milliseconds
  int test_skip_tile       = 0;     // B2R_TEST_SKIP_TILE test hook: the producer of the first CTA never requests tile (value - 1)
};

inline int env_int(const char* name, int dflt)
{
  const char* s = std::getenv(name);
  if (s == nullptr || *s == 0) return dflt;
  const int v = std::atoi(s);
  return v > 0 ? v : dflt;
}

inline Tuning read_tuning_from_env()
{
  Tuning x;
  x.row_ctas_per_sm      = env_int("B2R_ROW_CPS", x.row_ctas_per_sm);
  x.row_chunk_threshold  = env_int("B2R_ROW_CHUNK", x.row_chunk_threshold);
  x.row_cpl              = env_int("B2R_ROW_CPL", x.row_cpl);
  x.col_ctas_per_sm      = env_int("B2R_COL_CPS", x.col_ctas_per_sm);
  x.col_gy_round         = env_int("B2R_COL_GY_ROUND", x.col_gy_round);
  x.split_min_kb         = env_int("B2R_SPLIT_MIN_KB", x.split_min_kb);
  x.split_ctas_per_sm    = env_int("B2R_SPLIT_CPS", x.split_ctas_per_sm);
  x.key_block_rows       = env_int("B2R_KEY_BLOCK", x.key_block_rows);
  x.key_window_rows      = env_int("B2R_KEY_WINDOW", x.key_window_rows);
  x.key_unit_rows        = env_int("B2R_KEY_UNIT_ROWS", x.key_unit_rows);
  x.key_algo             = env_int("B2R_KEY_ALGO", x.key_algo);
  x.colkey_algo          = env_int("B2R_COLKEY_ALGO", x.colkey_algo);
  x.colkey32_ch          = env_int("B2R_COLKEY32_CH", x.colkey32_ch);
  x.colkey32_rt          = env_int("B2R_COLKEY32_RT", x.colkey32_rt);
  x.colkey_walk_max_keys = env_int("B2R_COLKEY_WALK_MAX", x.colkey_walk_max_keys);
  x.colkey_table_cols    = env_int("B2R_COLKEY_TABLE_COLS", x.colkey_table_cols);
  x.colkey_table_w8_max  = env_int("B2R_COLKEY_TABLE_W8", x.colkey_table_w8_max);
  x.colkey_table_y       = env_int("B2R_COLKEY_TABLE_Y", x.colkey_table_y);
  x.colkey_table_max_keys = env_int("B2R_COLKEY_TABLE_MAX_KEYS", x.colkey_table_max_keys);
  x.colkey_tma           = env_int("B2R_COLKEY_TMA", x.colkey_tma);
  x.col_tma              = env_int("B2R_COL_TMA", x.col_tma);
  x.col_tma_tile_kb      = env_int("B2R_COL_TMA_KB", x.col_tma_tile_kb);
  x.col_tma2d_min_mb     = env_int("B2R_COL_TMA2D_MB", x.col_tma2d_min_mb);
  x.col_tma2d_max_row_kb = env_int("B2R_COL_TMA2D_ROW_KB", x.col_tma2d_max_row_kb);
  x.tma_stages           = env_int("B2R_TMA_STAGES", x.tma_stages);
  if (x.tma_stages < 2) x.tma_stages = 2;
  if (x.tma_stages > 8) x.tma_stages = 8;
  x.row_tma              = env_int("B2R_ROW_TMA", x.row_tma);
  x.row_ring_min_vec     = env_int("B2R_ROW_RING_MINVEC", x.row_ring_min_vec);
  x.row_ring_max_vec     = env_int("B2R_ROW_RING_MAXVEC", x.row_ring_max_vec);
  x.row_ring_min_mb      = env_int("B2R_ROW_RING_MIN_MB", x.row_ring_min_mb);
  x.row_shifted_min      = env_int("B2R_ROW_SHIFTED_MIN", x.row_shifted_min);
  x.row_tma_tile_kb      = env_int("B2R_ROW_TMA_KB", x.row_tma_tile_kb);
  x.row_tma_stages       = env_int("B2R_ROW_TMA_STAGES", x.row_tma_stages);
  if (x.row_tma_stages < 2) x.row_tma_stages = 2;
  if (x.row_tma_stages > 8) x.row_tma_stages = 8;
  x.row_bpc_mode         = env_int("B2R_ROW_BPC", x.row_bpc_mode);
  x.row_staged           = env_int("B2R_ROW_STAGED", x.row_staged);
  x.row_staged_aligned   = env_int("B2R_ROW_STAGED_ALIGNED", x.row_staged_aligned);
  x.row_staged_aligned_max = env_int("B2R_ROW_STAGED_ALIGNED_MAX", x.row_staged_aligned_max);
  x.row_staged_max       = env_int("B2R_ROW_STAGED_MAX", x.row_staged_max);
  x.row_staged_min_kb    = env_int("B2R_ROW_STAGED_MIN_KB", x.row_staged_min_kb);
  x.row_staged_wide_min_kb = env_int("B2R_ROW_STAGED_WIDE_MIN_KB", x.row_staged_wide_min_kb);
  x.row_staged_tile_kb   = env_int("B2R_ROW_STAGED_KB", x.row_staged_tile_kb);
  x.row_staged_ring_kb   = env_int("B2R_ROW_STAGED_RING_KB", x.row_staged_ring_kb);
  if (x.row_staged_ring_kb > 200) x.row_staged_ring_kb = 200;
  x.row_split_ring       = env_int("B2R_ROW_SPLIT_RING", x.row_split_ring);
  x.row_split_ring_min_mb = env_int("B2R_ROW_SPLIT_RING_MB", x.row_split_ring_min_mb);
  x.dep_launch           = env_int("B2R_DEP_LAUNCH", x.dep_launch);
  x.normalize_ctas_per_sm = env_int("B2R_NORMALIZE_CPS", x.normalize_ctas_per_sm);
  x.wait_limit_ms        = env_int("B2R_WAIT_LIMIT_MS", x.wait_limit_ms);
  x.test_skip_tile       = env_int("B2R_TEST_SKIP_TILE", x.test_skip_tile);
  return x;
}

// The knobs are read from the environment ONCE, at the first call (a call costs no getenv
// afterwards); reload_tuning() reads them again, for a benchmark that sweeps them within one
// process. Reloading must not run concurrently with other calls into the library.
struct TuningCache {
  std::atomic<bool> ready{false};
  std::mutex lock;
  Tuning value;
};
inline TuningCache& tuning_cache()
{
  static TuningCache c;
  return c;
}
inline const Tuning& tuning()
{
  TuningCache& c = tuning_cache();
  if (!c.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> g(c.lock);
    if (!c.ready.load(std::memory_order_relaxed)) {
      c.value = read_tuning_from_env();
      c.ready.store(true, std::memory_order_release);
    }
  }
  return c.value;
}
inline void reload_tuning()
{
  TuningCache& c = tuning_cache();
  std::lock_guard<std::mutex> g(c.lock);
  c.value = read_tuning_from_env();
  c.ready.store(true, std::memory_order_release);
}

// Bound of the waits inside the ring kernels: the knob, unless the process has set one (b2r_set_wait_limit_ms).
inline std::atomic<unsigned>& wait_limit_override_ms()
{
  static std::atomic<unsigned> v{0};
  return v;
}
inline RingCtl ring_ctl(int* status)
{
  RingCtl c;
  c.status          = status;
  const unsigned ov = wait_limit_override_ms().load(std::memory_order_relaxed);
  c.limit_ns        = (unsigned long long)(ov != 0 ? ov : unsigned(tuning().wait_limit_ms)) * 1000000ull;
  c.skip_tile       = tuning().test_skip_tile - 1;
  return c;
}

// Opt-in to more than 48 KB of dynamic shared memory, remembered per (kernel, device): the driver
// call is made only when a kernel needs more than it was granted before.
inline cudaError_t ensure_dynamic_smem(const void* kern, size_t bytes)
{
  static std::mutex lock;
  static std::unordered_map<const void*, size_t> granted[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
  std::lock_guard<std::mutex> g(lock);
  size_t& have = granted[dev][kern];
  if (bytes <= have) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
  if (e == cudaSuccess) have = bytes;
  return e;
}
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kern, size_t bytes)
{
  return ensure_dynamic_smem(reinterpret_cast<const void*>(kern), bytes);
}

// Launch of a kernel that begins with grid_dep_sync(): with programmatic stream serialization its CTAs may be
// scheduled while the previous kernel of the stream drains (measured: about 1 us per kernel boundary). ONLY for
// kernels that call grid_dep_sync() before their first access to global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args)
{
  // Grids smaller than the machine are launched the ordinary way: scheduled early they are packed onto the few
  // SMs that happen to be free while the predecessor runs, and then run there side by side (the units kernel of
  // the keyed row sums, 9 CTAs of 1024 threads: 19 -> 40 us).
  const bool off = size_t(grid.x) * grid.y * grid.z < size_t(sm_count());
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = grid;
  cfg.blockDim           = block;
  cfg.dynamicSmemBytes   = smem;
  cfg.stream             = stream;
  cudaLaunchAttribute at[1];
  at[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs                                        = at;
  cfg.numAttrs                                     = (tuning().dep_launch == 1 && !off) ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

// Resident CTAs per SM of a kernel. The column kernels, the chunk mode of the row kernel and the queue-driven
// kernels launch one or two resident waves of long-lived CTAs and loop inside the kernel (measured on the
// register-staged column kernel: ~15 % faster than many short CTAs); the direct row kernels do the opposite (see
// launch_row_reduce).
template <typename Kernel>
inline int resident_ctas(Kernel kern, int tpb, size_t smem)
{
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, tpb, smem) != cudaSuccess || n < 1) {
    (void)cudaGetLastError();
    n = 1;
  }
  return n;
}

template <typename T>
inline bool aligned16(const T* p)
{
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <typename D, typename S>
__global__ void convert_kernel(D* dst, const S* src, int64_t n)
{
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = static_cast<D>(src[i]);
}

template <typename D, typename S>
inline cudaError_t launch_convert(D* dst, const S* src, int64_t n, cudaStream_t stream)
{
  if (n <= 0) return cudaSuccess;
  convert_kernel<D, S><<<unsigned(ceil_div<int64_t>(n, 256)), 256, 0, stream>>>(dst, src, n);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Row-wise (contiguous axis) reduction.
// ---------------------------------------------------------------------------------------
template <typename CarryT>
inline size_t row_reduce_scratch_bytes(int64_t n_rows, int64_t row_len, size_t in_size, int* n_seg_out)
{
  // One warp per row leaves the machine idle when there are few rows: below 16 warps' worth of
  // rows per SM, rows of 8 KB and more get a CTA each (n_seg = 1, no scratch), and are cut into
  // segments of at least 32 KB when even that gives too few CTAs.
  const int sms           = sm_count();
  const int64_t row_bytes = row_len * int64_t(in_size);
  int n_seg               = 0;  // 0: warp-per-row kernels
  if (n_rows < int64_t(sms) * 16 && row_bytes >= (int64_t(8) << 10)) {
    // few long segments while the launch and the fold of the partials still count (measured up to 270 MB), four
    // times as many CTAs with segments of at least 128 KB from 400 MB on (fp32 2000 x 200000: 5.99 -> 6.63 TB/s,
    // 200 x 2 000 000: 6.18 -> 6.66, 1024 x 131072: 5.08 -> 6.07; 16 x 4 000 000 would lose: 5.5 -> 4.9)
    const bool large      = n_rows * row_bytes >= (int64_t(400) << 20);
    const int cps         = tuning().split_ctas_per_sm > 0 ? tuning().split_ctas_per_sm : (large ? 16 : 4);
    const int min_kb      = tuning().split_min_kb > 0 ? tuning().split_min_kb : (large ? 128 : 32);
    const int64_t want    = ceil_div<int64_t>(int64_t(sms) * cps, n_rows);
    const int64_t max_seg = row_bytes / (int64_t(min_kb) << 10);
    n_seg                 = int(want < max_seg ? want : max_seg);
    if (n_seg < 1) n_seg = 1;
  }
  if (n_seg_out) *n_seg_out = n_seg;
  return n_seg > 1 ? align_up(size_t(n_rows) * n_seg * sizeof(CarryT), 256) : 0;
}

// Smallest matrix (bytes) for which the staged row reduction beats the direct kernels, measured with a
// cold L2: the ring needs a few tiles per CTA to get going, the direct kernels ramp up faster.
inline size_t staged_min_bytes(int64_t row_len, bool vec_ok)
{
  const size_t narrow = size_t(tuning().row_staged_min_kb) << 10;
  const size_t wide   = size_t(tuning().row_staged_wide_min_kb) << 10;
  // rows up to 64 elements: 32 MB on 16-byte boundaries, 64 MB off them; longer rows: 256 MB and 128 MB
  // (the direct kernels are at their best on long aligned rows)
  if (row_len <= 64) return vec_ok ? narrow : 2 * narrow;
  return vec_ok ? 2 * wide : wide;
}

// Shape of a launch of the shared-memory staged row kernels (row_reduce_staged.cuh,
// row_normalize_staged.cuh) over a contiguous matrix.
struct StagedPlan {
  bool ok;            // false: the rows do not fit the ring, take another kernel
  int m;              // every m-th row starts on a 16-byte boundary
  int64_t n_main;     // rows the staged kernel takes (a multiple of m); the rest goes to a direct kernel
  int G;              // lanes per row
  int rot;            // bank rotation per row slot, in vectors
  int stages;
  int64_t tile_rows;
  int64_t rows_per_cta;
  int64_t ctas;
  size_t stage_bytes;
  size_t smem;        // stages x stage_bytes
};

inline StagedPlan plan_staged_rows(int64_t n_rows, size_t row_bytes, int nvec, bool vec_ok)
{
  StagedPlan p{};
  // every m-th row starts on a boundary
  size_t gcd16 = 16;
  while (row_bytes % gcd16 != 0) gcd16 >>= 1;
  p.m                 = int(16 / gcd16);
  const int m         = p.m;
  const size_t budget = size_t(tuning().row_staged_tile_kb) << 10;
  p.n_main            = n_rows - n_rows % m;
  const size_t ring   = size_t(tuning().row_staged_ring_kb) << 10;
  // rows a tile may hold: the budget, less for small inputs so that every CTA still gets a few tiles
  // (two CTAs resident per SM with a ring of up to 100 KB, else one)
  const int64_t ctas0 = int64_t(sm_count()) * (ring <= (size_t(104) << 10) ? 2 : 1);
  int64_t max_rows    = int64_t(budget / row_bytes);
  const int64_t fit   = p.n_main / (ctas0 * 4);
  if (max_rows > fit) max_rows = fit;
  max_rows            = max_rows / m * m;
  if (max_rows < m) max_rows = m;
  if (!(size_t(max_rows) * row_bytes <= budget && 2 * (budget + 128) <= ring && p.n_main > 0)) return p;
  // Lanes per row and rows per tile: a tile is a whole number of passes of the 256 consumers
  // (256 / G rows each). What a lane does per row besides summing - set-up, shuffles, the store -
  // weighs more the fewer vectors it gets, so: the FEWEST lanes per row whose tiles still fill
  // seven tenths of the ring (the bytes in flight), else the choice that fills it best.
  // A last pass that is at least nine tenths busy counts as whole.
  int Gs            = 32;
  int64_t tile_rows = max_rows;  // rows too long for a whole pass: one partial pass with 32 lanes per row
  size_t best_fill  = 0;
  for (int g2 = 1; g2 <= 32; g2 <<= 1) {
    const int64_t rpp = kTmaConsumers / g2;
    int64_t tr        = max_rows / rpp * rpp;  // rpp is a multiple of 8, so of m
    if (max_rows * 10 >= ceil_div<int64_t>(max_rows, rpp) * rpp * 9) tr = max_rows;
    if (tr == 0 || (g2 > 1 && nvec < 2 * g2)) continue;
    const size_t tile = (size_t(tr) * row_bytes + 127) / 128 * 128;
    size_t n_st       = ring / tile;
    n_st              = n_st > size_t(kTmaMaxStages) ? size_t(kTmaMaxStages) : n_st;
    const size_t fill = n_st * tile;
    if (fill > best_fill) {
      best_fill = fill;
      Gs        = g2;
      tile_rows = tr;
    }
    if (fill * 10 >= ring * 7) break;
  }
  // Bank rotation, 16-byte loads only: eight lanes are served at a time, so with fewer than eight
  // lanes per row they sit on different rows, (row pitch + rot) vectors apart; with that distance
  // congruent to G modulo 2 G they fall into different banks. Single elements of rows off the
  // boundaries: the pitch is odd or twice an odd number, at worst a two-way conflict - not worth
  // the index arithmetic per element.
  p.rot         = (vec_ok && Gs < 8) ? (Gs - nvec % (2 * Gs) + 2 * Gs) % (2 * Gs) : 0;
  p.G           = Gs;
  p.tile_rows   = tile_rows;
  p.stage_bytes = (size_t(tile_rows) * row_bytes + 127) / 128 * 128;
  // what keeps HBM busy is the bytes in flight: as many stages as the ring holds
  int stages    = int(ring / p.stage_bytes);
  p.stages      = stages > kTmaMaxStages ? kTmaMaxStages : stages;
  p.smem        = size_t(p.stages) * p.stage_bytes;
  int64_t rpc   = ceil_div<int64_t>(p.n_main, ctas0);
  p.rows_per_cta = ceil_div<int64_t>(rpc, tile_rows) * tile_rows;
  p.ctas        = ceil_div<int64_t>(p.n_main, p.rows_per_cta);
  p.ok          = true;
  return p;
}

// `out` may point to a type other than the accumulator type OutT (what final_op returns).
template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp,
          typename StoreT = OutT>
cudaError_t launch_row_reduce(StoreT* out,
                              const InT* data,
                              int64_t n_rows,
                              int64_t row_len,
                              int64_t ld,
                              OutT init,
                              bool inplace,
                              MainOp main_op,
                              ReduceOp reduce_op,
                              FinalOp final_op,
                              cudaStream_t stream,
                              Workspace ws = Workspace{})
{
  constexpr int TPB = 256;
  constexpr int U   = 8;
  constexpr int V16 = vec16<InT>::value;
  if (n_rows <= 0) return cudaSuccess;

  const bool vec_ok = V16 > 1 && row_len % V16 == 0 && ld % V16 == 0 && aligned16(data);
  int n_seg         = 1;
  using CarryT      = typename state_for<OutT, ReduceOp>::type::carry_t;
  const size_t need = row_reduce_scratch_bytes<CarryT>(n_rows, row_len, sizeof(InT), &n_seg);

  if (n_seg >= 1 || row_len > int64_t(0x7fffffff)) {
    if (n_seg < 1) n_seg = 1;
    // long rows: CTA per (segment, row), then fold the segment partials
    Scratch scratch(ws, need, stream);
    if (scratch.error() != cudaSuccess) return scratch.error();
    CarryT* partial       = static_cast<CarryT*>(scratch.get());
    // every row must start on a 16-byte boundary; a ragged row end is handled by the kernel
    const bool vec_split  = V16 > 1 && aligned16(data) && (ld % V16 == 0 || n_rows == 1);
    const int vec         = vec_split ? V16 : 1;
    const int64_t nvec    = row_len / vec;
    int64_t seg_vecs      = ceil_div<int64_t>(nvec, n_seg);
    seg_vecs              = ceil_div<int64_t>(seg_vecs, TPB) * TPB;
    n_seg                 = int(ceil_div<int64_t>(nvec, seg_vecs));
    if (n_seg < 1) n_seg = 1;
    // Ring form (row_reduce_tma.cuh) for a handful of rows of at least `row_split_ring_min_mb` MiB each: one CTA
    // per SM and row segment, fed by 32 KB bulk copies. Measured on a 4.3 GB single row: 7.2 TB/s against
    // 6.35 for the loads of row_split_kernel.
    if constexpr (V16 > 1) {
      const int64_t ring_rows = 16;
      if (vec_split && tuning().row_split_ring == 1 && n_rows <= ring_rows &&
          size_t(row_len) * sizeof(InT) >= (size_t(tuning().row_split_ring_min_mb) << 20) && n_seg > 1) {
        const int tile_vecs = int((size_t(32) << 10) / 16);
        const int stages    = 4;
        int64_t segs        = ceil_div<int64_t>(sm_count(), n_rows);
        if (segs > n_seg) segs = n_seg;  // the scratch was sized for n_seg partials per row
        int64_t sv = ceil_div<int64_t>(nvec, segs);
        sv         = ceil_div<int64_t>(sv, tile_vecs) * tile_vecs;
        segs       = ceil_div<int64_t>(nvec, sv);
        const size_t smem = size_t(stages) * size_t(tile_vecs) * 16;
        auto kern         = row_split_ring_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16, StoreT>;
        cudaError_t ea    = ensure_dynamic_smem(kern, smem);
        if (ea != cudaSuccess) return ea;
        const dim3 rgrid{unsigned(segs), unsigned(n_rows), 1u};
        (void)launch_dep(kern, dim3(rgrid), dim3(kTmaThreads), smem, stream, out, partial, data, n_rows, row_len, ld,
                         init, inplace, main_op, reduce_op, final_op, sv, tile_vecs, stages, ring_ctl(ws.status));
        ea = cudaGetLastError();
        if (ea != cudaSuccess || segs == 1) return ea;
        (void)launch_dep(row_finalize_kernel<OutT, ReduceOp, FinalOp, TPB, StoreT>,
                         dim3(unsigned(ceil_div<int64_t>(n_rows, TPB / 32))), dim3(TPB), 0, stream, out, partial,
                         n_rows, int(segs), init, inplace, reduce_op, final_op);
        return cudaGetLastError();
      }
    }
    const dim3 grid{unsigned(n_seg), unsigned(n_rows < 65535 ? n_rows : 65535), 1u};
    if (vec_split) {
      (void)launch_dep(row_split_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16, 4, TPB, StoreT>, dim3(grid),
                       dim3(TPB), 0, stream, out, partial, data, n_rows, row_len, ld, init, inplace, main_op,
                       reduce_op, final_op, seg_vecs);
    } else {
      (void)launch_dep(row_split_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, 1, 4, TPB, StoreT>, dim3(grid),
                       dim3(TPB), 0, stream, out, partial, data, n_rows, row_len, ld, init, inplace, main_op,
                       reduce_op, final_op, seg_vecs);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || n_seg == 1) return e;
    (void)launch_dep(row_finalize_kernel<OutT, ReduceOp, FinalOp, TPB, StoreT>,
                     dim3(unsigned(ceil_div<int64_t>(n_rows, TPB / 32))), dim3(TPB), 0, stream, out, partial, n_rows,
                     n_seg, init, inplace, reduce_op, final_op);
    return cudaGetLastError();
  }

  const int vec        = vec_ok ? V16 : 1;
  const int nvec       = int(row_len / vec);
  // lanes per row and chunks per lane: a lane sums up to four chunks of a row by itself (fewer
  // exchanges afterwards), as long as a group still reads at least 64 contiguous bytes per load
  int cpl              = tuning().row_cpl;
  // scalar path (rows that do not start on 16-byte boundaries): a load brings 4 bytes instead of 16, so
  // a lane takes four elements of a row whenever the row has them and keeps 32 loads in flight
  if (cpl == 0 && !vec_ok) cpl = nvec >= 4 ? 4 : (nvec >= 2 ? 2 : 1);
  // (rows of exactly four vectors: a lane takes the whole row - measured 12.3 against 14.3 us at 400 000 x 16 fp32)
  if (cpl == 0) cpl = nvec >= 32 ? 4 : (nvec >= 8 ? 2 : (nvec == 4 ? 4 : 1));
  if (cpl != 1 && cpl != 2 && cpl != 4) cpl = 1;
  unsigned g           = next_pow2(unsigned(nvec > 0 ? ceil_div<int>(nvec, cpl) : 1));
  const int G          = int(g > 32u ? 32u : g);
  const bool chunks    = nvec >= G * cpl * tuning().row_chunk_threshold;
  const int gpw        = 32 / G;
  // Ring variant (row_reduce_tma.cuh): short contiguous rows, plenty of them - one pass of G x cpl chunks per
  // row out of shared-memory tiles that a producer thread keeps filled. Chosen by itself for rows whose vector
  // count is exactly G x cpl (a power of two; other lengths leave lanes idle in the consumers, which are bound
  // by instruction issue: 24 / 48 / 96 / 192 columns measured 4.5-5.1 TB/s against 6.5 direct), between
  // `row_ring_min_vec` and `row_ring_max_vec` vectors, in matrices of at least `row_ring_min_mb` MiB. Measured,
  // fp32, TB/s ring / direct: 1 GiB of rows of 32 columns 6.5 / 6.1, 64: 6.55 / 6.3, 128: 6.6 / 6.3, 256: 6.6 / 6.4,
  // 512: 6.6 / 6.5; 2 GiB x 64 argmin 6.8 / 6.3; but 512 MB x 128: 6.05 / 6.3 and 128 MB: 4.7 / 4.9 - the ring
  // takes longer to fill and to drain. B2R_ROW_TMA=1 forces it wherever it fits, 2 turns it off.
  if constexpr (V16 > 1) {
    const size_t row_bytes = size_t(row_len) * sizeof(InT);
    const int ring_mode    = tuning().row_tma;
    const bool fits        = vec_ok && !chunks && ld == row_len && nvec <= G * cpl && sizeof(OutT) <= 8;
    const bool wanted      = ring_mode == 1 ? n_rows >= 4096
                                            : (ring_mode != 2 && nvec == G * cpl && nvec >= tuning().row_ring_min_vec &&
                                          nvec <= tuning().row_ring_max_vec &&
                                          size_t(n_rows) * row_bytes >= (size_t(tuning().row_ring_min_mb) << 20));
    if (fits && wanted) {
      const int64_t unit = int64_t(kTmaConsumers / 32) * (U / cpl) * gpw;  // rows of one pass of the 8 consumer warps
      int64_t k          = int64_t((size_t(tuning().row_tma_tile_kb) << 10) / (size_t(unit) * row_bytes));
      if (k < 1) k = 1;
      const int64_t tile_rows = unit * k;
      // a stage must always be used by the same team of consumers (a team that skips tiles could otherwise
      // wait for a phase of a barrier two phases ahead of it): a multiple of the team count
      int stages              = tuning().row_tma_stages / kRingTeams * kRingTeams;
      if (stages < kRingTeams) stages = kRingTeams;
      const size_t smem       = size_t(stages) * ((size_t(tile_rows) * row_bytes + 127) / 128 * 128);
      if (smem <= (size_t(220) << 10)) {
        int64_t ctas = sm_count();
        int64_t rpc  = ceil_div<int64_t>(n_rows, ctas);
        rpc          = ceil_div<int64_t>(rpc, tile_rows) * tile_rows;
        ctas         = ceil_div<int64_t>(n_rows, rpc);
#define B2R_LAUNCH_RING(U_, CPL_)                                                                              \
  do {                                                                                                         \
    auto kern      = row_reduce_ring_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16, U_, CPL_, kRingTeams, StoreT>; \
    cudaError_t ea = ensure_dynamic_smem(kern, smem);                                                          \
    if (ea != cudaSuccess) return ea;                                                                          \
    (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(kRingTeams * kTmaConsumers + 32), smem, stream,          \
      out, data, n_rows, int(row_len), init, inplace, main_op, reduce_op, final_op, G, int(tile_rows), rpc,    \
      stages, ring_ctl(ws.status));                                                                            \
  } while (0)
        if (cpl == 4) {
          B2R_LAUNCH_RING(U / 4, 4);
        } else if (cpl == 2) {
          B2R_LAUNCH_RING(U / 2, 2);
        } else {
          B2R_LAUNCH_RING(U, 1);
        }
#undef B2R_LAUNCH_RING
        return cudaGetLastError();
      }
    }
  }
  // Rows staged through shared memory (row_reduce_staged.cuh), contiguous matrices only:
  //  - rows that do not start on 16-byte boundaries: blocks of rows do, so whole blocks are copied
  //    (cp.async.bulk) and summed from shared memory, where alignment costs nothing;
  //  - aligned rows whose vector count fits the power-of-two lane groups of the direct kernels badly.
  if constexpr (V16 > 1 && sizeof(InT) >= 2) {
    const size_t row_bytes = size_t(row_len) * sizeof(InT);
    bool staged            = tuning().row_staged == 1 && ld == row_len && aligned16(data) &&
                  row_len <= tuning().row_staged_max &&
                  size_t(n_rows) * row_bytes >= staged_min_bytes(row_len, vec_ok);
    if (staged && vec_ok) {
      // slots of the direct kernel's lane groups that would stay empty
      const int64_t slots = int64_t(G) * cpl * ceil_div<int64_t>(nvec, int64_t(G) * cpl);
      const int mode      = tuning().row_staged_aligned;  // 1: when a tenth of the slots is wasted, 2: always, 3: never
      // (rows of up to 64 bytes: the staged kernel's lane per row beats the direct kernel's shuffles)
      staged              = mode == 2 || (mode == 1 && (int64_t(nvec) * 10 < slots * 9 || row_bytes <= 64) &&
                                 row_len <= tuning().row_staged_aligned_max);
    }
    if (staged) {
      const StagedPlan sp = plan_staged_rows(n_rows, row_bytes, nvec, vec_ok);
      if (sp.ok) {
        const int64_t n_main = sp.n_main;
        const int Gs = sp.G, rot = sp.rot, stages = sp.stages;
        const int64_t tile_rows = sp.tile_rows, rpc = sp.rows_per_cta, ctas = sp.ctas;
        const size_t smem = sp.smem;
#define B2R_LAUNCH_STAGED(VEC_)                                                                              \
  do {                                                                                                       \
    auto kern      = row_reduce_staged_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, VEC_, StoreT>;     \
    cudaError_t ea = ensure_dynamic_smem(kern, smem);                                                        \
    if (ea != cudaSuccess) return ea;                                                                        \
    (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(kTmaThreads), smem, stream, out, data, n_main,         \
                     int(row_len), init, inplace, main_op, reduce_op, final_op, Gs, rot, int(tile_rows),     \
                     rpc, stages, ring_ctl(ws.status));                                                      \
  } while (0)
        if (vec_ok) {
          B2R_LAUNCH_STAGED(V16);
        } else {
          B2R_LAUNCH_STAGED(1);
        }
#undef B2R_LAUNCH_STAGED
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess || n_main == n_rows) return e;
        // the up to m - 1 rows behind the last boundary: the direct kernels
        return launch_row_reduce<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, StoreT>(
          out + n_main, data + n_main * row_len, n_rows - n_main, row_len, ld, init, inplace, main_op, reduce_op,
          final_op, stream, ws);
      }
    }
  }
  // rows of 48 elements and more that do not start on 16-byte boundaries: the vector kernel in
  // chunk mode, one warp per row, takes the few leading / trailing elements of a row one by one
  // and everything in between with aligned 16-byte loads
  const bool shifted   = V16 > 1 && !vec_ok && row_len >= tuning().row_shifted_min && sizeof(InT) * V16 == 16 &&
                       (reinterpret_cast<uintptr_t>(data) % sizeof(InT)) == 0;
  // lanes per row in that mode: about sixteen vectors per lane (measured best: few lanes per row keep
  // the per-row reduction short), at least four lanes (they also take the up to three leading and
  // trailing elements)
  unsigned gs          = next_pow2(unsigned(ceil_div<int64_t>(row_len / (V16 > 1 ? V16 : 1), 16)));
  const int G_shifted  = int(gs > 32u ? 32u : (gs < 4u ? 4u : gs));
  const int u_scalar   = cpl == 4 ? 8 : 16;     // rows per group and pass on the scalar path
  const int u_rows     = (chunks || shifted) ? 1 : (vec_ok ? U / cpl : u_scalar);  // rows per group and pass
  const int64_t per_b  = int64_t(u_rows) * (shifted ? 32 / G_shifted : gpw);
  const int64_t n_b    = ceil_div<int64_t>(n_rows, per_b);
  const int rl         = int(row_len);
  const int cps_knob   = tuning().row_ctas_per_sm;
  const int sms        = sm_count();

  // Many short CTAs: by default a CTA gets one batch per warp (kRowCtasPerSm is only a bound), the hardware hands
  // CTAs to the SMs as they free up, and a fresh warp issues all its loads at once. Measured against two resident
  // waves of long-lived CTAs that loop over their batches (a warp has no load in flight while it reduces and stores
  // a batch): 1 000 000 x 128 fp32 6.63 -> 6.96 TB/s, 100 000 x 1024 6.52 -> 6.95, 250 000 x 1024 6.95 -> 7.28,
  // 4 000 000 x 32 6.32 -> 6.70, row argmin 8 388 608 x 64 (ring off) 6.41 -> 6.92. Rows of 8192 columns and more
  // (chunk mode: a warp streams a whole row) keep two resident waves: they do not care back to back and lose 2 %
  // on a cold single call (32768 x 32768).
  constexpr int kRowCtasPerSm = 256;
#define B2R_LAUNCH_ROW(VEC_, MODE_, U_, CPL_)                                                    \
  do {                                                                                           \
    auto kern      = row_reduce_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, VEC_, U_, MODE_, TPB, CPL_, StoreT>; \
    static int occ = resident_ctas(kern, TPB, 0);                                                \
    int64_t ctas   = int64_t(sms) * (cps_knob > 0 ? cps_knob : (MODE_ == kChunks ? 2 * occ : kRowCtasPerSm)); \
    const int64_t most = ceil_div<int64_t>(n_b, TPB / 32);                                       \
    if (ctas > most) ctas = most;                                                                \
    int64_t bpc = ceil_div<int64_t>(n_b, ctas);                                                  \
    /* A multiple of the CTA's 8 warps keeps the warps of a CTA even, but with 30-100 batches   */ \
    /* per CTA the rounding gives every CTA up to a tenth more than its share and leaves the    */ \
    /* last wave partly empty (measured 8-10 % at 1280 / 1536 / 2560 / 3072 / 6144 columns):    */ \
    /* round only when that costs less than 7 % (up to 6 % the even warps win: 1 000 000 x 128  */ \
    /* measured 3 % faster with 112 than with 106 batches per CTA; so do long rows with up to   */ \
    /* 32 batches per CTA: 32768 x 32768 measured 2 % faster with 32 than with 28).             */ \
    {                                                                                            \
      const int64_t r8 = ceil_div<int64_t>(bpc, TPB / 32) * (TPB / 32);                          \
      const int mode   = tuning().row_bpc_mode;                                                  \
      if (mode == 2 || (mode == 1 && ((r8 - bpc) * 14 < bpc || bpc <= 32))) {                                   \
        bpc = r8;                                                                                \
      } else if (mode == 3) {                                                                    \
        bpc |= 1;                                                                                \
      }                                                                                          \
    }                                                                                            \
    ctas        = ceil_div<int64_t>(n_b, bpc);                                                   \
    (void)launch_dep(kern, dim3(unsigned(ctas)), dim3(TPB), 0, stream,                           \
      out, data, n_rows, rl, ld, init, inplace, main_op, reduce_op, final_op,                    \
      shifted ? G_shifted : G,                                                                   \
      bpc, shifted);                                                                             \
  } while (0)
  if (shifted) {
    if constexpr (V16 > 1) { B2R_LAUNCH_ROW(V16, kChunks, U, 1); }
  } else if (vec_ok) {
    if (chunks) {
      B2R_LAUNCH_ROW(V16, kChunks, U, 1);
    } else if (cpl == 4) {
      B2R_LAUNCH_ROW(V16, kRows, U / 4, 4);
    } else if (cpl == 2) {
      B2R_LAUNCH_ROW(V16, kRows, U / 2, 2);
    } else {
      B2R_LAUNCH_ROW(V16, kRows, U, 1);
    }
  } else {
    if (chunks) {
      B2R_LAUNCH_ROW(1, kChunks, U, 1);
    } else if (cpl == 4) {
      B2R_LAUNCH_ROW(1, kRows, 8, 4);
    } else if (cpl == 2) {
      B2R_LAUNCH_ROW(1, kRows, 16, 2);
    } else {
      B2R_LAUNCH_ROW(1, kRows, 16, 1);
    }
  }
#undef B2R_LAUNCH_ROW
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Column-wise (strided axis) reduction of a row-major matrix.
// ---------------------------------------------------------------------------------------
struct ColPlan {
  bool tma;          // TMA-staged kernel (narrow, contiguous rows)
  bool tma2d;        // tiled-TMA kernel (wide matrices): grid_x column blocks x grid_y row ranges
  int tile_rows;     // rows per TMA tile
  int stages;        // stages of the TMA ring
  size_t off_status; // byte offset of the per-CTA status words inside the scratch
  int vec;
  int TX;
  int TY;
  unsigned grid_x;
  unsigned grid_y;
  int64_t rows_per_cta;
  size_t smem;
  size_t scratch;
  // the register-staged plan, kept beside a tiled-TMA plan in case the tensor map cannot be made
  unsigned reg_grid_x;
  unsigned reg_grid_y;
  int64_t reg_rows_per_cta;
  size_t reg_smem;
};

// `scratch_cap` (0: none) bounds the scratch the plan may ask for: a caller with a fixed scratch area gets
// fewer row ranges / CTAs (down to a single row range, which needs no scratch at all) instead of a refusal.
template <typename InT, typename OutT, typename State>
inline ColPlan plan_col_reduce(const InT* data, int64_t n_rows, int64_t n_cols, int64_t ld, size_t scratch_cap = 0)
{
  constexpr int TPB = 256;
  constexpr int U   = 8;
  constexpr int V16 = vec16<InT>::value;
  ColPlan p;
  const bool vec_ok = V16 > 1 && n_cols % V16 == 0 && ld % V16 == 0 && aligned16(data);
  p.vec             = vec_ok ? V16 : 1;
  const int64_t ncv = ceil_div<int64_t>(n_cols, p.vec);
  unsigned tx       = next_pow2(unsigned(ncv < 32 ? ncv : 32));
  p.TX              = int(tx);
  p.TY              = TPB / p.TX;
  p.grid_x          = unsigned(ceil_div<int64_t>(ncv, p.TX));
  // whole waves: column blocks x row ranges must not end just past a multiple of the resident CTAs (rounding the
  // row ranges up did: 8192 x 8192 fp32 got 640 CTAs for 592 slots, two waves for the work of one)
  const int64_t target = int64_t(sm_count()) * tuning().col_ctas_per_sm;
  int64_t gy           = tuning().col_gy_round == 2 ? ceil_div<int64_t>(target, p.grid_x) : target / p.grid_x;
  if (gy < 1) gy = 1;
  const int64_t max_gy = ceil_div<int64_t>(n_rows, int64_t(p.TY) * U);  // >= one full unrolled step each
  if (gy > max_gy) gy = max_gy;
  if (gy > 65535) gy = 65535;
  const size_t part_row = size_t(n_cols) * sizeof(typename State::carry_t);  // one partial row
  if (scratch_cap > 0 && gy > 1 && align_up(size_t(gy) * part_row, 256) > scratch_cap)
    gy = int64_t((scratch_cap - 255) / part_row);
  if (gy < 1) gy = 1;
  int64_t rpc     = ceil_div<int64_t>(n_rows, gy);
  rpc             = ceil_div<int64_t>(rpc, p.TY) * p.TY;
  gy              = ceil_div<int64_t>(n_rows, rpc);
  if (gy < 1) gy = 1;
  p.grid_y       = unsigned(gy);
  p.rows_per_cta = rpc;
  p.smem         = size_t(TPB) * p.vec * sizeof(State);
  p.scratch      = gy > 1 ? align_up(size_t(gy) * size_t(n_cols) * sizeof(typename State::carry_t), 256) : 0;
  p.tma          = false;
  p.tma2d        = false;
  p.stages       = 0;
  p.tile_rows    = 0;
  p.off_status   = 0;
  p.reg_grid_x   = p.grid_x;
  p.reg_grid_y   = p.grid_y;
  p.reg_rows_per_cta = rpc;
  p.reg_smem     = p.smem;
  // TMA-staged variant: rows contiguous, the whole width in one CTA, enough rows to stream
  const size_t row_bytes = size_t(n_cols) * sizeof(InT);
  if (tuning().col_tma == 1 && vec_ok && ld == n_cols && ncv <= kTmaConsumers && row_bytes % 16 == 0 &&
      n_rows >= 8192) {
    unsigned txp = next_pow2(unsigned(ncv));
    const int ty = kTmaConsumers / int(txp);
    size_t tile  = size_t(tuning().col_tma_tile_kb) << 10;
    int64_t tr   = int64_t(tile / row_bytes) / ty * ty;
    if (tr < ty) tr = ty;
    int64_t ctas = sm_count();
    // a partial row and a status word per CTA: fewer CTAs when the caller's scratch is bounded
    if (scratch_cap > 0 && align_up(size_t(ctas) * part_row, 256) + align_up(size_t(ctas) * sizeof(int), 256) > scratch_cap)
      ctas = scratch_cap > 1024 ? int64_t((scratch_cap - 1024) / (part_row + sizeof(int))) : 0;
    const size_t stage = (size_t(tr) * row_bytes + 127) / 128 * 128;
    const size_t smem  = size_t(tuning().tma_stages) * stage + size_t(kTmaConsumers) * p.vec * sizeof(State);
    // (a quarter of the SMs and fewer: the register-staged plan above, with its four CTAs per SM, is the better one)
    if (ctas * 4 >= sm_count() && smem <= (size_t(220) << 10)) {
      int64_t rpc2 = ceil_div<int64_t>(n_rows, ctas);
      rpc2         = ceil_div<int64_t>(rpc2, tr) * tr;
      ctas         = ceil_div<int64_t>(n_rows, rpc2);
      if (ctas > 1) {
        p.TX           = int(txp);
        p.TY           = kTmaConsumers / p.TX;
        p.tile_rows    = int(tr);
        p.grid_x       = unsigned(ctas);
        p.grid_y       = 1;
        p.rows_per_cta = rpc2;
        p.stages       = tuning().tma_stages;
        p.smem         = smem;
        const size_t parts = align_up(size_t(ctas) * part_row, 256);
        p.off_status   = parts;
        p.scratch      = parts + align_up(size_t(ctas) * sizeof(int), 256);
        p.tma          = true;
      }
    }
  }
  // tiled-TMA variant: wide matrices (more than one 32-vector column block), 16-byte aligned rows,
  // and enough data that filling the rings pays (measured: on par with the register-staged kernel
  // at 256 MB, 5-6 % faster for fp32 and 10-23 % for fp64 in the GB range)
  if constexpr (tensor_map_dtype<InT>::supported) {
    const int64_t BX = int64_t(32) * V16;
    if (!p.tma && tuning().col_tma == 1 && vec_ok && V16 > 1 && n_cols > BX && n_rows >= 4096 &&
        n_rows < (int64_t(1) << 31) && n_cols < (int64_t(1) << 31) && (size_t(ld) * sizeof(InT)) % 16 == 0 &&
        size_t(n_rows) * size_t(n_cols) * sizeof(InT) >= (size_t(tuning().col_tma2d_min_mb) << 20) &&
        row_bytes <= (size_t(tuning().col_tma2d_max_row_kb) << 10)) {
      const int64_t gx  = ceil_div<int64_t>(n_cols, BX);
      const int sms     = sm_count();
      int64_t best_gy = 0, best_cost = 0;
      const int64_t max_gy = n_rows / (4 * kBoxRows);  // at least four boxes per CTA
      // at most four CTAs per SM in all, like the register-staged kernel: the partial rows stay
      // within a few hundred KB whatever the shape
      for (int64_t gy = 2; gy <= max_gy && gx * gy <= int64_t(4) * sms; ++gy) {
        if (scratch_cap > 0 && align_up(size_t(gy) * part_row, 256) + align_up(size_t(gy) * sizeof(int), 256) > scratch_cap)
          break;  // a partial row and a status word per row range must fit the caller's scratch
        int64_t rpc         = ceil_div<int64_t>(ceil_div<int64_t>(n_rows, gy), kBoxRows) * kBoxRows;
        const int64_t gy_r  = ceil_div<int64_t>(n_rows, rpc);
        const int64_t waves = ceil_div<int64_t>(gx * gy_r, sms);
        const int64_t cost  = waves * (rpc + 2 * kBoxRows);  // per-CTA ramp-up of about two boxes
        if (best_gy == 0 || cost < best_cost) {
          best_gy   = gy_r;
          best_cost = cost;
        }
      }
      if (best_gy >= 2) {
        const int64_t rpc2   = ceil_div<int64_t>(ceil_div<int64_t>(n_rows, best_gy), kBoxRows) * kBoxRows;
        const unsigned gy2   = unsigned(ceil_div<int64_t>(n_rows, rpc2));
        const size_t smem2   = size_t(4) * size_t(kBoxRows) * size_t(BX) * sizeof(InT) +
                             size_t(kTmaConsumers / 32) * size_t(BX) * sizeof(State);
        if (gy2 >= 2 && smem2 <= (size_t(220) << 10)) {
          p.grid_x       = unsigned(gx);
          p.grid_y       = gy2;
          p.rows_per_cta = rpc2;
          p.stages       = 4;
          p.smem         = smem2;
          const size_t parts = align_up(size_t(gy2) * part_row, 256);
          p.off_status   = parts;
          // (the register-staged plan's partial rows fit too: it is the fallback of this one)
          const size_t need = parts + align_up(size_t(gy2) * sizeof(int), 256);
          p.scratch      = need > p.scratch ? need : p.scratch;
          p.tma2d        = true;
        }
      }
    }
  }
  return p;
}

template <typename InT, typename OutT, typename ReduceOp>
inline size_t col_reduce_scratch_bytes(const InT* data, int64_t n_rows, int64_t n_cols, int64_t ld, size_t scratch_cap = 0)
{
  using State = typename state_for<OutT, ReduceOp>::type;
  if (n_rows <= 0 || n_cols <= 0) return 0;
  return plan_col_reduce<InT, OutT, State>(data, n_rows, n_cols, ld, scratch_cap).scratch;
}

template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp>
cudaError_t launch_col_reduce(OutT* out,
                              const InT* data,
                              int64_t n_rows,
                              int64_t n_cols,
                              int64_t ld,
                              OutT init,
                              bool inplace,
                              MainOp main_op,
                              ReduceOp reduce_op,
                              FinalOp final_op,
                              cudaStream_t stream,
                              Workspace ws = Workspace{},
                              size_t scratch_cap = 0)
{
  constexpr int TPB = 256;
  constexpr int U   = 8;
  constexpr int V16 = vec16<InT>::value;
  using State       = typename state_for<OutT, ReduceOp>::type;
  if (n_cols <= 0) return cudaSuccess;
  if (n_rows < 0) n_rows = 0;

  ColPlan p = plan_col_reduce<InT, OutT, State>(data, n_rows > 0 ? n_rows : 1, n_cols, ld, scratch_cap);
  Scratch scratch(ws, p.scratch, stream);
  if (scratch.error() != cudaSuccess) return scratch.error();
  using CarryT    = typename State::carry_t;
  CarryT* partial = static_cast<CarryT*>(scratch.get());
  if (p.tma) {
    if constexpr (V16 > 1) {
      int* cta_status = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch.get()) + p.off_status);
      auto kern       = col_partial_tma_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16>;
      cudaError_t ea  = ensure_dynamic_smem(kern, size_t(p.smem));
      if (ea != cudaSuccess) return ea;
      (void)launch_dep(kern, dim3(p.grid_x), dim3(kTmaThreads), p.smem, stream, out, partial, data, n_rows,
                       int(n_cols), init, inplace, main_op, reduce_op, final_op, p.TX, p.tile_rows, p.rows_per_cta,
                       p.stages, cta_status, ring_ctl(ws.status));
      ea = cudaGetLastError();
      if (ea != cudaSuccess) return ea;
      const unsigned fin = unsigned(ceil_div<int64_t>(n_cols, TPB / 32));
      (void)launch_dep(col_finalize_kernel<OutT, ReduceOp, FinalOp, TPB>, dim3(fin), dim3(TPB), 0, stream, out,
                       partial, int(p.grid_x), n_cols, init, inplace, reduce_op, final_op, cta_status);
      return cudaGetLastError();
    }
  }
  if (p.tma2d) {
    if constexpr (V16 > 1 && tensor_map_dtype<InT>::supported) {
      CUtensorMap tmap;
      cudaError_t ea = make_tensor_map_2d<InT>(&tmap, data, n_rows, n_cols, ld, kBoxRows, 32 * V16);
      if (ea == cudaSuccess) {
        int* cta_status = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch.get()) + p.off_status);
        ea              = cudaMemsetAsync(cta_status, 0, size_t(p.grid_y) * sizeof(int), stream);
        if (ea != cudaSuccess) return ea;
        auto kern = col_partial_tma2d_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16>;
        ea        = ensure_dynamic_smem(kern, size_t(p.smem));
        if (ea != cudaSuccess) return ea;
        const dim3 grid2(p.grid_x, p.grid_y);
        (void)launch_dep(kern, dim3(grid2), dim3(kTmaThreads), p.smem, stream, out, partial, tmap, n_rows, n_cols,
                         init, inplace, main_op, reduce_op, final_op, p.rows_per_cta, p.stages, cta_status,
                         ring_ctl(ws.status));
        ea = cudaGetLastError();
        if (ea != cudaSuccess) return ea;
        const unsigned fin = unsigned(ceil_div<int64_t>(n_cols, TPB / 32));
        (void)launch_dep(col_finalize_kernel<OutT, ReduceOp, FinalOp, TPB>, dim3(fin), dim3(TPB), 0, stream, out,
                         partial, int(p.grid_y), n_cols, init, inplace, reduce_op, final_op, cta_status);
        return cudaGetLastError();
      }
      // no tensor map (driver entry point missing): the register-staged plan, whose partial rows
      // [row ranges][n_cols] fit the same scratch
      p.grid_x       = p.reg_grid_x;
      p.grid_y       = p.reg_grid_y;
      p.rows_per_cta = p.reg_rows_per_cta;
      p.smem         = p.reg_smem;
    }
  }
  const dim3 grid(p.grid_x, p.grid_y);

  if (p.vec > 1) {
    (void)launch_dep(col_partial_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16, U, TPB>, dim3(grid),
                     dim3(TPB), p.smem, stream, out, partial, data, n_rows, n_cols, ld, init, inplace, main_op,
                     reduce_op, final_op, p.TX, p.rows_per_cta);
  } else {
    (void)launch_dep(col_partial_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, 1, U, TPB>, dim3(grid), dim3(TPB),
                     p.smem, stream, out, partial, data, n_rows, n_cols, ld, init, inplace, main_op, reduce_op,
                     final_op, p.TX, p.rows_per_cta);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || p.grid_y == 1) return e;
  const unsigned fin_ctas = unsigned(ceil_div<int64_t>(n_cols, TPB / 32));
  (void)launch_dep(col_finalize_kernel<OutT, ReduceOp, FinalOp, TPB>, dim3(fin_ctas), dim3(TPB), 0, stream, out,
                   partial, int(p.grid_y), n_cols, init, inplace, reduce_op, final_op, static_cast<const int*>(nullptr));
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
