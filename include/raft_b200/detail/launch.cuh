// Host-side shape policies and launchers for the reduction kernels. Header-only templates:
// the shared library instantiates them for the operator set of the C ABI, the drop-in
// raft::linalg headers instantiate them for caller-supplied functors.
//
// All launchers are asynchronous on the given stream and return a cudaError_t; none of
// them synchronises. Kernels that need scratch memory (row partials, column partials) take
// it from the caller's workspace when one is passed and large enough, otherwise from the
// stream-ordered allocator (cudaMallocAsync / cudaFreeAsync on the same stream), which is
// what the reference does for its only scratch user (coalesced_reduction-inl.cuh:560).
#pragma once

#include "col_reduce.cuh"
#include "row_reduce.cuh"

#include <cstdlib>

namespace raft_b200 {
namespace detail {

struct Workspace {
  void* ptr    = nullptr;
  size_t bytes = 0;
};

// Stream-ordered scratch with a caller-provided fast path.
class Scratch {
 public:
  Scratch(const Workspace& ws, size_t need, cudaStream_t stream) : stream_(stream)
  {
    if (need == 0) return;
    if (ws.ptr != nullptr && ws.bytes >= need) {
      ptr_ = ws.ptr;
    } else {
      err_   = cudaMallocAsync(&ptr_, need, stream);
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
  static int cached[64] = {};
  int dev               = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Launch-shape knobs. The defaults are the measured best on B200; the environment
// variables exist so that a benchmark can sweep them without rebuilding.
struct Tuning {
  int row_ctas_per_sm      = 0;   // B2R_ROW_CPS   row-kernel CTAs per SM (0: as many as are resident)
  int row_chunk_threshold  = 4;   // B2R_ROW_CHUNK rows with >= this many vectors per lane use kChunks
  int col_ctas_per_sm      = 4;   // B2R_COL_CPS   column-partial CTAs per SM (one resident wave)
  int split_ctas_per_sm    = 4;   // B2R_SPLIT_CPS
  int key_block_rows       = 8192;  // B2R_KEY_BLOCK  rows per sorted block (rows-by-key, table algorithm)
  int key_window_rows      = 0;     // B2R_KEY_WINDOW rows per sort window (rows-by-key, sorted algorithm; 0: auto)
  int key_algo             = 0;     // B2R_KEY_ALGO   0: auto, 1: shared-memory table, 2: sort then stream
};

inline int env_int(const char* name, int dflt)
{
  const char* s = std::getenv(name);
  if (s == nullptr || *s == 0) return dflt;
  const int v = std::atoi(s);
  return v > 0 ? v : dflt;
}

inline Tuning tuning()
{
  // read on every call (five getenv look-ups) so that a benchmark can sweep within one process
  Tuning x;
  x.row_ctas_per_sm      = env_int("B2R_ROW_CPS", x.row_ctas_per_sm);
  x.row_chunk_threshold  = env_int("B2R_ROW_CHUNK", x.row_chunk_threshold);
  x.col_ctas_per_sm      = env_int("B2R_COL_CPS", x.col_ctas_per_sm);
  x.split_ctas_per_sm    = env_int("B2R_SPLIT_CPS", x.split_ctas_per_sm);
  x.key_block_rows       = env_int("B2R_KEY_BLOCK", x.key_block_rows);
  x.key_window_rows      = env_int("B2R_KEY_WINDOW", x.key_window_rows);
  x.key_algo             = env_int("B2R_KEY_ALGO", x.key_algo);
  return x;
}

// Resident CTAs per SM of a kernel: the reductions launch exactly one resident wave and loop
// inside the kernel (measured on B200: one wave of long-lived CTAs reads ~15 % faster than
// many short ones).
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
  // Split rows only when there are too few rows to occupy the machine with one warp per
  // row and the rows are long enough that a segment still amortises a CTA.
  const int sms           = sm_count();
  const int64_t row_bytes = row_len * int64_t(in_size);
  int n_seg               = 1;
  if (n_rows < int64_t(sms) * 8 && row_bytes >= (int64_t(64) << 10)) {
    const int64_t want    = ceil_div<int64_t>(int64_t(sms) * tuning().split_ctas_per_sm, n_rows);
    const int64_t max_seg = ceil_div<int64_t>(row_bytes, int64_t(32) << 10);
    n_seg                 = int(want < max_seg ? want : max_seg);
    if (n_seg < 1) n_seg = 1;
  }
  if (n_seg_out) *n_seg_out = n_seg;
  return n_seg > 1 ? align_up(size_t(n_rows) * n_seg * sizeof(CarryT), 256) : 0;
}

template <typename InT,
          typename OutT,
          typename IdxT,
          typename MainOp,
          typename ReduceOp,
          typename FinalOp>
cudaError_t launch_row_reduce(OutT* out,
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

  if (n_seg > 1 || row_len > int64_t(0x7fffffff)) {
    // long rows: CTA per (segment, row), then fold the segment partials
    Scratch scratch(ws, need, stream);
    if (scratch.error() != cudaSuccess) return scratch.error();
    CarryT* partial       = static_cast<CarryT*>(scratch.get());
    const int vec         = vec_ok ? V16 : 1;
    const int64_t nvec    = row_len / vec;
    int64_t seg_vecs      = ceil_div<int64_t>(nvec, n_seg);
    seg_vecs              = ceil_div<int64_t>(seg_vecs, TPB) * TPB;
    n_seg                 = int(ceil_div<int64_t>(nvec, seg_vecs));
    if (n_seg < 1) n_seg = 1;
    const dim3 grid{unsigned(n_seg), unsigned(n_rows < 65535 ? n_rows : 65535), 1u};
    if (vec_ok) {
      row_split_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16, 4, TPB>
        <<<grid, TPB, 0, stream>>>(
          out, partial, data, n_rows, row_len, ld, init, inplace, main_op, reduce_op, final_op, seg_vecs);
    } else {
      row_split_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, 1, 4, TPB>
        <<<grid, TPB, 0, stream>>>(
          out, partial, data, n_rows, row_len, ld, init, inplace, main_op, reduce_op, final_op, seg_vecs);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || n_seg == 1) return e;
    row_finalize_kernel<OutT, ReduceOp, FinalOp, TPB>
      <<<unsigned(ceil_div<int64_t>(n_rows, TPB / 32)), TPB, 0, stream>>>(
        out, partial, n_rows, n_seg, init, inplace, reduce_op, final_op);
    return cudaGetLastError();
  }

  const int vec        = vec_ok ? V16 : 1;
  const int nvec       = int(row_len / vec);
  unsigned g           = next_pow2(unsigned(nvec > 0 ? nvec : 1));
  const int G          = int(g > 32u ? 32u : g);
  const bool chunks    = nvec >= G * tuning().row_chunk_threshold;
  const int gpw        = 32 / G;
  const int64_t per_b  = chunks ? gpw : int64_t(U) * gpw;
  const int64_t n_b    = ceil_div<int64_t>(n_rows, per_b);
  const int rl         = int(row_len);
  const int cps_knob   = tuning().row_ctas_per_sm;
  const int sms        = sm_count();

#define B2R_LAUNCH_ROW(VEC_, MODE_)                                                              \
  do {                                                                                           \
    auto kern      = row_reduce_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, VEC_, U, MODE_, TPB>; \
    static int occ = resident_ctas(kern, TPB, 0);                                                \
    int64_t ctas   = int64_t(sms) * (cps_knob > 0 ? cps_knob : occ);                             \
    const int64_t most = ceil_div<int64_t>(n_b, TPB / 32);                                       \
    if (ctas > most) ctas = most;                                                                \
    int64_t bpc = ceil_div<int64_t>(n_b, ctas);                                                  \
    bpc         = ceil_div<int64_t>(bpc, TPB / 32) * (TPB / 32);                                 \
    ctas        = ceil_div<int64_t>(n_b, bpc);                                                   \
    kern<<<unsigned(ctas), TPB, 0, stream>>>(                                                    \
      out, data, n_rows, rl, ld, init, inplace, main_op, reduce_op, final_op, G, bpc);           \
  } while (0)
  if (vec_ok) {
    if (chunks) {
      B2R_LAUNCH_ROW(V16, kChunks);
    } else {
      B2R_LAUNCH_ROW(V16, kRows);
    }
  } else {
    if (chunks) {
      B2R_LAUNCH_ROW(1, kChunks);
    } else {
      B2R_LAUNCH_ROW(1, kRows);
    }
  }
#undef B2R_LAUNCH_ROW
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Column-wise (strided axis) reduction of a row-major matrix.
// ---------------------------------------------------------------------------------------
struct ColPlan {
  int vec;
  int TX;
  int TY;
  unsigned grid_x;
  unsigned grid_y;
  int64_t rows_per_cta;
  size_t smem;
  size_t scratch;
};

template <typename InT, typename OutT, typename State>
inline ColPlan plan_col_reduce(const InT* data, int64_t n_rows, int64_t n_cols, int64_t ld)
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
  const int64_t target = int64_t(sm_count()) * tuning().col_ctas_per_sm;
  int64_t gy           = ceil_div<int64_t>(target, p.grid_x);
  const int64_t max_gy = ceil_div<int64_t>(n_rows, int64_t(p.TY) * U);  // >= one full unrolled step each
  if (gy > max_gy) gy = max_gy;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  int64_t rpc     = ceil_div<int64_t>(n_rows, gy);
  rpc             = ceil_div<int64_t>(rpc, p.TY) * p.TY;
  gy              = ceil_div<int64_t>(n_rows, rpc);
  if (gy < 1) gy = 1;
  p.grid_y       = unsigned(gy);
  p.rows_per_cta = rpc;
  p.smem         = size_t(TPB) * p.vec * sizeof(State);
  p.scratch      = gy > 1 ? align_up(size_t(gy) * size_t(n_cols) * sizeof(typename State::carry_t), 256) : 0;
  return p;
}

template <typename InT, typename OutT, typename ReduceOp>
inline size_t col_reduce_scratch_bytes(const InT* data, int64_t n_rows, int64_t n_cols, int64_t ld)
{
  using State = typename state_for<OutT, ReduceOp>::type;
  if (n_rows <= 0 || n_cols <= 0) return 0;
  return plan_col_reduce<InT, OutT, State>(data, n_rows, n_cols, ld).scratch;
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
                              Workspace ws = Workspace{})
{
  constexpr int TPB = 256;
  constexpr int U   = 8;
  constexpr int V16 = vec16<InT>::value;
  using State       = typename state_for<OutT, ReduceOp>::type;
  if (n_cols <= 0) return cudaSuccess;
  if (n_rows < 0) n_rows = 0;

  const ColPlan p = plan_col_reduce<InT, OutT, State>(data, n_rows > 0 ? n_rows : 1, n_cols, ld);
  Scratch scratch(ws, p.scratch, stream);
  if (scratch.error() != cudaSuccess) return scratch.error();
  using CarryT    = typename State::carry_t;
  CarryT* partial = static_cast<CarryT*>(scratch.get());
  const dim3 grid(p.grid_x, p.grid_y);

  if (p.vec > 1) {
    col_partial_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, V16, U, TPB>
      <<<grid, TPB, p.smem, stream>>>(out, partial, data, n_rows, n_cols, ld, init, inplace,
                                      main_op, reduce_op, final_op, p.TX, p.rows_per_cta);
  } else {
    col_partial_kernel<InT, OutT, IdxT, MainOp, ReduceOp, FinalOp, 1, U, TPB>
      <<<grid, TPB, p.smem, stream>>>(out, partial, data, n_rows, n_cols, ld, init, inplace,
                                      main_op, reduce_op, final_op, p.TX, p.rows_per_cta);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || p.grid_y == 1) return e;
  const unsigned fin_ctas = unsigned(ceil_div<int64_t>(n_cols, TPB));
  col_finalize_kernel<OutT, ReduceOp, FinalOp, TPB><<<fin_ctas, TPB, 0, stream>>>(
    out, partial, int(p.grid_y), n_cols, init, inplace, reduce_op, final_op);
  return cudaGetLastError();
}

}  // namespace detail
}  // namespace raft_b200
