// b2r_column_sum_f32_noalloc: column sums with a fixed, library-owned scratch area.
//
// The regular column reduction (b2r_reduce along the strided axis) needs a few hundred KB of
// scratch for its per-CTA partial rows and gets them from the caller's workspace or from
// cudaMallocAsync. Some callers can do neither: a serving loop that has promised its host
// process no allocator traffic after start-up (cudaMalloc and cudaFree take driver locks and
// can stall every stream of the device), a plugin that is handed two pointers and a stream and
// nothing else, or a process whose memory pools are disabled. For them this entry point runs
// the SAME kernels as the column path of b2r_reduce on a scratch array that is
// part of the library image: kNoAllocScratchBytes of device memory on every GPU that loads the
// library, held until the process exits.
//
// The array's name is only a host-side handle here; the device address the kernels need comes
// from cudaGetSymbolAddress, looked up once per device (with that device current) and cached.
#include "capi_internal.cuh"

#include <mutex>

namespace raft_b200 {
namespace capi {

constexpr size_t kNoAllocScratchBytes = size_t(1) << 20;  // 1 MiB
constexpr int kMaxDevices             = 64;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

static std::mutex g_noalloc_mutex;
static void* g_noalloc_ptr[kMaxDevices] = {};

// Device address of g_noalloc_scratch on the CURRENT device; resolved on first use per device.
static cudaError_t noalloc_scratch(void** out)
{
  int dev       = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e       = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return cudaSuccess;
}

}  // namespace capi
}  // namespace raft_b200

using namespace raft_b200;
using namespace raft_b200::capi;

extern "C" int b2r_column_sum_f32_noalloc(float* out, const float* in, int64_t n_rows, int64_t n_cols,
                                          int32_t final_op, double final_scalar, b2r_stream_t stream)
{
  if (n_rows < 0 || n_cols < 0) return B2R_ERR_BAD_ARG;
  if (n_cols > 0 && out == nullptr) return B2R_ERR_BAD_ARG;
  if (n_rows > 0 && n_cols > 0 && in == nullptr) return B2R_ERR_BAD_ARG;
  if (final_op < B2R_FINAL_IDENTITY || final_op > B2R_FINAL_ABS) return B2R_ERR_BAD_ARG;
  if (n_cols == 0) return B2R_OK;
  // The launch shape is planned under the array's size: shapes whose preferred plan would need more
  // (a partial row per CTA of 148 x n_cols x 8 bytes for n_cols near 1024, two row ranges of more than
  // 65536 columns) get fewer CTAs or a single row range, which needs no scratch at all. The check
  // stays as the guard of the array: refuse, never allocate.
  const size_t need = detail::col_reduce_scratch_bytes<float, float, op::Add>(in, n_rows, n_cols, n_cols,
                                                                              kNoAllocScratchBytes);
  if (need > kNoAllocScratchBytes) return B2R_ERR_TOO_LARGE;
  void* scratch = nullptr;
  cudaError_t e = noalloc_scratch(&scratch);
  if (e != cudaSuccess) return set_cuda_error(e);
  detail::Workspace ws;
  ws.ptr    = scratch;
  ws.bytes  = kNoAllocScratchBytes;
  ws.status = kernel_status_word();  // an address lookup on the first call per device, no allocation
  op::RuntimeFinal<float> fin{final_op, float(final_scalar)};
  e = detail::launch_col_reduce<float, float, int64_t>(out, in, n_rows, n_cols, n_cols, 0.0f, false, op::Identity{},
                                                       op::Add{}, fin, to_stream(stream), ws, kNoAllocScratchBytes);
  return set_cuda_error(e);
}

extern "C" size_t b2r_column_sum_f32_noalloc_max_scratch(void) { return kNoAllocScratchBytes; }
