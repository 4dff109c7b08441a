// C ABI of the peer-memory all-reduce (include/raft_b200/detail/peer_allreduce.cuh): the exchange
// area, its hand-over between the processes of a node (CUDA IPC) or the devices of one process
// (direct pointers), and the one-kernel all-reduce of per-GPU partial sums and counts.
#include "capi_internal.cuh"

#include <raft_b200/detail/peer_allreduce.cuh>

#include <cstring>
#include <new>

namespace raft_b200 {
namespace capi {

struct PeerArea {
  int world;
  int rank;
  int device;
  size_t slot_bytes;
  size_t set_stride;
  size_t flags_off;
  size_t status_off;
  size_t ll_off;
  size_t bytes;
  unsigned char* local;
  unsigned char* base[detail::kPeerMaxWorld];
  bool ipc_opened[detail::kPeerMaxWorld];
  unsigned long long calls;
  unsigned long long limit_ns;
};

}  // namespace capi
}  // namespace raft_b200

using namespace raft_b200;
using namespace raft_b200::capi;

extern "C" int b2r_peer_area_create(int32_t world, int32_t rank, size_t max_payload_bytes, void** area_out)
{
  if (area_out == nullptr || world < 1 || world > detail::kPeerMaxWorld || rank < 0 || rank >= world)
    return B2R_ERR_BAD_ARG;
  *area_out = nullptr;
  PeerArea* a = new (std::nothrow) PeerArea();
  if (a == nullptr) return B2R_ERR_BAD_ARG;
  std::memset(a, 0, sizeof(*a));
  a->world      = world;
  a->rank       = rank;
  a->slot_bytes = detail::align_up(max_payload_bytes > 0 ? max_payload_bytes : 16, 256);
  a->set_stride = a->slot_bytes * size_t(world);
  a->flags_off  = 2 * a->set_stride;
  a->status_off = a->flags_off + detail::align_up(size_t(2) * size_t(world) * detail::kPeerMaxCtas * sizeof(unsigned), 256);
  a->ll_off     = a->status_off + 256;
  a->bytes      = a->ll_off + size_t(2) * size_t(world) * 2 * detail::kPeerLLBytes;
  a->limit_ns   = 2000ull * 1000ull * 1000ull;
  cudaError_t e = cudaGetDevice(&a->device);
  // plain cudaMalloc: memory of a stream-ordered pool cannot be exported through cudaIpcGetMemHandle
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&a->local), a->bytes);
  if (e == cudaSuccess) e = cudaMemset(a->local, 0, a->bytes);
  if (e != cudaSuccess) {
    if (a->local != nullptr) cudaFree(a->local);
    delete a;
    return set_cuda_error(e);
  }
  a->base[rank] = a->local;
  *area_out     = a;
  return B2R_OK;
}

extern "C" int b2r_peer_area_ipc_handle(void* area, void* handle_out_64_bytes)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  if (a == nullptr || handle_out_64_bytes == nullptr) return B2R_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, a->local);
  if (e != cudaSuccess) return set_cuda_error(e);
  std::memcpy(handle_out_64_bytes, &h, 64);
  return B2R_OK;
}

extern "C" int b2r_peer_area_open(void* area, int32_t peer_rank, const void* handle_64_bytes)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  if (a == nullptr || handle_64_bytes == nullptr || peer_rank < 0 || peer_rank >= a->world || peer_rank == a->rank)
    return B2R_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle_64_bytes, 64);
  void* p       = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return set_cuda_error(e);
  a->base[peer_rank]       = static_cast<unsigned char*>(p);
  a->ipc_opened[peer_rank] = true;
  return B2R_OK;
}

extern "C" int b2r_peer_area_link(void* area, int32_t peer_rank, void* peer_area_same_process)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  PeerArea* b = static_cast<PeerArea*>(peer_area_same_process);
  if (a == nullptr || b == nullptr || peer_rank < 0 || peer_rank >= a->world || peer_rank == a->rank ||
      b->rank != peer_rank || b->world != a->world || b->slot_bytes != a->slot_bytes)
    return B2R_ERR_BAD_ARG;
  if (b->device != a->device) {
    int can = 0;
    cudaError_t e = cudaDeviceCanAccessPeer(&can, a->device, b->device);
    if (e != cudaSuccess) return set_cuda_error(e);
    if (!can) return B2R_ERR_UNSUPPORTED;
    e = cudaDeviceEnablePeerAccess(b->device, 0);  // for the current device, which must be the area's
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      (void)cudaGetLastError();
    } else if (e != cudaSuccess) {
      return set_cuda_error(e);
    }
  }
  a->base[peer_rank] = b->local;
  return B2R_OK;
}

extern "C" int b2r_peer_area_set_wait_limit_ms(void* area, uint32_t ms)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  if (a == nullptr || ms == 0) return B2R_ERR_BAD_ARG;
  a->limit_ns = (unsigned long long)ms * 1000ull * 1000ull;
  return B2R_OK;
}

extern "C" int b2r_peer_allreduce_sum(void* area, float* sums, int64_t n_f32, long long* counts, int64_t n_i64,
                                      double scale, b2r_stream_t stream)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  if (a == nullptr || n_f32 < 0 || n_i64 < 0 || (n_f32 > 0 && sums == nullptr) || (n_i64 > 0 && counts == nullptr))
    return B2R_ERR_BAD_ARG;
  const int64_t nv_f32 = (n_f32 + 3) / 4, nv_i64 = (n_i64 + 1) / 2, nvec = nv_f32 + nv_i64;
  if (nvec == 0) return B2R_OK;
  if (size_t(nvec) * 16 > a->slot_bytes) return B2R_ERR_TOO_LARGE;
  for (int p = 0; p < a->world; ++p)
    if (a->base[p] == nullptr) return B2R_ERR_BAD_ARG;  // a peer was never opened / linked
  detail::PeerParams P;
  for (int p = 0; p < detail::kPeerMaxWorld; ++p)
    P.base[p] = p < a->world ? a->base[p] : nullptr;
  P.world      = a->world;
  P.rank       = a->rank;
  P.seq        = unsigned(a->calls % 0xFFFFFFFEull) + 1u;
  P.set        = unsigned(a->calls & 1ull);
  a->calls += 1;
  P.slot_bytes = a->slot_bytes;
  P.set_stride = a->set_stride;
  P.flags_off  = a->flags_off;
  P.ll_off     = a->ll_off;
  P.limit_ns   = a->limit_ns;
  P.status     = reinterpret_cast<int*>(a->local + a->status_off);
  if (size_t(n_f32) * 4 + size_t(n_i64) * 8 <= size_t(detail::kPeerLLBytes)) {
    // small payload: tagged words, no flag (the same choice on every rank - it depends on the sizes only)
    detail::peer_allreduce_ll_kernel<<<1, detail::kPeerThreads, 0, to_stream(stream)>>>(P, sums, n_f32, counts, n_i64,
                                                                                       float(scale));
    return set_cuda_error(cudaGetLastError());
  }
  // the same split of the payload on every rank: chunks of at least two vectors per thread, at most 64 CTAs
  int64_t ctas = detail::ceil_div<int64_t>(nvec, 2 * detail::kPeerThreads);
  if (ctas > detail::kPeerMaxCtas) ctas = detail::kPeerMaxCtas;
  if (ctas < 1) ctas = 1;
  const int64_t vpc = detail::ceil_div<int64_t>(nvec, ctas);
  ctas              = detail::ceil_div<int64_t>(nvec, vpc);
  detail::peer_allreduce_kernel<<<unsigned(ctas), detail::kPeerThreads, 0, to_stream(stream)>>>(
    P, sums, n_f32, counts, n_i64, float(scale), nvec, vpc);
  return set_cuda_error(cudaGetLastError());
}

extern "C" int b2r_peer_area_status(void* area, int32_t* status_out, int32_t clear)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  if (a == nullptr || status_out == nullptr) return B2R_ERR_BAD_ARG;
  int v         = 0;
  cudaError_t e = cudaMemcpy(&v, a->local + a->status_off, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && clear != 0 && v != 0) e = cudaMemset(a->local + a->status_off, 0, sizeof(int));
  if (e != cudaSuccess) return set_cuda_error(e);
  *status_out = v != 0 ? B2R_ERR_TIMEOUT : B2R_OK;
  return B2R_OK;
}

extern "C" int b2r_peer_area_destroy(void* area)
{
  PeerArea* a = static_cast<PeerArea*>(area);
  if (a == nullptr) return B2R_OK;
  cudaError_t first = cudaSuccess;
  for (int p = 0; p < a->world; ++p) {
    if (a->ipc_opened[p]) {
      cudaError_t e = cudaIpcCloseMemHandle(a->base[p]);
      if (first == cudaSuccess) first = e;
    }
  }
  cudaError_t e = cudaFree(a->local);
  if (first == cudaSuccess) first = e;
  delete a;
  return set_cuda_error(first);
}
