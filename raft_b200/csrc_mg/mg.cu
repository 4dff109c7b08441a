// libraft_b200_mg.so: row-sharded reductions over several devices of one node from one host
// process. Per-device work goes through the C ABI of libraft_b200.so; partial results of column
// and by-key reductions are combined with ncclAllReduce inside one NCCL group.
#include <raft_b200_mg.h>

#include <cuda_runtime.h>
#include <nccl.h>

#include <cstring>
#include <new>
#include <vector>

struct b2r_mg_comm {
  std::vector<int> devices;
  std::vector<ncclComm_t> comms;
  std::vector<cudaStream_t> streams;
  bool owns_comms = false;
};

namespace {

// restores the caller's current device on scope exit
struct DeviceGuard {
  int prev = 0;
  DeviceGuard() { cudaGetDevice(&prev); }
  ~DeviceGuard() { cudaSetDevice(prev); }
};

bool nccl_type(int32_t dtype, ncclDataType_t* t)
{
  switch (dtype) {
    case B2R_F32: *t = ncclFloat32; return true;
    case B2R_F64: *t = ncclFloat64; return true;
    case B2R_F16: *t = ncclFloat16; return true;
    case B2R_I32: *t = ncclInt32; return true;
    case B2R_I64: *t = ncclInt64; return true;
    case B2R_U32: *t = ncclUint32; return true;
    default: return false;
  }
}

bool nccl_op(int32_t reduce_op, ncclRedOp_t* op)
{
  switch (reduce_op) {
    case B2R_REDUCE_ADD: *op = ncclSum; return true;
    case B2R_REDUCE_MIN: *op = ncclMin; return true;
    case B2R_REDUCE_MAX: *op = ncclMax; return true;
    default: return false;
  }
}

cudaStream_t stream_of(const b2r_mg_comm* c, const b2r_stream_t* streams, int d)
{
  return streams != nullptr ? reinterpret_cast<cudaStream_t>(streams[d]) : c->streams[d];
}

int create_common(b2r_mg_comm** out, const int* devices, int n, void* const* adopt)
{
  if (out == nullptr || devices == nullptr || n <= 0) return B2R_ERR_BAD_ARG;
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess) return B2R_ERR_CUDA;
  for (int i = 0; i < n; ++i) {
    if (devices[i] < 0 || devices[i] >= visible) return B2R_ERR_BAD_ARG;
    for (int j = 0; j < i; ++j)
      if (devices[j] == devices[i]) return B2R_ERR_BAD_ARG;
  }
  b2r_mg_comm* c = new (std::nothrow) b2r_mg_comm;
  if (c == nullptr) return B2R_ERR_CUDA;
  c->devices.assign(devices, devices + n);
  c->comms.resize(n);
  c->streams.assign(n, nullptr);
  DeviceGuard guard;
  if (adopt != nullptr) {
    for (int i = 0; i < n; ++i)
      c->comms[i] = static_cast<ncclComm_t>(adopt[i]);
  } else {
    if (ncclCommInitAll(c->comms.data(), n, devices) != ncclSuccess) {
      delete c;
      return B2R_ERR_CUDA;
    }
    c->owns_comms = true;
  }
  for (int i = 0; i < n; ++i) {
    if (cudaSetDevice(devices[i]) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->streams[i], cudaStreamNonBlocking) != cudaSuccess) {
      b2r_mg_comm_destroy(c);
      return B2R_ERR_CUDA;
    }
  }
  *out = c;
  return B2R_OK;
}

}  // namespace

extern "C" int b2r_mg_comm_create(b2r_mg_comm** comm, const int* devices, int n_devices)
{
  return create_common(comm, devices, n_devices, nullptr);
}

extern "C" int b2r_mg_comm_adopt(b2r_mg_comm** comm, const int* devices, int n_devices, void* const* nccl_comms)
{
  if (nccl_comms == nullptr) return B2R_ERR_BAD_ARG;
  return create_common(comm, devices, n_devices, nccl_comms);
}

extern "C" int b2r_mg_comm_destroy(b2r_mg_comm* c)
{
  if (c == nullptr) return B2R_OK;
  DeviceGuard guard;
  for (size_t i = 0; i < c->devices.size(); ++i) {
    cudaSetDevice(c->devices[i]);
    if (c->streams[i] != nullptr) {
      cudaStreamSynchronize(c->streams[i]);
      cudaStreamDestroy(c->streams[i]);
    }
    if (c->owns_comms && c->comms[i] != nullptr) ncclCommDestroy(c->comms[i]);
  }
  delete c;
  return B2R_OK;
}

extern "C" int b2r_mg_comm_size(const b2r_mg_comm* c) { return c != nullptr ? int(c->devices.size()) : 0; }

extern "C" int b2r_mg_sync(b2r_mg_comm* c)
{
  if (c == nullptr) return B2R_ERR_BAD_ARG;
  DeviceGuard guard;
  for (size_t i = 0; i < c->devices.size(); ++i) {
    if (cudaSetDevice(c->devices[i]) != cudaSuccess) return B2R_ERR_CUDA;
    if (cudaStreamSynchronize(c->streams[i]) != cudaSuccess) return B2R_ERR_CUDA;
  }
  return B2R_OK;
}

extern "C" int b2r_mg_reduce(b2r_mg_comm* c, const b2r_reduce_desc* desc, void* const* outs, const void* const* ins,
                             const int64_t* shard_rows, const b2r_stream_t* streams)
{
  if (c == nullptr || desc == nullptr || outs == nullptr || ins == nullptr || shard_rows == nullptr)
    return B2R_ERR_BAD_ARG;
  const int n           = int(c->devices.size());
  const bool per_column = desc->apply == B2R_ALONG_COLUMNS;
  ncclDataType_t dt     = ncclFloat32;
  ncclRedOp_t op        = ncclSum;
  if (per_column) {
    if (desc->inplace != 0) return B2R_ERR_UNSUPPORTED;
    if (!nccl_op(desc->reduce_op, &op) || !nccl_type(desc->out_dtype, &dt)) return B2R_ERR_UNSUPPORTED;
  }
  for (int d = 0; d < n; ++d)
    if (shard_rows[d] < 0) return B2R_ERR_BAD_ARG;
  DeviceGuard guard;
  // 1. every device reduces its shard (the column form without final_op; the start value of a sum
  //    enters once, on device 0)
  for (int d = 0; d < n; ++d) {
    if (cudaSetDevice(c->devices[d]) != cudaSuccess) return B2R_ERR_CUDA;
    b2r_reduce_desc local = *desc;
    local.n_rows          = shard_rows[d];
    if (per_column) {
      local.final_op     = B2R_FINAL_IDENTITY;
      local.final_scalar = 1.0;
      if (desc->reduce_op == B2R_REDUCE_ADD && d > 0) {
        local.init   = 0.0;
        local.init_i = 0;
      }
    }
    const int st = b2r_reduce(&local, outs[d], ins[d], nullptr, 0, reinterpret_cast<b2r_stream_t>(stream_of(c, streams, d)));
    if (st != B2R_OK) return st;
  }
  if (!per_column || desc->n_cols <= 0) return B2R_OK;
  // 2. all-reduce of the n_cols partials, in place, one NCCL group over the devices
  if (n > 1) {
    if (ncclGroupStart() != ncclSuccess) return B2R_ERR_CUDA;
    bool ok = true;
    for (int d = 0; d < n; ++d)
      ok = ok && ncclAllReduce(outs[d], outs[d], size_t(desc->n_cols), dt, op, c->comms[d], stream_of(c, streams, d)) ==
                   ncclSuccess;
    if (ncclGroupEnd() != ncclSuccess || !ok) return B2R_ERR_CUDA;
  }
  // 3. final_op on every device
  if (desc->final_op != B2R_FINAL_IDENTITY) {
    for (int d = 0; d < n; ++d) {
      if (cudaSetDevice(c->devices[d]) != cudaSuccess) return B2R_ERR_CUDA;
      const int st = b2r_apply_final(outs[d], desc->out_dtype, desc->n_cols, desc->final_op, desc->final_scalar,
                                     reinterpret_cast<b2r_stream_t>(stream_of(c, streams, d)));
      if (st != B2R_OK) return st;
    }
  }
  return B2R_OK;
}

extern "C" int b2r_mg_reduce_rows_by_key(b2r_mg_comm* c, void* const* sums, int64_t* const* counts, const void* const* A,
                                         int64_t lda, const void* const* keys, const void* const* weights,
                                         int32_t data_dtype, int32_t key_dtype, const int64_t* shard_rows, int64_t ncols,
                                         int64_t nkeys, int32_t reset, const b2r_stream_t* streams)
{
  if (c == nullptr || sums == nullptr || A == nullptr || keys == nullptr || shard_rows == nullptr)
    return B2R_ERR_BAD_ARG;
  const int n       = int(c->devices.size());
  ncclDataType_t dt = ncclFloat32;
  if (!nccl_type(data_dtype, &dt)) return B2R_ERR_UNSUPPORTED;
  if (counts != nullptr)
    for (int d = 0; d < n; ++d)
      if (counts[d] == nullptr) return B2R_ERR_BAD_ARG;
  DeviceGuard guard;
  for (int d = 0; d < n; ++d) {
    if (cudaSetDevice(c->devices[d]) != cudaSuccess) return B2R_ERR_CUDA;
    // accumulation onto earlier content: device 0 keeps its table, the others start from zero
    const int32_t local_reset = (reset != 0 || d > 0) ? 1 : 0;
    const int st = b2r_reduce_rows_by_key(sums[d], counts != nullptr ? counts[d] : nullptr, A[d], lda, keys[d],
                                          weights != nullptr ? weights[d] : nullptr, data_dtype, key_dtype,
                                          shard_rows[d], ncols, nkeys, local_reset, nullptr, 0,
                                          reinterpret_cast<b2r_stream_t>(stream_of(c, streams, d)));
    if (st != B2R_OK) return st;
  }
  if (n == 1 || ncols <= 0 || nkeys <= 0) return B2R_OK;
  if (ncclGroupStart() != ncclSuccess) return B2R_ERR_CUDA;
  bool ok = true;
  for (int d = 0; d < n; ++d) {
    cudaStream_t s = stream_of(c, streams, d);
    ok = ok && ncclAllReduce(sums[d], sums[d], size_t(nkeys) * size_t(ncols), dt, ncclSum, c->comms[d], s) == ncclSuccess;
    if (counts != nullptr)
      ok = ok && ncclAllReduce(counts[d], counts[d], size_t(nkeys), ncclInt64, ncclSum, c->comms[d], s) == ncclSuccess;
  }
  if (ncclGroupEnd() != ncclSuccess || !ok) return B2R_ERR_CUDA;
  return B2R_OK;
}
