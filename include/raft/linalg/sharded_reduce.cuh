// Row-sharded forms of raft::linalg::reduce and reduce_rows_by_key for the reference's single-process
// multi-GPU handle. The reference has no multi-GPU form of these primitives; what it has is the handle:
// raft::device_resources_snmg (core/device_resources_snmg.hpp:36-150) keeps one raft::resources per device
// in its MULTI_GPU resource (core/resource/multi_gpu.hpp:64-129) and one NCCL communicator per device in its
// NCCL_COMM resource (core/resource/nccl_comm.hpp:22-95). The overloads below take such a handle - any
// raft::resources that carries those two resources - and one view per device, in rank order:
//   * outputs per ROW: every device reduces its own rows, nothing is exchanged;
//   * outputs per COLUMN and keyed row sums: every device reduces its shard without final_op, the partials are
//     all-reduced over the handle's own communicators (ncclAllReduce, as comms_t::allreduce does in
//     comms/detail/std_comms.hpp:366-375), final_op runs on every device, every device holds the full result.
// Work for device d is enqueued on the stream of the handle's resources for rank d; the calls do not
// synchronise. They forward to the C ABI of libraft_b200_mg.so (include/raft_b200_mg.h), so the functors must
// be ones an enum can name (raft::identity_op, sq_op, abs_op, nz_op / add_op, min_op, max_op / identity_op,
// sqrt_op, abs_op, mul_const_op, div_const_op); link -lraft_b200_mg -lraft_b200 -lnccl.
#pragma once

#include "detail/b200_dispatch.cuh"

#include <raft/core/device_mdspan.hpp>
#include <raft/core/resource/cuda_stream.hpp>
#include <raft/core/resource/device_id.hpp>
#include <raft/core/resource/multi_gpu.hpp>
#include <raft/core/resource/nccl_comm.hpp>
#include <raft/core/resources.hpp>

#include <raft_b200_mg.h>

#include <vector>

namespace raft {
namespace linalg {
namespace b200 {

// The library's communicator object over the devices and NCCL communicators a handle already owns; it
// lives for one call (adopting costs one stream per device, which the call does not use).
class adopted_comm {
 public:
  explicit adopted_comm(raft::resources const& handle)
  {
    RAFT_EXPECTS(raft::resource::is_multi_gpu(handle), "the handle carries no multi-GPU resource");
    auto& world = raft::resource::get_multi_gpu_resource(handle);
    RAFT_EXPECTS(!world.empty(), "the handle's multi-GPU world is empty");
    auto& comms = raft::resource::get_nccl_comms(handle);
    std::vector<int> devices(world.size());
    std::vector<void*> raw(world.size());
    streams_.resize(world.size());
    for (size_t d = 0; d < world.size(); ++d) {
      devices[d]  = raft::resource::get_device_id(world[d]);
      raw[d]      = static_cast<void*>(comms[d]);
      streams_[d] = reinterpret_cast<b2r_stream_t>(static_cast<cudaStream_t>(raft::resource::get_cuda_stream(world[d])));
    }
    check(b2r_mg_comm_adopt(&comm_, devices.data(), int(devices.size()), raw.data()), "b2r_mg_comm_adopt");
  }
  ~adopted_comm() { b2r_mg_comm_destroy(comm_); }
  adopted_comm(const adopted_comm&)            = delete;
  adopted_comm& operator=(const adopted_comm&) = delete;
  b2r_mg_comm* get() const { return comm_; }
  const b2r_stream_t* streams() const { return streams_.data(); }
  size_t size() const { return streams_.size(); }

 private:
  b2r_mg_comm* comm_ = nullptr;
  std::vector<b2r_stream_t> streams_;
};

}  // namespace b200

/**
 * Row-sharded reduce: shards[d] is the [rows_d x n_cols] block of rows that device d holds (row-major), in
 * rank order of the handle. apply == ALONG_ROWS: dots[d] receives the rows_d outputs of that block.
 * apply == ALONG_COLUMNS: every dots[d] receives all n_cols outputs of the WHOLE matrix.
 */
template <typename InType,
          typename OutType,
          typename IdxType,
          typename MainLambda   = raft::identity_op,
          typename ReduceLambda = raft::add_op,
          typename FinalLambda  = raft::identity_op>
void reduce(raft::resources const& snmg_handle,
            std::vector<raft::device_matrix_view<const InType, IdxType, raft::row_major>> const& shards,
            std::vector<raft::device_vector_view<OutType, IdxType>> const& dots,
            OutType init,
            raft::Apply apply,
            MainLambda main_op     = raft::identity_op(),
            ReduceLambda reduce_op = raft::add_op(),
            FinalLambda final_op   = raft::identity_op())
{
  constexpr int mainE = b200::main_enum<MainLambda>::value;
  constexpr int redE  = b200::reduce_enum<ReduceLambda>::value;
  constexpr int finE  = b200::final_enum<FinalLambda>::value;
  static_assert(mainE >= 0 && redE >= 0 && finE >= 0 && b200::combo_built<mainE, redE>::value &&
                  b200::abi_pair<InType, OutType>::value,
                "the sharded reduce takes the named raft functors and the type pairs of the C ABI");
  (void)main_op;
  (void)reduce_op;
  b200::adopted_comm comm(snmg_handle);
  RAFT_EXPECTS(shards.size() == comm.size() && dots.size() == comm.size(), "one shard and one output per device");
  const IdxType n_cols = shards[0].extent(1);
  std::vector<const void*> ins(comm.size());
  std::vector<void*> outs(comm.size());
  std::vector<int64_t> rows(comm.size());
  for (size_t d = 0; d < comm.size(); ++d) {
    RAFT_EXPECTS(shards[d].extent(1) == n_cols, "All shards must have the same number of columns");
    RAFT_EXPECTS(dots[d].extent(0) == (apply == raft::Apply::ALONG_ROWS ? shards[d].extent(0) : n_cols),
                 apply == raft::Apply::ALONG_ROWS ? "Output should be equal to number of rows in Input"
                                                  : "Output should be equal to number of columns in Input");
    ins[d]  = shards[d].data_handle();
    outs[d] = dots[d].data_handle();
    rows[d] = int64_t(shards[d].extent(0));
  }
  b2r_reduce_desc d = {};
  d.in_dtype        = b200::dtype_of<InType>::value;
  d.out_dtype       = b200::dtype_of<OutType>::value;
  d.layout          = B2R_ROW_MAJOR;
  d.apply           = apply == raft::Apply::ALONG_ROWS ? B2R_ALONG_ROWS : B2R_ALONG_COLUMNS;
  d.n_cols          = int64_t(n_cols);
  d.main_op         = mainE;
  d.reduce_op       = redE;
  d.final_op        = finE;
  d.init            = double(init);
  d.init_i          = std::is_integral<OutType>::value ? static_cast<long long>(init) : 0;
  d.final_scalar    = b200::final_enum<FinalLambda>::scalar(final_op);
  b200::check(b2r_mg_reduce(comm.get(), &d, outs.data(), ins.data(), rows.data(), comm.streams()),
              "raft::linalg::reduce (sharded)");
}

/**
 * Row-sharded reduce_rows_by_key: d_A[d] is the [rows_d x ncols] block of device d (row-major), d_keys[d] its
 * rows_d keys; every d_sums[d] ([n_unique_keys x ncols]) receives the sums over ALL shards.
 */
template <typename ElementType, typename KeyType, typename IndexType>
void reduce_rows_by_key(raft::resources const& snmg_handle,
                        std::vector<raft::device_matrix_view<const ElementType, IndexType, raft::row_major>> const& d_A,
                        std::vector<raft::device_vector_view<const KeyType, IndexType>> const& d_keys,
                        std::vector<raft::device_matrix_view<ElementType, IndexType, raft::row_major>> const& d_sums,
                        IndexType n_unique_keys,
                        bool reset_sums = true)
{
  static_assert(b200::dtype_of<ElementType>::value == B2R_F32 || b200::dtype_of<ElementType>::value == B2R_F64,
                "fp32 or fp64 data");
  static_assert(b200::dtype_of<KeyType>::value == B2R_I32 || b200::dtype_of<KeyType>::value == B2R_U32 ||
                  b200::dtype_of<KeyType>::value == B2R_I64,
                "int32, uint32 or int64 keys");
  b200::adopted_comm comm(snmg_handle);
  RAFT_EXPECTS(d_A.size() == comm.size() && d_keys.size() == comm.size() && d_sums.size() == comm.size(),
               "one shard, one key vector and one output per device");
  const IndexType ncols = d_A[0].extent(1);
  std::vector<const void*> A(comm.size()), keys(comm.size());
  std::vector<void*> sums(comm.size());
  std::vector<int64_t> rows(comm.size());
  for (size_t d = 0; d < comm.size(); ++d) {
    RAFT_EXPECTS(d_A[d].extent(1) == ncols, "All shards must have the same number of columns");
    RAFT_EXPECTS(d_keys[d].extent(0) == d_A[d].extent(0), "Keys is not of size nrows");
    RAFT_EXPECTS(d_sums[d].extent(0) == n_unique_keys && d_sums[d].extent(1) == ncols,
                 "Output is not of size ncols * n_unique_keys");
    A[d]    = d_A[d].data_handle();
    keys[d] = d_keys[d].data_handle();
    sums[d] = d_sums[d].data_handle();
    rows[d] = int64_t(d_A[d].extent(0));
  }
  b200::check(b2r_mg_reduce_rows_by_key(comm.get(), sums.data(), nullptr, A.data(), int64_t(ncols), keys.data(), nullptr,
                                        b200::dtype_of<ElementType>::value, b200::dtype_of<KeyType>::value, rows.data(),
                                        int64_t(ncols), int64_t(n_unique_keys), reset_sums ? 1 : 0, comm.streams()),
              "raft::linalg::reduce_rows_by_key (sharded)");
}

}  // namespace linalg
}  // namespace raft
