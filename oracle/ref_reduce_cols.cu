// oracle/_ref: the reference's raft::linalg::reduce along the strided axis.
#include "ref_common.cuh"

using namespace refwrap;

template <bool RowMajor, bool AlongRows, typename T>
static int dispatch(const b2r_reduce_desc& d, void* out, const void* in, cudaStream_t s)
{
  const T init = T(d.init);
  const int key = d.main_op * 100 + d.reduce_op * 10 + d.final_op;
  switch (key) {
    case 0: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::identity_op{}, raft::add_op{}, raft::identity_op{}, s);
    case 2: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::identity_op{}, raft::add_op{}, raft::mul_const_op<T>(T(d.final_scalar)), s);
    case 3: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::identity_op{}, raft::add_op{}, raft::div_const_op<T>(T(d.final_scalar)), s);
    case 100: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::sq_op{}, raft::add_op{}, raft::identity_op{}, s);
    case 101: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::sq_op{}, raft::add_op{}, raft::sqrt_op{}, s);
    case 20: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::identity_op{}, raft::max_op{}, raft::identity_op{}, s);
    case 220: return run<RowMajor, AlongRows, T, T>(d, out, in, init, raft::abs_op{}, raft::max_op{}, raft::identity_op{}, s);
    default: return B2R_ERR_UNSUPPORTED;
  }
}

// strided-axis reductions: (row-major, along columns) and (column-major, along rows)
REF_EXPORT int ref_reduce_strided(const b2r_reduce_desc* d, void* out, const void* in, cudaStream_t s)
{
  const bool rm = d->layout == B2R_ROW_MAJOR;
  if (d->in_dtype == B2R_F32 && d->out_dtype == B2R_F32)
    return rm ? dispatch<true, false, float>(*d, out, in, s) : dispatch<false, true, float>(*d, out, in, s);
  if (d->in_dtype == B2R_F64 && d->out_dtype == B2R_F64)
    return rm ? dispatch<true, false, double>(*d, out, in, s) : dispatch<false, true, double>(*d, out, in, s);
  return B2R_ERR_UNSUPPORTED;
}
