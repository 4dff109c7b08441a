/*
 * raft_b200 - C ABI of the B200 (sm_100a) dense-reduction kernels.
 *
 * This is the whole boundary between host code and the CUDA kernels: plain pointers, sizes,
 * enums and a stream. The drop-in C++ headers under include/raft/linalg/ forward to these
 * entry points when the caller's functors are ones an enum can name, and any other language
 * can bind them directly (see the ctypes binding in raft_b200/_lib.py).
 *
 * The reference (RAFT 26.10) has no ABI for this path - its reductions are header-only
 * function templates - so each entry point below names the reference template it stands for.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless stated otherwise; the caller owns all buffers;
 *  - every call is asynchronous on `stream` and never synchronises;
 *  - the return value is a b2r_status; B2R_ERR_CUDA means a CUDA runtime call failed and
 *    b2r_last_cuda_error() returns its cudaError_t (per host thread);
 *  - `workspace` may be NULL: kernels that need scratch memory then take it from a
 *    library-owned stream-ordered pool (allocation and free ordered on `stream`). A caller that
 *    wants no allocation inside the call passes b2r_*_workspace_bytes() bytes of device memory.
 */
#ifndef RAFT_B200_H
#define RAFT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B2R_API
#else
#define B2R_API __attribute__((visibility("default")))
#endif

/* Same underlying type as cudaStream_t, without requiring the CUDA headers. */
typedef struct CUstream_st* b2r_stream_t;

typedef enum {
  B2R_OK              = 0,
  B2R_ERR_BAD_ARG     = 1, /* null pointer, negative size, inconsistent descriptor           */
  B2R_ERR_UNSUPPORTED = 2, /* a dtype / operator combination the library was not built for   */
  B2R_ERR_CUDA        = 3, /* a CUDA runtime call failed, see b2r_last_cuda_error()          */
  B2R_ERR_TOO_LARGE   = 4, /* a size beyond a stated limit of the entry point                */
  B2R_ERR_TIMEOUT     = 5  /* a bounded wait inside a kernel ran out (reported by the status queries) */
} b2r_status;

typedef enum {
  B2R_F32 = 0,
  B2R_F64 = 1,
  B2R_F16 = 2,
  B2R_I32 = 3,
  B2R_I64 = 4,
  B2R_I16 = 5,
  B2R_U32 = 6,
  /* {int32 key; V value} pairs, laid out like raft::KeyValuePair<int, V> (core/kvp.hpp:20-27) */
  B2R_KVP_I32_F32 = 16,
  B2R_KVP_I32_F64 = 17,
  B2R_KVP_I32_I16 = 18,
  B2R_KVP_I32_I32 = 19
} b2r_dtype;

typedef enum { B2R_ROW_MAJOR = 0, B2R_COL_MAJOR = 1 } b2r_layout;

/* raft::Apply (core/types.hpp:16): ALONG_ROWS gives one output per row. */
typedef enum { B2R_ALONG_ROWS = 0, B2R_ALONG_COLUMNS = 1 } b2r_apply;

/* main_op(x, index along the reduced axis) - core/operators.hpp:27-107 */
typedef enum {
  B2R_MAIN_IDENTITY = 0, /* raft::identity_op */
  B2R_MAIN_SQ       = 1, /* raft::sq_op       */
  B2R_MAIN_ABS      = 2, /* raft::abs_op      */
  B2R_MAIN_NZ       = 3, /* raft::nz_op       */
  B2R_MAIN_TO_KVP   = 4  /* x, j -> {j, x}; required with ARGMIN / ARGMAX */
} b2r_main_op;

/* reduce_op - core/operators.hpp:109-199 */
typedef enum {
  B2R_REDUCE_ADD    = 0, /* raft::add_op, compensated summation */
  B2R_REDUCE_MIN    = 1, /* raft::min_op */
  B2R_REDUCE_MAX    = 2, /* raft::max_op */
  B2R_REDUCE_ARGMIN = 3, /* raft::argmin_op: smaller value wins, ties -> lower key */
  B2R_REDUCE_ARGMAX = 4  /* raft::argmax_op: larger value wins,  ties -> lower key */
} b2r_reduce_op;

/* final_op - core/operators.hpp:69-75, 300-310 */
typedef enum {
  B2R_FINAL_IDENTITY  = 0,
  B2R_FINAL_SQRT      = 1, /* raft::sqrt_op                      */
  B2R_FINAL_MUL_CONST = 2, /* raft::mul_const_op(final_scalar)   */
  B2R_FINAL_DIV_CONST = 3, /* raft::div_const_op(final_scalar)   */
  B2R_FINAL_ABS       = 4  /* raft::abs_op                       */
} b2r_final_op;

/* raft::linalg::NormType (linalg/norm_types.hpp:13-23) */
typedef enum { B2R_NORM_L0 = 0, B2R_NORM_L1 = 1, B2R_NORM_L2 = 2, B2R_NORM_LINF = 3 } b2r_norm_type;

typedef struct {
  int32_t in_dtype;   /* b2r_dtype of the matrix elements                                   */
  int32_t out_dtype;  /* b2r_dtype of the outputs (= accumulator type, as in the reference) */
  int32_t layout;     /* b2r_layout of the matrix; it must be contiguous                    */
  int32_t apply;      /* b2r_apply                                                          */
  int64_t n_rows;     /* matrix extent 0                                                    */
  int64_t n_cols;     /* matrix extent 1                                                    */
  int32_t main_op;    /* b2r_main_op                                                        */
  int32_t reduce_op;  /* b2r_reduce_op                                                      */
  int32_t final_op;   /* b2r_final_op                                                       */
  int32_t inplace;    /* non-zero: out = final(reduce(out_old, acc))                        */
  double init;        /* initial value (floating outputs; value part of a KVP)              */
  int64_t init_i;     /* initial value (integer outputs; integer value part of a KVP)       */
  int64_t init_key;   /* key part of a KVP initial value                                    */
  double final_scalar;/* operand of MUL_CONST / DIV_CONST                                   */
} b2r_reduce_desc;

/*
 * raft::linalg::reduce - raw-pointer form linalg/reduce.cuh:55-76, mdspan form :140-180,
 * dispatch linalg/detail/reduce.cuh:25-49 - and with it coalesced_reduction
 * (linalg/coalesced_reduction.cuh:48-67, 104-149) and strided_reduction
 * (linalg/strided_reduction.cuh:51-78, 115-160):
 *     out[k] = final_op(reduce_op over the reduced axis of main_op(in[..], index))
 * `init` must be the identity of reduce_op (for ADD it is added exactly once). As in the
 * reference, ARGMIN / ARGMAX outputs are only available along the contiguous axis
 * (linalg/strided_reduction.cuh:70-77).
 */
B2R_API int b2r_reduce(const b2r_reduce_desc* desc,
                       void* out,
                       const void* in,
                       void* workspace,
                       size_t workspace_bytes,
                       b2r_stream_t stream);

/* Scratch bytes b2r_reduce would allocate for this descriptor and input pointer (0: none). */
B2R_API size_t b2r_reduce_workspace_bytes(const b2r_reduce_desc* desc, const void* in);

/*
 * raft::linalg::norm / rowNorm / colNorm - linalg/norm.cuh:45-59, 76-90, 112-148,
 * linalg/detail/norm.cuh:17-61. L1 = (abs, add), L2 = (sq, add; no root unless final_op is
 * SQRT), Linf = (abs, max); init 0, never in place. B2R_NORM_L0 returns
 * B2R_ERR_UNSUPPORTED, as the reference throws for it.
 */
B2R_API int b2r_norm(int32_t norm_type,
                     int32_t apply,
                     int32_t layout,
                     int32_t in_dtype,
                     int32_t out_dtype,
                     int64_t n_rows,
                     int64_t n_cols,
                     int32_t final_op,
                     double final_scalar,
                     void* out,
                     const void* in,
                     void* workspace,
                     size_t workspace_bytes,
                     b2r_stream_t stream);

/*
 * raft::linalg::reduce_rows_by_key - linalg/reduce_rows_by_key.cuh:52-71 (weighted),
 * :92-116 (unweighted), impl linalg/detail/reduce_rows_by_key.cuh:353-385:
 *     sums[keys[i]][0..ncols) += weights[i] * A[i][0..ncols)      A row-major, row stride lda
 * `weights` may be NULL (unit weights). `reset` non-zero overwrites sums, zero accumulates
 * into them. Keys must lie in [0, nkeys) (unchecked, as in the reference).
 * data_dtype: B2R_F32 or B2R_F64 (sums and weights have the same type); key_dtype: B2R_I32,
 * B2R_U32 or B2R_I64.
 * `counts` (may be NULL) is an extension with no counterpart in the reference: int64 number of
 * rows per key, overwritten or accumulated like sums.
 * The reference's char scratch `d_keys_char` is not needed and has no parameter here.
 */
B2R_API int b2r_reduce_rows_by_key(void* sums,
                                   int64_t* counts,
                                   const void* A,
                                   int64_t lda,
                                   const void* keys,
                                   const void* weights,
                                   int32_t data_dtype,
                                   int32_t key_dtype,
                                   int64_t nrows,
                                   int64_t ncols,
                                   int64_t nkeys,
                                   int32_t reset,
                                   void* workspace,
                                   size_t workspace_bytes,
                                   b2r_stream_t stream);

B2R_API size_t b2r_reduce_rows_by_key_workspace_bytes(
  const void* A, int64_t lda, int32_t data_dtype, int64_t nrows, int64_t ncols, int64_t nkeys);

/*
 * raft::linalg::reduce_cols_by_key - linalg/reduce_cols_by_key.cuh:39-50, 76-102, impl
 * linalg/detail/reduce_cols_by_key.cuh:89-138:
 *     out[r][keys[c]] += data[r][c]        data row-major [nrows x ncols], out [nrows x nkeys]
 * dtype: B2R_F32 or B2R_F64; key_dtype: B2R_I32, B2R_U32 or B2R_I64. The reference is stateless and the
 * caller owns every buffer (docs/source/developer_guide.md:77-81): `workspace` of
 * b2r_reduce_cols_by_key_workspace_bytes() bytes keeps the call allocation-free (the sorted column
 * offsets and per-split tables of the large-input algorithm; 0 for small inputs).
 */
B2R_API int b2r_reduce_cols_by_key(void* out,
                                   const void* data,
                                   const void* keys,
                                   int32_t dtype,
                                   int32_t key_dtype,
                                   int64_t nrows,
                                   int64_t ncols,
                                   int64_t nkeys,
                                   int32_t reset,
                                   void* workspace,
                                   size_t workspace_bytes,
                                   b2r_stream_t stream);

B2R_API size_t b2r_reduce_cols_by_key_workspace_bytes(
  const void* data, int32_t dtype, int64_t nrows, int64_t ncols, int64_t nkeys);

/*
 * raft::linalg::row_normalize<norm_type> - linalg/normalize.cuh:88-107, kernels
 * linalg/detail/normalize.cuh:26-197: every row of a row-major [n_rows x n_cols] matrix is divided
 * by its L1 / L2 (with root) / Linf norm; a row whose norm is <= eps is NOT written (out keeps its
 * previous content there), as in the reference. dtype: B2R_F32 or B2R_F64 (input and output).
 * `out` may be `in`. One pass: every element is read once and written once.
 */
B2R_API int b2r_row_normalize(void* out,
                              const void* in,
                              int32_t dtype,
                              int64_t n_rows,
                              int64_t n_cols,
                              int32_t norm_type,
                              double eps,
                              b2r_stream_t stream);

/*
 * raft::matrix::argmin / argmax - matrix/argmin.cuh:27-39, matrix/argmax.cuh:27-39, kernel
 * matrix/detail/math.cuh:291-352: out[r] = column index of the smallest / largest element of row r
 * of a row-major [n_rows x n_cols] matrix; on equal values the lowest index wins (cub::ArgMin /
 * cub::ArgMax). in_dtype: B2R_F32 or B2R_F64; out_dtype: B2R_I32 or B2R_I64.
 */
B2R_API int b2r_matrix_argmin(void* out,
                              int32_t out_dtype,
                              const void* in,
                              int32_t in_dtype,
                              int64_t n_rows,
                              int64_t n_cols,
                              b2r_stream_t stream);

B2R_API int b2r_matrix_argmax(void* out,
                              int32_t out_dtype,
                              const void* in,
                              int32_t in_dtype,
                              int64_t n_rows,
                              int64_t n_cols,
                              b2r_stream_t stream);

/*
 * Column sums of a row-major fp32 matrix without any allocation:
 *     out[j] = final_op(sum over i of in[i][j]),   in [n_rows x n_cols], out [n_cols]
 * This entry point has no counterpart in the reference. It is b2r_reduce's column path
 * (identity main_op, add, init 0, not in place) for callers that may not allocate device
 * memory and have no workspace to pass - for example a plugin called with only its input,
 * its output and a stream, or a service that forbids allocator calls once it is serving,
 * because cudaMalloc / cudaFree take driver-wide locks. The scratch the kernels need lives in
 * a 1 MiB array inside the library image (present on every GPU that loads the library, for
 * the life of the process); the call uses no cudaMalloc, cudaFree, cudaMallocAsync or any
 * other allocating routine.
 *  - The call needs one fp64 partial row (n_cols x 8 bytes) per row range of the launch, plus a
 *    status word per CTA for the TMA-staged kernel. The launch shape is planned UNDER the array's
 *    size: where the preferred shape would need more (148 CTAs x n_cols x 8 bytes for n_cols near
 *    1024; two row ranges of more than 65536 columns) the call uses fewer CTAs or row ranges, down
 *    to a single row range, which needs no scratch at all - so every n_rows x n_cols is accepted
 *    on today's GPUs, a few of them on fewer CTAs than b2r_reduce would use (its result then
 *    differs from b2r_reduce's in the last bits: another summation order). Should a plan ever not
 *    fit, the call returns B2R_ERR_TOO_LARGE and launches nothing.
 *    b2r_column_sum_f32_noalloc_max_scratch() returns the size of the array.
 *  - The first call on each device looks up the array's device address; make that first call
 *    before any stream capture begins on that device.
 *  - All calls on a device share the one array. Its contents are fully rewritten by each call
 *    before they are read, so nothing has to be cleared, but two calls that can run at the same
 *    time on one device (different streams, or different host threads) race on it: serialise
 *    them.
 */
B2R_API int b2r_column_sum_f32_noalloc(float* out,
                                       const float* in,
                                       int64_t n_rows,
                                       int64_t n_cols,
                                       int32_t final_op,
                                       double final_scalar,
                                       b2r_stream_t stream);

B2R_API size_t b2r_column_sum_f32_noalloc_max_scratch(void);

/*
 * Applies a final_op to a vector in place: v[i] = final_op(v[i]). Used by the multi-GPU
 * host layer, which all-reduces raw per-GPU partials and applies final_op afterwards; in the
 * reference the same step is the trailing unaryOp of linalg/detail/strided_reduction.cuh:194-195.
 */
B2R_API int b2r_apply_final(void* v,
                            int32_t dtype,
                            int64_t n,
                            int32_t final_op,
                            double final_scalar,
                            b2r_stream_t stream);

/*
 * Synthetic workload generator (counter based: element i of a buffer depends only on
 * (seed, i + first_index), so any shard of a matrix can be generated in place and a host
 * implementation of the same hash reproduces it bit for bit). Has no counterpart in the
 * reference, whose tests use raft::random. `kind`:
 *   0 uniform in [lo, hi)            (f32 / f64)
 *   1 approximately standard normal  (f32 / f64; sum of eight 16-bit uniforms, unit variance)
 *   2 integer-valued uniform in {lo .. hi-1}   (f32 / f64 / i32 / i16 / u32 / i64)
 */
B2R_API int b2r_synth_fill(void* dst,
                           int32_t dtype,
                           int64_t n,
                           int64_t first_index,
                           uint64_t seed,
                           int32_t kind,
                           double lo,
                           double hi,
                           b2r_stream_t stream);

/*
 * All-reduce (sum) of small per-GPU partials over peer memory, for the row-sharded column and by-key
 * reductions: ONE kernel per GPU pushes its partial into every peer's exchange area with plain stores
 * over NVLink, raises a flag, waits (bounded) for the peers' flags in its own memory, sums the slots in
 * rank order and applies the deferred scale - in place of one library collective per tensor plus a
 * final_op launch. The collective it stands for in the reference is comms_t::allreduce
 * (cpp/include/raft/comms/detail/std_comms.hpp:366-375); the reference has no kernel of this kind.
 *
 *  b2r_peer_area_create      allocates this rank's exchange area on the current device (cudaMalloc, a
 *                            set-up call): 2 x world slots of `max_payload_bytes` plus flags. HOST pointer out.
 *  b2r_peer_area_ipc_handle  writes the 64-byte CUDA IPC handle of the area (to send to the other processes).
 *  b2r_peer_area_open        maps the area of `peer_rank` (another process on this node) from its handle.
 *  b2r_peer_area_link        the same for an area of another device of THIS process (enables peer access).
 *  b2r_peer_allreduce_sum    sums[0..n_f32) and counts[0..n_i64) (device, either may be empty) become the
 *                            sums over all ranks, fp32 sums multiplied by `scale`; asynchronous on `stream`.
 *                            Every rank must make the same sequence of calls with the same sizes. A payload
 *                            above the area's slot size returns B2R_ERR_TOO_LARGE.
 *  b2r_peer_area_status      (synchronising, after the caller's own sync) B2R_ERR_TIMEOUT in *status_out if a
 *                            wait of an earlier call ran out - that call left its outputs unfinished -, else
 *                            B2R_OK; `clear` resets it. The limit is 2 s unless b2r_peer_area_set_wait_limit_ms.
 */
B2R_API int b2r_peer_area_create(int32_t world, int32_t rank, size_t max_payload_bytes, void** area_out);
B2R_API int b2r_peer_area_ipc_handle(void* area, void* handle_out_64_bytes);
B2R_API int b2r_peer_area_open(void* area, int32_t peer_rank, const void* handle_64_bytes);
B2R_API int b2r_peer_area_link(void* area, int32_t peer_rank, void* peer_area_same_process);
B2R_API int b2r_peer_area_set_wait_limit_ms(void* area, uint32_t ms);
B2R_API int b2r_peer_allreduce_sum(void* area,
                                   float* sums,
                                   int64_t n_f32,
                                   long long* counts,
                                   int64_t n_i64,
                                   double scale,
                                   b2r_stream_t stream);
B2R_API int b2r_peer_area_status(void* area, int32_t* status_out, int32_t clear);
B2R_API int b2r_peer_area_destroy(void* area);

/*
 * Measurement aids (no counterpart in the reference, whose benchmarks report times without a
 * floor): an empty kernel - what a pair of events around any launch costs - and a kernel that
 * only reads `bytes` bytes at `data` (16-byte aligned) once, every SM streaming, which is the
 * fastest any kernel of this library could consume them. `sink` may be NULL.
 */
B2R_API int b2r_probe_empty_launch(b2r_stream_t stream);
B2R_API int b2r_probe_stream_read(const void* data, size_t bytes, float* sink, b2r_stream_t stream);

/*
 * Scratch the library allocates for itself (calls made with workspace == NULL) comes from a
 * stream-ordered memory pool the library owns, one per device, which keeps freed blocks for
 * re-use. This call gives the cached blocks of the current device back to the driver. No
 * counterpart in the reference (rmm plays this role there).
 */
B2R_API int b2r_trim_scratch_pool(void);

/*
 * Launch-shape knobs (environment variables B2R_*, listed in raft_b200/detail/launch.cuh) are read
 * once, at the first call into the library. This call reads them again - for a benchmark that
 * sweeps them within one process. It must not run concurrently with other calls.
 */
B2R_API int b2r_reload_tuning(void);

/*
 * Kernels of this library that stage tiles through shared memory wait on hardware barriers; every such
 * wait is bounded (a second unless changed here; B2R_WAIT_LIMIT_MS sets the default of a process). A CTA
 * whose wait runs out stops, lets its copies in flight land, fills the floating-point outputs it did not
 * finish with NaN and sets a status word on its device; the call itself has long returned (it is
 * asynchronous, as launch errors are in the reference: util/kernel_launch.hpp:41-42), so the outcome is
 * read afterwards:
 *  b2r_last_kernel_status   after the caller's own synchronisation: *status_out = B2R_ERR_TIMEOUT if a wait
 *                           of any earlier call on the CURRENT device ran out, else B2R_OK (the reference's
 *                           comms report SUCCESS / ERROR / ABORT the same way, core/comms.hpp:31-35);
 *                           `clear` resets the word. Synchronising itself (a small device-to-host copy).
 *  b2r_set_wait_limit_ms    the bound of every wait, for calls made from now on; 0 = back to the default.
 */
B2R_API int b2r_last_kernel_status(int32_t* status_out, int32_t clear);
B2R_API int b2r_set_wait_limit_ms(uint32_t ms);

B2R_API const char* b2r_status_string(int status);
B2R_API int b2r_last_cuda_error(void);
B2R_API const char* b2r_version(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* RAFT_B200_H */
